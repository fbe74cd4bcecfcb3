"""The Python entry point: prompts in, generated tokens out.

`LLM` owns an `Engine` (model, cache, step function), the C++ `Scheduler` and a
`Sampler`, and drives them the way the reference's runner drives its model
(rust/engine/src/runner/model_runner.rs:698-897): plan a step, run it, accept
the sampled tokens, finish and free.  Token ids go in and come out; text is
handled at the command line only.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Optional, Sequence, Union

from ..cache import manager as cache_mod
from ..config.base import read_generation_eos
from ..sampling import Sampler, SamplingConfig
from .decode_graph import DecodeGraphs
from .engine import Engine, Entry


@dataclasses.dataclass
class GenerationResult:
    request_id: int
    prompt_tokens: list[int]
    tokens: list[int]
    finish_reason: str          # "length" | "eos" | "capacity" | "invalid" | "cancelled"
    message: str = ""
    preemptions: int = 0
    ttft: Optional[float] = None


class LLM:
    def __init__(self, model_dir: str, dtype: str = "bf16", *, max_batch_tokens: int = 512,
                 kv_tokens: Optional[int] = None, page_size: int = 16, max_requests: int = 64,
                 max_seq_len: Optional[int] = None, reserve_future: bool = True, cuda_graph: bool = False,
                 lookahead: bool = True, device: str = "cuda:0"):
        self.engine = Engine(model_dir, dtype, max_tokens=kv_tokens, page_size=page_size, max_requests=max_requests,
                             max_batch_tokens=max_batch_tokens, max_seq_len=max_seq_len, device=device)
        rt = cache_mod.runtime()
        self.scheduler = rt.Scheduler(self.engine.cache, max_batch_tokens, self.engine.max_seq_len, max_requests,
                                      reserve_future)
        self.sampler = Sampler(self.engine.device)
        # generation_config.json, where the folder has one, names the ids that end a sequence
        # (rust/engine/src/runner/model/qwen2/engine.rs:403-407); else the model configuration does.
        file_eos = read_generation_eos(model_dir) if isinstance(model_dir, str) else None
        self.model_eos = list(file_eos if file_eos is not None else self.engine.model.blueprint.eos_token_ids)
        # Models with fixed-size per-request state step eagerly (see DecodeGraphs).
        self.cuda_graph = bool(cuda_graph) and not self.engine.stateful
        self.graphs = DecodeGraphs(self.engine) if self.cuda_graph else None
        # With graphs: while a decode step runs, the next one is planned and launched before the first
        # one's tokens have reached the host (the device feeds the sampled ids forward), so the host's
        # work between steps no longer idles the GPU.
        self.lookahead = bool(lookahead) and self.cuda_graph
        if self.cuda_graph:
            self.engine.enable_step_graphs()      # prompt portions of a repeating shape as well
        # (time the step's tokens reached the host, tokens, decode?, tokens its requests hold after it)
        self.step_log: list[tuple[float, int, bool, int]] = []
        self._next_id = 0
        self.steps = 0
        self.trace = None      # optional callable taking one dict per step (the CLI's --trace-steps)

    # ------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling: Union[None, SamplingConfig, Sequence[SamplingConfig]] = None) -> list[GenerationResult]:
        """Runs all prompts to their end with continuous batching; results in prompt order."""
        if sampling is None:
            sampling = SamplingConfig()
        configs = list(sampling) if isinstance(sampling, (list, tuple)) else [sampling] * len(prompts)
        if len(configs) != len(prompts):
            raise ValueError("one SamplingConfig per prompt, or one for all")
        ids = []
        by_id = {}
        vocab = self.engine.vocab
        for prompt, cfg in zip(prompts, configs):
            cfg.validate()
            prompt = [int(t) for t in prompt]
            rid = self._next_id
            self._next_id += 1
            ids.append(rid)
            by_id[rid] = {"cfg": cfg, "prompt": prompt, "t0": time.perf_counter(), "ttft": None}
            if any(t < 0 or t >= vocab for t in prompt):
                by_id[rid]["result"] = GenerationResult(rid, prompt, [], "invalid", f"token id outside [0, {vocab})")
                continue
            self.scheduler.add(rid, prompt, cfg.max_new_tokens, cfg.eos_ids(self.model_eos), cfg.ignore_eos)
        self._run(by_id)
        return [by_id[r]["result"] for r in ids]

    def _collect(self, by_id) -> None:
        for f in self.scheduler.take_finished():
            rec = by_id[f.id]
            rec["result"] = GenerationResult(f.id, rec["prompt"], list(f.generated), f.reason.name, f.message,
                                             f.preemptions, rec["ttft"])

    def _run(self, by_id) -> None:
        sched = self.scheduler
        last_decode_ids = None     # requests of the previous step, if it was a decode step from a graph
        while True:
            plan = sched.plan()
            self._collect(by_id)
            if not plan:
                if sched.idle:
                    return
                raise RuntimeError("the scheduler has requests left but plans no step")
            pure_decode = all(e.n == 1 and e.sample for e in plan)
            if self.graphs is not None and pure_decode:
                last_decode_ids = self._decode_run(by_id, plan, last_decode_ids)
                continue
            last_decode_ids = None
            rows = [e for e in plan if e.sample]
            sampled = []
            try:
                cfgs = [by_id[e.id]["cfg"] for e in rows]
                temps = [c.effective_temperature() for c in cfgs]
                seeds = [c.seed for c in cfgs]
                entries = [Entry(e.id, sched.portion(e.id, e.start, e.n), [e.n - 1] if e.sample else [])
                           for e in plan]
                positions = [e.start + e.n for e in rows]
                if rows and not self.cuda_graph:
                    # the head picks the tokens itself: no logits are written
                    tokens = self.engine.step(entries, reserved=True, pick=self.sampler.device_args(temps, seeds, positions))
                    sampled = self.sampler.check(tokens.cpu().tolist(), self.engine.vocab)
                else:
                    logits = self.engine.step(entries, reserved=True)
                    if logits is not None:
                        sampled = self.sampler.pick(logits, temps, seeds, positions)
            except Exception:
                sched.abandon(plan)
                raise
            self._step_done(by_id, plan, sampled, False)

    def _decode_run(self, by_id, plan, last_decode_ids):
        """Decode steps from CUDA graphs, every request one token a step, for as long as the
        scheduler can look ahead: step n + 1 is planned and launched before the tokens of step n are
        read.  Returns the requests of the last step launched."""
        sched, graphs = self.scheduler, self.graphs
        ids = [e.id for e in plan]
        try:
            tokens = [sched.portion(e.id, e.start, 1)[0] for e in plan]
            if ids == last_decode_ids:
                # the same requests as in the step before: temperatures and seeds are on the device
                ticket = graphs.step(ids, tokens, None, None, reserved=True, keep=True)
            else:
                cfgs = [by_id[i]["cfg"] for i in ids]
                ticket = graphs.step(ids, tokens, [c.effective_temperature() for c in cfgs],
                                     [c.seed for c in cfgs], reserved=True, keep=True)
        except Exception:
            sched.abandon(plan)
            raise
        while True:
            ahead = sched.plan_ahead(plan) if self.lookahead else []
            next_ticket = None
            try:
                if ahead:
                    next_ticket = graphs.step(ids, None, None, None, reserved=True, keep=True)
                sampled = self.sampler.check(graphs.read(ticket), self.engine.vocab)
            except Exception:
                sched.abandon(ahead if ahead else plan)
                raise
            self._step_done(by_id, plan, sampled, True)
            if not ahead:
                return ids
            plan, ticket = ahead, next_ticket

    def _step_done(self, by_id, plan, sampled, pure_decode) -> None:
        now = time.perf_counter()
        self.step_log.append((now, sum(e.n for e in plan), pure_decode, sum(e.start + e.n for e in plan)))
        for e in plan:
            if e.sample and by_id[e.id]["ttft"] is None:
                by_id[e.id]["ttft"] = now - by_id[e.id]["t0"]
        self.scheduler.complete(plan, sampled)
        self.steps += 1
        if self.trace is not None:
            self.trace({"event": "step_completed", "step": self.steps, "requests": len(plan),
                        "tokens": sum(e.n for e in plan), "sampled": len(sampled),
                        "free_pages": self.engine.free_pages()})
        self._collect(by_id)
