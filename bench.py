#!/usr/bin/env python3
"""Benchmark: decode tokens/s and prefill tokens/s for the Qwen2.5-0.5B shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--impl ours|reference]

A "step" is one decode step of a batch of requests (default 8) that each hold a prompt of
512 tokens; W untimed warm-up steps, then exactly K timed steps between CUDA events.
`value` is decoded tokens per second with the sampled ids staying on the device (the
reference's --gpu-feedback mode, rust/engine/benches/qwen2.rs:182-229); `e2e` is the same
through the Python entry point `LLM.generate`, with host token ids going in and coming out
every step.  The line also carries a 2,048-token prefill, the decode step's HBM roofline
fraction, decode at batch 1 and 64, the GPU's clocks during the timed region and the number
of this repository's kernel launches inside it.  Inputs are larger than the L2 cache: a
decode step streams about 1 GB of weights, so nothing is flushed between steps.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the Qwen2.5-0.5B shape (random weights, seed 0, N(0, 0.02)).
QWEN25_05B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=151936, hidden_size=896,
    intermediate_size=4864, num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2,
    rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=4096, hidden_act="silu",
    tie_word_embeddings=True, use_sliding_window=False, eos_token_id=151645)
# Further sizes of the same architecture (--shape), for measurements beyond the headline configuration.
SHAPES = {
    "0.5B": QWEN25_05B,
    "1.5B": dict(QWEN25_05B, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28, num_attention_heads=12,
                 num_key_value_heads=2, max_position_embeddings=8192),
    "7B": dict(QWEN25_05B, vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28,
               num_attention_heads=28, num_key_value_heads=4, max_position_embeddings=16384,
               tie_word_embeddings=False),
}
PROMPT_LEN, NEW_TOKENS, PREFILL_TOKENS, PAGE_SIZE = 512, 256, 2048, 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            raw = json.load(open(path))
            return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"])}, "measured"
        except Exception:  # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "25"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.rows.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = [int(r[0]) for r in self.rows if r[0].isdigit()]
        mx = [int(r[1]) for r in self.rows if r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def model_folder(cfg_dict, layers):
    """A random-weights model folder for the configuration (made once per machine and size)."""
    import torch
    from llm_inference_lab_b200.registry import resolve
    from llm_inference_lab_b200.weights import write_random_model

    cfg_dict = dict(cfg_dict, num_hidden_layers=layers)
    folder = os.path.join(tempfile.gettempdir(), f"lab_b200_bench_qwen2_H{cfg_dict['hidden_size']}_L{layers}_{os.getuid()}")
    marker = os.path.join(folder, ".complete")
    if not os.path.exists(marker):
        cfg = resolve(cfg_dict).config_class.from_dict(cfg_dict)
        write_random_model(cfg, folder, seed=0, dtype=torch.bfloat16, std=0.02, norm_std=0.0)
        open(marker, "w").write("ok")
    return folder


def decode_bytes(cfg, layers, batch, mean_ctx):
    """Bytes a decode step has to read: every weight once, and the cache of the live requests."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d = h // cfg["num_attention_heads"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    per_layer = (nq + 2 * nkv) * d * h + (nq + 2 * nkv) * d + nq * d * h + 3 * h * i + 2 * h
    weights = 2 * (layers * per_layer + v * h + h)   # the head's matrix once (tied or not, a decode step reads one)
    cache = 2 * batch * mean_ctx * layers * 2 * nkv * d
    return weights + cache


def prefill_flops(cfg, layers, tokens):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    d = h // cfg["num_attention_heads"]
    nq, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    linear = 2 * tokens * layers * ((nq + 2 * nkv) * d * h + nq * d * h + 3 * h * i) + 2 * v * h
    attention = layers * nq * 2 * 2 * d * tokens * (tokens + 1) // 2
    return linear + attention


def run_decode(engine, graphs, batch, steps, warmup, rng, clocks=None, repeats=1):
    """Prefill `batch` prompts of PROMPT_LEN tokens, then time `steps` decode steps `repeats` times
    (device feedback: the sampled ids stay on the device).  `graphs` None: every step is launched
    kernel by kernel (eager) instead of replayed from a CUDA graph.  Returns a list of
    (ms of the region, launches, mean context length) per repeat."""
    import torch
    from llm_inference_lab_b200.engine import Entry
    from llm_inference_lab_b200.kernels import ops

    ids = list(range(batch))
    vocab = engine.vocab
    first = []
    for r in ids:
        prompt = [int(t) for t in rng.integers(0, vocab, PROMPT_LEN)]
        logits = engine.step([Entry(r, prompt, [PROMPT_LEN - 1])])
        first.append(int(logits.argmax(dim=-1).item()))
    if graphs is not None:
        out = graphs.step(ids, tokens=first)
        step = lambda: graphs.step(ids)  # noqa: E731
    else:
        eager = EagerDecode(engine, ids, first)
        out = eager.step()
        step = eager.step
    for _ in range(max(warmup - 1, 0)):
        out = step()
    torch.cuda.synchronize()
    regions = []
    if clocks is not None:
        clocks.__enter__()
    for _ in range(repeats):
        ctx0 = engine.cache.length(ids[0])
        launches0 = ops.COUNTER.launches
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            out = step()
        e1.record()
        torch.cuda.synchronize()
        regions.append((e0.elapsed_time(e1), ops.COUNTER.launches - launches0, ctx0 + (steps + 1) / 2.0))
    if clocks is not None:
        clocks.__exit__(None, None, None)
    tokens = out.cpu().tolist()
    assert all(0 <= t < vocab for t in tokens), "decode produced an invalid token"
    ops.take_device_errors()
    for r in ids:
        engine.close(r)
    return regions


class EagerDecode:
    """Decode steps launched kernel by kernel through `Engine.step`, the sampled ids fed forward on
    the device (the host never reads them): the eager twin of the decode graphs, for the figure the
    reference reports beside its graph mode (roadmap.md:653-656)."""

    def __init__(self, engine, ids, first):
        import torch
        self.engine, self.ids = engine, ids
        self.tokens = torch.tensor(first, dtype=torch.int32, device=engine.device)
        self.rows = torch.arange(len(ids), dtype=torch.int32, device=engine.device)

    def step(self):
        from llm_inference_lab_b200.kernels import ops
        eng = self.engine
        pairs = [(r, 1) for r in self.ids]
        began = eng._begin(pairs, False)
        try:
            ctx, _ = eng._pack_pairs(pairs, self.tokens)
            logits = eng.model.forward(ctx, eng.views, self.rows)
            ops.sample(logits, None, None, None, out=self.tokens)
        except Exception:
            eng._fail(began)
            raise
        eng._end(pairs, False)
        return self.tokens


def run_stack_stamps(engine, batch, rng):
    """The decode stack's own clock: CTA 0 stamps every phase (start, first operand built, first item
    done, all items done) and every CTA stamps the end of its share; printed per kind of phase."""
    import numpy as np
    import torch
    from llm_inference_lab_b200.engine import Entry

    stack = engine.model.decode_stack
    if stack is None:
        return {"error": "the model's layers do not fit the decode stack"}
    calls = len(stack.order)
    for r in range(batch):
        engine.step([Entry(r, [int(t) for t in rng.integers(0, engine.vocab, PROMPT_LEN)], [])])
    stack.stamps = torch.zeros((4 * 5 * calls + 1 + 5 * calls * stack.grid,), dtype=torch.int64, device="cuda")
    for _ in range(4):
        engine.step([Entry(r, [5], [0]) for r in range(batch)])
        torch.cuda.synchronize()
    full = stack.stamps.cpu().numpy().astype(np.int64)
    stack.stamps = None
    for r in range(batch):
        engine.close(r)
    t, per = full[: 4 * 5 * calls + 1], full[4 * 5 * calls + 1:].reshape(5 * calls, stack.grid)
    ph = t[:-1].reshape(calls, 5, 4)
    starts = np.concatenate([t[:-1].reshape(-1, 4)[:, 0], t[-1:]])
    out = {"kernel_us": round(float(t[-1] - t[0]) / 1e3, 1), "layer_calls": calls, "batch": batch, "phases": {}}
    skip = min(2, calls - 1)
    for k, name in enumerate(["qkv", "attention", "o_proj", "gate_up", "down"]):
        length = (starts[1:] - starts[:-1]).reshape(calls, 5)[skip:, k]
        entry = {"phase_us": round(float(length.mean()) / 1e3, 2)}
        if k != 1:      # (the warp that stamps takes no part in the attention phase)
            done = (per.reshape(calls, 5, -1)[skip:, k] - ph[skip:, k, 0][:, None]) / 1e3
            entry["cta_done_us_median"] = round(float(np.median(done)), 2)
            entry["cta_done_us_max"] = round(float(done.max(1).mean()), 2)
            entry["cta0_operand_us"] = round(float((ph[skip:, k, 1] - ph[skip:, k, 0]).mean()) / 1e3, 2)
            entry["cta0_item_us"] = round(float((ph[skip:, k, 2] - ph[skip:, k, 1]).mean()) / 1e3, 2)
        out["phases"][name] = entry
    return out


def median_region(regions):
    ordered = sorted(regions, key=lambda r: r[0])
    return ordered[len(ordered) // 2]


def run_prefill(engine, rng, repeats=5):
    import torch
    from llm_inference_lab_b200.engine import Entry

    times = []
    for it in range(3 + repeats):
        prompt = [int(t) for t in rng.integers(0, engine.vocab, PREFILL_TOKENS)]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits = engine.step([Entry(1000 + it, prompt, [PREFILL_TOKENS - 1])])
        e1.record()
        torch.cuda.synchronize()
        assert bool(torch.isfinite(logits).all())
        engine.close(1000 + it)
        if it >= 3:
            times.append(e0.elapsed_time(e1))
    return statistics.median(times)


def run_e2e(folder, batch, steps, warmup):
    """Decode tokens/s through LLM.generate: host ids in and out every step."""
    import numpy as np
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    llm = LLM(folder, "bf16", max_batch_tokens=8192, page_size=PAGE_SIZE,
              kv_tokens=batch * (PROMPT_LEN + NEW_TOKENS + PAGE_SIZE), max_requests=max(batch, 1),
              max_seq_len=4096, cuda_graph=True)
    rng = np.random.default_rng(1)
    prompts = [[int(t) for t in rng.integers(0, llm.engine.vocab, PROMPT_LEN)] for _ in range(batch)]
    n_new = min(NEW_TOKENS, warmup + steps + 2)
    llm.generate(prompts, SamplingConfig(max_new_tokens=4, ignore_eos=True))          # compiles and captures
    llm.step_log.clear()
    results = llm.generate(prompts, SamplingConfig(max_new_tokens=n_new, ignore_eos=True))
    assert all(len(r.tokens) == n_new for r in results)
    decode = [(t, n) for t, n, is_decode, _ in llm.step_log if is_decode and n == batch]
    timed = decode[warmup: warmup + steps + 1]
    k = len(timed) - 1
    seconds = timed[-1][0] - timed[0][0]
    meta_words = llm.graphs.cached[next(iter(llm.graphs.cached))].layout.total
    # Every decode step copies its metadata (positions, cache slots, block tables, lengths) from pinned
    # host memory and its sampled ids back to the host.  The ids themselves go from one step to the
    # next on the device: the step after is launched before the host has read them (lookahead).
    return {"value": batch * k / seconds, "unit": "tokens/s", "steps": k,
            "h2d_bytes_per_step": 4 * meta_words, "d2h_bytes_per_step": 4 * batch,
            "note": "LLM.generate; each step is launched one step ahead of the host's read of the sampled ids"}


def run_serve(folder, cfg, layers, requests, chunk, new_tokens, max_seq, lo=128, hi=2048, graph=True):
    """Continuous batching through LLM.generate: `requests` prompts of lo..hi tokens arrive at once, prompts
    are cut into portions under a budget of `chunk` tokens a step (decoding requests first), and every
    request decodes `new_tokens` tokens.  Timed on the host around the whole call, after two untimed
    runs of the same work (they compile, and capture the graphs the timed run replays)."""
    import numpy as np
    import torch
    from llm_inference_lab_b200.engine.llm import LLM
    from llm_inference_lab_b200.sampling import SamplingConfig

    rng = np.random.default_rng(2)
    lengths = [int(n) for n in rng.integers(lo, hi + 1, requests)]
    need = sum(-(-(n + new_tokens) // PAGE_SIZE) * PAGE_SIZE for n in lengths)
    llm = LLM(folder, "bf16", max_batch_tokens=chunk, page_size=PAGE_SIZE, kv_tokens=need + 64 * PAGE_SIZE,
              max_requests=requests, max_seq_len=max_seq, cuda_graph=graph)
    prompts = [[int(t) for t in rng.integers(0, llm.engine.vocab, n)] for n in lengths]
    sampling = SamplingConfig(max_new_tokens=new_tokens, ignore_eos=True)
    for _ in range(2):      # the second run captures the step shapes that came twice
        llm.generate(prompts, sampling)
    torch.cuda.synchronize()
    llm.step_log.clear()
    steps0 = llm.steps
    replays0 = (llm.graphs.replays if llm.graphs else 0, llm.engine.graph_replays)
    t0 = time.perf_counter()
    results = llm.generate(prompts, sampling)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    assert all(r.finish_reason == "length" and len(r.tokens) == new_tokens for r in results)
    generated = requests * new_tokens
    steps = llm.steps - steps0
    log = llm.step_log
    decode_steps = sum(1 for _, _, is_decode, _ in log if is_decode)
    from_graphs = ((llm.graphs.replays if llm.graphs else 0) - replays0[0]) + (llm.engine.graph_replays - replays0[1])
    # Pure decode steps against the HBM roofline: the bytes each has to read (every weight once and
    # the cache of its requests) over the time between its tokens and the previous step's reaching
    # the host (steps run back to back, one launched ahead).
    nbytes = seconds_decode = 0.0
    for prev, cur in zip(log, log[1:]):
        if cur[2] and prev[2]:
            nbytes += decode_bytes(cfg, layers, 0, 0) + kv_bytes_per_token(cfg, layers) * cur[3]
            seconds_decode += cur[0] - prev[0]
    return {"workload": f"continuous batching: {requests} requests at once, prompts of {lo}..{hi} tokens, "
                        f"{chunk} tokens a step, {new_tokens} new tokens each",
            "seconds": round(seconds, 4), "prompt_tokens": sum(lengths), "generated_tokens": generated,
            "total_tokens_per_s": round((sum(lengths) + generated) / seconds, 1),
            "generated_tokens_per_s": round(generated / seconds, 1),
            "steps": steps, "pure_decode_steps": decode_steps,
            "steps_from_graphs": from_graphs, "eager_share": round(1.0 - from_graphs / max(steps, 1), 4),
            "ms_per_step": round(1e3 * seconds / max(steps, 1), 4),
            "decode_hbm_gbs": round(nbytes / max(seconds_decode, 1e-9) / 1e9, 1),
            "ttft_ms_median": round(1e3 * statistics.median(r.ttft for r in results), 2),
            "preemptions": sum(r.preemptions for r in results)}


def kv_bytes_per_token(cfg, layers):
    d = cfg["hidden_size"] // cfg["num_attention_heads"]
    return 2 * layers * 2 * cfg["num_key_value_heads"] * d


def main() -> int:
    global PROMPT_LEN, PREFILL_TOKENS
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--shape", default="0.5B", choices=sorted(SHAPES),
                    help="layer sizes of another model of the architecture (the headline is 0.5B)")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="tokens each request holds before decoding")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out decode at batch 1 and 64 and the prefill")
    ap.add_argument("--skip-e2e", action="store_true", help="leave out the run through LLM.generate")
    ap.add_argument("--no-graph", action="store_true",
                    help="time decode steps launched kernel by kernel instead of replayed from CUDA graphs")
    ap.add_argument("--serve", type=int, default=0, metavar="REQUESTS",
                    help="instead of the headline run: REQUESTS prompts of 128..2,048 tokens through LLM.generate "
                         "with 512 tokens a step and 128 new tokens each (continuous batching); prints its own line")
    ap.add_argument("--stack-stamps", action="store_true",
                    help="run a few eager decode steps with the decode stack's in-kernel clock on and print what "
                         "each kind of phase took")
    ap.add_argument("--only-prefill", type=int, default=0, metavar="TOKENS",
                    help="run only a prefill of TOKENS tokens a few times and print its time (for profiling)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "pochenai/llm-inference-lab is a Rust + cuTile engine: no cargo/rustc or cuTile toolchain "
                          "offline, and the offline pip install stops at metadata-generation-failed (its pyproject.toml holds no engine)"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "this engine runs on one GPU; --gpus must be 1", "n_gpus": args.gpus}))
        return 2
    warmup = max(args.warmup, 3)
    steps = max(1, min(args.steps, NEW_TOKENS - warmup - 2))
    PROMPT_LEN = args.prompt_len
    cfg = SHAPES[args.shape]
    args.layers = args.layers or cfg["num_hidden_layers"]
    headline = args.shape == "0.5B" and PROMPT_LEN == 512
    max_seq = max(4096, PROMPT_LEN + NEW_TOKENS + PAGE_SIZE, args.only_prefill + PAGE_SIZE)
    live = max(64 if headline else 0, args.batch)      # requests that hold pages at the same time

    import numpy as np
    import torch
    from llm_inference_lab_b200.engine import Engine
    from llm_inference_lab_b200.engine.decode_graph import DecodeGraphs

    folder = model_folder(cfg, args.layers)
    pk, pk_src = peaks()
    if args.serve:
        clocks = ClockSampler()
        with clocks:
            out = run_serve(folder, cfg, args.layers, args.serve, 512, 128, max(max_seq, 2048 + 128 + PAGE_SIZE),
                            graph=not args.no_graph)
        out["decode_hbm_frac"] = round(out["decode_hbm_gbs"] / pk["hbm_gbs"], 4)
        out.update({"model": f"Qwen2.5-{args.shape} shape", "layers": args.layers,
                    "layers_of_config": cfg["num_hidden_layers"], "dtype": "bf16",
                    "mode": "eager launches" if args.no_graph else "cuda graphs", "peaks": pk_src,
                    "clocks": clocks.summary()})
        print(json.dumps(out))
        return 0
    rng = np.random.default_rng(0)
    engine = Engine(folder, "bf16", max_tokens=live * (PROMPT_LEN + NEW_TOKENS + PAGE_SIZE) + max(4096, args.only_prefill),
                    page_size=PAGE_SIZE,
                    max_requests=live, max_batch_tokens=max(8192, PROMPT_LEN, args.only_prefill), max_seq_len=max_seq)
    graphs = DecodeGraphs(engine)
    engine.enable_step_graphs()   # a prefill of a repeating shape is replayed from a CUDA graph

    if args.stack_stamps:
        print(json.dumps(run_stack_stamps(engine, args.batch, rng)))
        return 0
    if args.only_prefill:
        PREFILL_TOKENS = args.only_prefill
        pms = run_prefill(engine, rng, repeats=2)
        print(json.dumps({"prefill_tokens": PREFILL_TOKENS, "ms": round(pms, 4), "layers": args.layers,
                          "tokens_per_s": round(PREFILL_TOKENS / (pms / 1e3), 1)}))
        return 0

    # The timed region (K steps between two events) is taken R times in a row, as far as the requests'
    # budgets of new tokens allow; the line reports the median region, with the fastest and the slowest.
    repeats = max(1, min(5, (NEW_TOKENS - warmup - 2) // steps))
    clocks = ClockSampler()
    regions = run_decode(engine, None if args.no_graph else graphs, args.batch, steps, warmup, rng, clocks, repeats)
    ms, launches, mean_ctx = median_region(regions)
    value = args.batch * steps / (ms / 1e3)
    nbytes = decode_bytes(cfg, args.layers, args.batch, mean_ctx)
    achieved = nbytes / (ms / steps / 1e3) / 1e9

    line = {
        "metric": f"decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Qwen2.5-{args.shape})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0, 0.02) seed 0, uniform-random token ids",
        "config": {
            "model": f"Qwen2.5-{args.shape} shape", "global_batch": args.batch, "seq_len": max_seq,
            "parallelism": "single-gpu",
            "layers": args.layers, "layers_of_config": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "rope_theta": cfg["rope_theta"], "tied_embeddings": cfg["tie_word_embeddings"],
            "prompt_len": PROMPT_LEN, "new_tokens": NEW_TOKENS, "page_size": PAGE_SIZE,
            "decode": ("eager launches" if args.no_graph else "cuda-graph") + ", device feedback",
            "l2": f"inputs larger than L2 ({nbytes / 1e9:.1f} GB of weights and cache per step)",
            "peaks": pk_src},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "gpu_launches": launches,
        "repeats": {"n": len(regions), "ms_per_step_min": round(min(r[0] for r in regions) / steps, 4),
                    "ms_per_step_max": round(max(r[0] for r in regions) / steps, 4)},
        "clocks": clocks.summary(),
    }
    if not args.skip_points:
        pms = run_prefill(engine, rng)
        flops = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
        line["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS,
                           "ms": round(pms, 4), "frac": round(flops / (pms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        points = {}
        for b in ((1, 64) if headline else ()):
            k = min(steps, 100)
            bms, _, _ = median_region(run_decode(engine, graphs, b, k, warmup, rng, repeats=min(repeats, 3)))
            points[f"decode_b{b}"] = round(b * k / (bms / 1e3), 1)
        if not args.no_graph:
            # the same steps launched kernel by kernel: the reference reports both modes
            k = min(steps, 100)
            ems, _, _ = median_region(run_decode(engine, None, args.batch, k, warmup, rng, repeats=min(repeats, 3)))
            points[f"decode_b{args.batch}_eager"] = round(args.batch * k / (ems / 1e3), 1)
        line["points"] = points
    del graphs, engine
    torch.cuda.empty_cache()
    if not args.skip_e2e and headline:
        try:
            line["e2e"] = {k: (round(v, 1) if isinstance(v, float) else v)
                           for k, v in run_e2e(folder, args.batch, steps, warmup).items()}
        except Exception as exc:  # noqa: BLE001 - the device-timed number stands on its own
            line["e2e"] = {"error": f"{type(exc).__name__}: {exc}"}
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
