"""The step function: one packed batch in, logits at the wanted places out.

`Engine.step` takes entries ``(request id, next tokens, wanted places)``:
portions of prompts beside single decoded tokens, cut anywhere.  It runs only
the tokens it is given, as one batch, on top of the cache that earlier steps
left, and returns 32-bit logits at the wanted places.  It is the counterpart of
the reference's `CausalModel::next_tokens` / `step_with_logits`
(rust/engine/src/runner/model/api.rs:203-243;
rust/engine/src/runner/model/qwen2/engine.rs:781-789, 916-1130), with the
difference that logits are produced only where asked (the reference computes a
prediction at the end of every portion and the runner drops it,
rust/engine/README.md:549-551).

Order inside a step, as in the reference's `execute_append_batch`
(rust/engine/src/runner/model/api.rs:80-106): validate, reserve pages, upload
the step's metadata, run the kernels, then commit the cache.  A step that fails
gives its reserved pages back.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache import manager as cache_mod
from ..kernels import ops
from ..models.builder import CausalLM, load_model
from ..parts.base import CacheView, GroupView, StepContext
from ..parts.spec import FixedState, PagedKV
from .. import profiling

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32,
          "fp32": torch.float32}


class InvalidInput(ValueError):
    """An entry the step refuses before anything runs (rust/engine/src/runner/model/error.rs:7-12)."""


@dataclasses.dataclass
class Entry:
    """One request's share of a step."""
    request: int
    tokens: Sequence[int]
    want: Sequence[int] = ()     # places among `tokens` whose logits are asked for


@dataclasses.dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name in (torch.bfloat16, torch.float32):
            return name
        raise ValueError(f"unsupported dtype {name}")
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r}: use bfloat16 or float32") from None


class Engine:
    """A model, its cache and the step function, on one GPU."""

    def __init__(self, model: CausalLM | str, dtype="bfloat16", *, max_tokens: Optional[int] = None,
                 page_size: int = 16, max_requests: int = 64, max_batch_tokens: int = 8192,
                 max_seq_len: Optional[int] = None, device="cuda:0"):
        ops.require_gpu()
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = parse_dtype(dtype)
        if isinstance(model, str):
            model, self.config = load_model(model, self.dtype, self.device)
        else:
            self.config = None
        if model.dtype != self.dtype:
            raise ValueError("the model was built for another dtype than the engine")
        self.model = model
        bp = model.blueprint
        self.vocab = bp.vocab
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_seq_len = int(min(max_seq_len or bp.max_positions, bp.max_positions))
        if max_tokens is None:
            max_tokens = self.max_seq_len * min(self.max_requests, 8)
        # Every request's count is rounded up to whole pages, so the pool is counted in pages.
        self.num_pages = -(-int(max_tokens) // self.page_size)
        plan = model.cache_plan
        rt = cache_mod.runtime()
        groups = [rt.GroupConfig(self.page_size, w, self.num_pages) for w in plan.group_windows]
        self.cache = rt.CacheManager(groups, self.max_requests)
        self.group_windows = list(plan.group_windows)
        self.views: list[CacheView] = []
        for need, group in zip(plan.needs, plan.group_of):
            if isinstance(need, PagedKV):
                shape = (self.num_pages, need.n_kv_heads, self.page_size, need.head_dim)
                # Pages are never cleared: what may be read is decided by lengths alone.
                k = torch.empty(shape, dtype=self.dtype, device=self.device)
                v = torch.empty(shape, dtype=self.dtype, device=self.device)
                self.views.append(CacheView(need, group=group, k=k, v=v))
            elif isinstance(need, FixedState):
                state = torch.zeros((self.max_requests,) + tuple(need.shape), dtype=torch.float32, device=self.device)
                self.views.append(CacheView(need, state=state))
            else:
                self.views.append(CacheView(None))
        self.stateful = any(v.state is not None for v in self.views)
        self.max_blocks = -(-self.max_seq_len // self.page_size)
        self.stats = EngineStats()
        self._staging = [self._new_staging() for _ in range(3)]
        self._staging_at = 0
        # Steps whose shape repeats (same token counts per request, same wanted counts) can be
        # replayed from CUDA graphs; off until `enable_step_graphs` is called.
        self._graphs_on = False
        self._graphs: dict = {}
        self._seen: dict = {}
        self._graphs_max = 8
        self.graph_replays = 0

    # ------------------------------------------------------------------------------------
    def _new_staging(self):
        n_groups = len(self.group_windows)
        cap_t, cap_b = self.max_batch_tokens, self.max_requests
        words = (cap_t * (4 + n_groups) + cap_b * (5 + n_groups * (self.max_blocks + 8)) + 64) + 4 * 16
        buf = torch.empty((words,), dtype=torch.int32, pin_memory=True)
        return {"host": buf, "np": buf.numpy(), "event": None}

    def _next_staging(self):
        st = self._staging[self._staging_at]
        self._staging_at = (self._staging_at + 1) % len(self._staging)
        if st["event"] is not None:
            st["event"].synchronize()
        return st

    def enable_step_graphs(self, max_cached: int = 8) -> None:
        """Replay steps of a repeating shape from CUDA graphs (captured when a shape comes a second
        time).  The logits a replayed step returns live in the graph's buffer: read them before the
        next step of the same shape.  Models with fixed-size per-request state keep running eagerly
        (their mixers may index the state on the host)."""
        self._graphs_on = not self.stateful
        self._graphs_max = max_cached

    # ------------------------------------------------------------------------------------
    def open(self, request: int) -> None:
        """A new request: takes a state slot.  Its fixed-size state is cleared here and again by the
        first step that brings it tokens (the scheduler opens requests without the engine)."""
        slot = self.cache.open(int(request))
        for view in self.views:
            if view.state is not None:
                view.state[slot].zero_()

    def close(self, request: int) -> None:
        """The request ends; its pages and its state slot may be used again."""
        self.cache.close(int(request))

    def has(self, request: int) -> bool:
        return self.cache.has(int(request))

    def length(self, request: int) -> int:
        return self.cache.length(int(request))

    def free_pages(self) -> list[int]:
        return [self.cache.free_pages(g) for g in range(self.cache.num_groups)]

    # ------------------------------------------------------------------------------------
    def validate(self, entries: Sequence[Entry], reserved: bool = False) -> None:
        """Refuses a step before anything runs.  With ``reserved`` the cache already counts this
        step's tokens for every entry."""
        if not entries:
            raise InvalidInput("a step needs at least one entry")
        seen = set()
        total = 0
        for e in entries:
            n = len(e.tokens)
            if e.request in seen:
                raise InvalidInput(f"request {e.request} appears twice in one step")
            seen.add(e.request)
            if n == 0:
                raise InvalidInput(f"request {e.request}: no tokens in this step")
            held = self.cache.reserved(e.request) if self.cache.has(e.request) else 0
            after = held if reserved else held + n
            if after > self.max_seq_len:
                raise InvalidInput(f"request {e.request}: {after} tokens exceed the maximum sequence length "
                                   f"{self.max_seq_len}")
            lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab:
                raise InvalidInput(f"request {e.request}: token id outside [0, {self.vocab})")
            for w in e.want:
                if not 0 <= w < n:
                    raise InvalidInput(f"request {e.request}: wanted place {w} outside its {n} tokens")
            total += n
        if total > self.max_batch_tokens:
            raise InvalidInput(f"{total} tokens in one step exceed max_batch_tokens {self.max_batch_tokens}")
        if len(entries) > self.max_requests:
            raise InvalidInput(f"{len(entries)} requests in one step exceed max_requests {self.max_requests}")

    def step(self, entries: Sequence[Entry], reserved: bool = False, pick=None) -> Optional[torch.Tensor]:
        """Runs one packed batch.  Returns 32-bit logits [wanted, vocab] on the device, in
        the order of the entries and of their `want`, or None if nothing was wanted.

        With ``reserved`` the caller (the scheduler) has reserved the pages already.  With ``pick`` =
        (temperatures, seeds, positions), device tensors with one element per wanted place (or three
        Nones for greedy), the step returns one token id per wanted place (int32 on the device)
        instead of logits: the head picks them itself and no logits are written.
        """
        entries = [e if isinstance(e, Entry) else Entry(*e) for e in entries]
        self.validate(entries, reserved)
        if not profiling.ON:
            return self._step(entries, reserved, pick)
        # The reference's label: a prefill step if any request brings more than one token or holds
        # nothing yet (rust/engine/src/runner/model/qwen2/engine.rs:862-864).
        prefill = any(len(e.tokens) > 1 or not self.cache.has(e.request) or self.cache.length(e.request) == 0
                      for e in entries)
        with profiling.scoped_range("step.prefill" if prefill else "step.decode"):
            return self._step(entries, reserved, pick)

    def _step(self, entries: Sequence[Entry], reserved: bool, pick=None) -> Optional[torch.Tensor]:
        pairs = [(int(e.request), len(e.tokens)) for e in entries]
        began = self._begin(pairs, reserved)
        try:
            logits = self._run(entries, pick)
        except Exception:
            self._fail(began)
            raise
        self._end(pairs, reserved)
        return logits

    # The three pieces of every step's book-keeping, shared by the eager path, the step graphs and
    # the decode graphs: begin (open, reserve, prepare fixed-size state), then end or fail.
    def _begin(self, pairs, reserved: bool):
        """Opens unknown requests, reserves pages unless the caller has, and prepares fixed-size
        state: a request that holds no committed token yet (new, or preempted and reopened, whoever
        opened it) starts from zeros, and the rows of the step's requests are saved so that a
        failed step can put them back.  Returns what `_fail` needs."""
        opened, taken, saved = [], [], None
        try:
            for r, _ in pairs:
                if not self.cache.has(r):
                    self.cache.open(r)
                    opened.append(r)
            if not reserved:
                for r, n in pairs:
                    self.cache.reserve(r, n)
                    taken.append(r)
            if self.stateful:
                slots = torch.tensor([self.cache.state_slot(r) for r, _ in pairs], dtype=torch.long,
                                     device=self.device)
                fresh = [i for i, (r, _) in enumerate(pairs) if self.cache.length(r) == 0]
                saved = []
                for view in self.views:
                    if view.state is None:
                        continue
                    if fresh:
                        view.state[slots[fresh]] = 0
                    saved.append((view.state, slots, view.state[slots]))
        except Exception:
            self._fail((opened, taken, None))
            raise
        return opened, taken, saved

    def _fail(self, began) -> None:
        """A step failed: fixed-size state goes back to what it was, pages reserved here are given
        back, requests opened here are closed."""
        opened, taken, saved = began
        for state, slots, rows in saved or ():
            state[slots] = rows
        for r in taken:
            self.cache.rollback(r)
        for r in opened:
            self.cache.close(r)

    def _end(self, pairs, reserved: bool) -> None:
        if not reserved:
            for r, n in pairs:
                self.cache.commit(r, n)
        self.stats.steps += 1
        for r, n in pairs:
            if n == 1 and self.cache.reserved(r) > 1:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += n

    # ------------------------------------------------------------------------------------
    def _run(self, entries: Sequence[Entry], pick=None):
        """Packs the step and runs the model, eagerly or from a CUDA graph of the same shape (a step
        that picks its tokens itself runs eagerly)."""
        if self._graphs_on and pick is None:
            max_kv = max(self.cache.reserved(e.request) for e in entries)
            bucket = 256
            while bucket < max_kv:
                bucket *= 2
            sig = (tuple(len(e.tokens) for e in entries), tuple(len(e.want) for e in entries), bucket)
            cap = self._graphs.get(sig)
            if cap is not None:
                self._fill(entries, cap["layout"], cap["widths"], cap["dev"], cap["tok_at"], cap["want_at"])
                cap["graph"].replay()
                ops.COUNTER.launches += cap["launches"]
                self.graph_replays += 1
                return cap["logits"]
            # Captured the second time a shape comes; a shape whose graph was pushed out by newer
            # ones is captured again only at its 4th, 8th, 16th... coming, so a workload of ever
            # changing shapes does not pay for a capture at every step.
            if len(self._seen) > 4096:      # shapes that never came back: forget the counts
                self._seen.clear()
            seen = self._seen[sig] = self._seen.get(sig, 0) + 1
            if seen >= 2 and seen & (seen - 1) == 0:
                return self._capture(sig, entries, bucket)
        ctx, logit_rows = self._pack(entries)
        if pick is not None and logit_rows is not None:
            return self.model.forward(ctx, self.views, logit_rows, pick=(*pick, None))
        return self.model.forward(ctx, self.views, logit_rows)

    def _capture(self, sig, entries, bucket):
        if len(self._graphs) >= self._graphs_max:
            self._graphs.pop(next(iter(self._graphs)))
        pairs = [(int(e.request), len(e.tokens)) for e in entries]
        T, B = sum(n for _, n in pairs), len(pairs)
        n_want = sum(len(e.want) for e in entries)
        widths = [self.max_blocks] * len(self.group_windows)
        layout = self.cache.layout(T, B, widths)
        tok_at = layout.total
        want_at = tok_at + ((T + 3) & ~3)
        total = want_at + ((n_want + 3) & ~3)
        dev = torch.zeros((total,), dtype=torch.int32, device=self.device)
        self._fill(entries, layout, widths, dev, tok_at, want_at)
        q_lens = [n for _, n in pairs]
        ctx = self._context(dev, layout, widths, T, B, q_lens, [bucket] * B, [], dev[tok_at: tok_at + T])
        rows = dev[want_at: want_at + n_want] if n_want else None
        # One eager run (it also configures kernels and warms the allocator), then the capture.
        # Running the step more than once is harmless: it writes the same cache entries again.
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self.model.forward(ctx, self.views, rows)
        torch.cuda.current_stream().wait_stream(side)
        ctx.scratch.clear()
        graph = torch.cuda.CUDAGraph()
        before = ops.COUNTER.launches
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx, self.views, rows)
        launches = ops.COUNTER.launches - before
        ops.COUNTER.launches = before
        cap = {"graph": graph, "layout": layout, "widths": widths, "dev": dev, "tok_at": tok_at, "want_at": want_at,
               "logits": logits, "launches": launches}
        self._graphs[sig] = cap
        graph.replay()
        ops.COUNTER.launches += launches
        self.graph_replays += 1
        return logits

    def _fill(self, entries, layout, widths, dev, tok_at, want_at, pairs=None) -> None:
        """Writes a step's metadata, token ids and wanted rows into `dev` through pinned memory."""
        if pairs is None:
            pairs = [(int(e.request), len(e.tokens)) for e in entries]
        n_want = sum(len(e.want) for e in entries)
        total = want_at + ((n_want + 3) & ~3)
        st = self._next_staging()
        if total > st["np"].shape[0]:
            raise InvalidInput("step metadata exceeds the staging buffer")
        host = st["np"]
        self.cache.pack(pairs, layout, host, 0, 0)
        row = 0
        wi = want_at
        for e in entries:
            n = len(e.tokens)
            host[tok_at + row: tok_at + row + n] = np.asarray(e.tokens, dtype=np.int32)
            for w in e.want:
                host[wi] = row + w
                wi += 1
            row += n
        ops.copy_to_device(dev, st["host"], 0, total)
        ev = torch.cuda.Event()
        ev.record()
        st["event"] = ev

    def _context(self, dev, layout, widths, T, B, q_lens, kv_lens, state_slots, token_ids) -> StepContext:
        def view(at, n):
            return dev[at: at + n]

        n_groups = len(self.group_windows)
        groups = [GroupView(self.page_size, self.group_windows[g], view(layout.row_slot[g], T),
                            view(layout.block_table[g], B * widths[g]).view(B, widths[g])) for g in range(n_groups)]
        return StepContext(
            dtype=self.dtype, device=self.device, n_tokens=T, n_requests=B,
            token_ids=token_ids, row_req=view(layout.row_req, T), row_pos=view(layout.row_pos, T),
            q_start=view(layout.q_start, B + 1), kv_len=view(layout.kv_len, B), pos0=view(layout.pos0, B),
            state_slot=view(layout.state_slot, B), groups=groups, q_lens=q_lens, kv_lens=kv_lens,
            state_slots=state_slots, max_q_len=max(q_lens), max_kv_len=max(kv_lens))

    def _pack(self, entries: Sequence[Entry]):
        return self._pack_pairs([(int(e.request), len(e.tokens)) for e in entries], None, entries)

    def _pack_pairs(self, pairs, token_ids: Optional[torch.Tensor], entries: Sequence[Entry] = ()):
        """The context of an eager step.  With `token_ids` (int32 on the device, one per row) the ids
        stay where they are and `entries` bring none; no rows are wanted then."""
        T = sum(n for _, n in pairs)
        B = len(pairs)
        widths = []
        for g in range(len(self.group_windows)):
            width = max(-(-self.cache.reserved(r) // self.page_size) for r, _ in pairs)
            widths.append((width + 7) & ~7)
        layout = self.cache.layout(T, B, widths)
        n_want = sum(len(e.want) for e in entries)
        tok_at = layout.total
        want_at = tok_at + ((T + 3) & ~3)
        total = want_at + ((n_want + 3) & ~3)
        dev = torch.empty((total,), dtype=torch.int32, device=self.device)
        self._fill(entries, layout, widths, dev, tok_at, want_at, pairs)
        ctx = self._context(dev, layout, widths, T, B, [n for _, n in pairs],
                            [self.cache.reserved(r) for r, _ in pairs],
                            [self.cache.state_slot(r) for r, _ in pairs],
                            dev[tok_at: tok_at + T] if token_ids is None else token_ids)
        logit_rows = dev[want_at: want_at + n_want] if n_want else None
        return ctx, logit_rows
