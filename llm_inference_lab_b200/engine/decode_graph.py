"""Decode steps replayed from CUDA graphs.

A step in which every request brings exactly one token has the same launches
every time; only the metadata (positions, cache slots, block tables, lengths)
and the token ids change.  Such a step is captured once per (batch size, number
of key splits) into a CUDA graph over fixed buffers; later steps copy their
metadata into those buffers and replay the graph.  The sampled tokens stay in a
device buffer that is also the next step's input, so a run of decode steps
needs no copy back to the host unless the caller wants the tokens.

The reference does the same for pure-decode steps: fixed metadata and source
buffers uploaded before replay, graphs keyed by (slot table, batch, splits), a
handful cached (rust/engine/src/runner/model/qwen2/graph.rs:18-151; capture in
rust/engine/src/runner/model/qwen2/engine.rs:467-640, replay 713-752).
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence

import numpy as np
import torch

from ..kernels import ops
from ..parts.base import StepContext
from .engine import InvalidInput


@dataclasses.dataclass
class _Captured:
    graph: torch.cuda.CUDAGraph
    layout: object
    buf: torch.Tensor           # one int32 device buffer: [temps B | seeds B | metadata | tokens B]
    dev: torch.Tensor           # view: the int32 metadata
    tokens: torch.Tensor        # view [B] int32: input ids of the step, overwritten with the sampled ids
    temps: torch.Tensor         # view [B] float32
    seeds: torch.Tensor         # view [B] int32
    rows: torch.Tensor          # [B] int32: 0..B-1, the rows whose logits are computed
    host_tokens: torch.Tensor   # [B] int32 in pinned memory: the sampled ids, copied by the graph itself
    logits: Optional[torch.Tensor] = None   # [B, vocab] float32 of the last replay (lives in the graph's pool)
    launches: int = 0           # kernels the graph holds


class DecodeGraphs:
    MAX_CACHED = 16
    MAX_KEPT_BATCH = 1024

    def __init__(self, engine):
        if engine.stateful:
            # A mixer with state of its own may index it on the host, and the warm-up run before a
            # capture would advance it twice: such models step eagerly.
            raise ValueError("decode graphs do not serve models with fixed-size per-request state")
        self.engine = engine
        self.cached: dict[tuple, _Captured] = {}
        self.replays = 0
        self.captures = 0
        self._last, self._last_requests = None, None
        self._pairs_of = None
        self._ring, self._ring_at = [], 0     # pinned buffers for the ids of steps launched with `keep`
        self._done = torch.cuda.Event()     # recorded after every replay

    # ------------------------------------------------------------------------------------
    def _key(self, n_requests: int, max_kv_len: int):
        return (n_requests, max(256, 1 << (int(max_kv_len) - 1).bit_length()))

    def _context(self, cap: _Captured, B: int, kv_bucket: int) -> StepContext:
        eng = self.engine
        widths = [eng.max_blocks] * len(eng.group_windows)
        return eng._context(cap.dev, cap.layout, widths, B, B, [1] * B, [kv_bucket] * B, [], cap.tokens)

    def _run(self, cap: _Captured, ctx: StepContext) -> torch.Tensor:
        logits = self.engine.model.forward(ctx, self.engine.views, cap.rows)
        # position of the token being drawn = tokens held after this step
        ops.sample(logits, cap.temps, cap.seeds, ctx.kv_len, out=cap.tokens)
        cap.host_tokens.copy_(cap.tokens, non_blocking=True)   # part of the graph: no launch of its own later
        return logits

    def _new_capture(self, key):
        eng = self.engine
        B, kv_bucket = key
        n_groups = len(eng.group_windows)
        layout = eng.cache.layout(B, B, [eng.max_blocks] * n_groups)
        # Temperatures and seeds before the metadata, tokens after it: whatever a step brings from
        # the host is one contiguous piece, and one copy.
        buf = torch.zeros((3 * B + layout.total,), dtype=torch.int32, device=eng.device)
        at = 2 * B
        cap = _Captured(graph=torch.cuda.CUDAGraph(), layout=layout, buf=buf, dev=buf[at: at + layout.total],
                        tokens=buf[at + layout.total: at + layout.total + B], temps=buf[0: B].view(torch.float32),
                        seeds=buf[B: 2 * B], rows=torch.arange(B, dtype=torch.int32, device=eng.device),
                        host_tokens=torch.zeros((B,), dtype=torch.int32, pin_memory=True))
        return cap, self._context(cap, B, kv_bucket)

    # ------------------------------------------------------------------------------------
    def step(self, requests: Sequence[int], tokens: Optional[Sequence[int]] = None,
             temps: Optional[Sequence[float]] = None, seeds: Optional[Sequence[int]] = None,
             reserved: bool = False, keep: bool = False):
        """One decode step for `requests` (each brings one token).  `tokens` are the input ids
        on the host; None means: the ids the previous step of the same batch sampled, which
        are still on the device.  Returns the device buffer [B] of sampled ids (valid until
        the next step of this batch size); with `keep`, a ticket for `read` instead: the ids are
        also copied into a pinned buffer of their own, so that they can be read after later steps
        have been launched."""
        eng = self.engine
        B = len(requests)
        if self._pairs_of is not None and self._pairs_of[0] == requests:
            pairs = self._pairs_of[1]           # the same batch as last time
        else:
            pairs = [(int(r), 1) for r in requests]
            if len(set(requests)) != B or B == 0:
                raise InvalidInput("a decode step needs one entry per request, and at least one")
            self._pairs_of = (list(requests), pairs)
        if tokens is not None and not all(0 <= t < eng.vocab for t in tokens):
            raise InvalidInput(f"token id outside [0, {eng.vocab})")
        same_batch = self._last is not None and self._last_requests == requests
        if tokens is None and not same_batch:
            raise InvalidInput("no input ids given, and the previous step was not one of these requests")
        began = eng._begin(pairs, reserved)
        try:
            cap = self._launch(pairs, B, tokens, temps, seeds, same_batch)
        except Exception:
            eng._fail(began)
            raise
        eng._end(pairs, reserved)
        self._last, self._last_requests = cap, list(requests)
        if keep:
            if not self._ring:
                self._ring = [(torch.zeros((self.MAX_KEPT_BATCH,), dtype=torch.int32, pin_memory=True),
                               torch.cuda.Event()) for _ in range(4)]
            if B > self.MAX_KEPT_BATCH:
                raise ValueError("batch too large for the kept-token buffers")
            buf, event = self._ring[self._ring_at]
            self._ring_at = (self._ring_at + 1) % len(self._ring)
            buf[:B].copy_(cap.tokens, non_blocking=True)
            event.record(ops.current_stream())
            return (buf, event, B)
        return cap.tokens

    def _launch(self, pairs, B, tokens, temps, seeds, same_batch) -> _Captured:
        """Uploads the step's metadata into the buffers of the graph that serves it (captured now if
        it is new) and replays it."""
        eng = self.engine
        max_kv = max(eng.cache.reserved(r) for r, _ in pairs)
        if max_kv > eng.max_seq_len:
            raise InvalidInput("a request exceeds the maximum sequence length")
        key = self._key(B, max_kv)
        fresh = key not in self.cached
        if fresh:
            if len(self.cached) >= self.MAX_CACHED:
                self.cached.pop(next(iter(self.cached)))
            cap, ctx = self._new_capture(key)
        else:
            cap = self.cached[key]
        st = eng._next_staging()
        n_meta = cap.layout.total
        host = st["np"]
        eng.cache.pack(pairs, cap.layout, host[2 * B:], 0, 0)
        lo, hi = 2 * B, 2 * B + n_meta
        moved = cap is not self._last
        if tokens is not None:
            host[hi: hi + B] = np.asarray(tokens, dtype=np.int32)
            hi += B
        elif moved:
            # the previous step of this batch ran from another graph (its context outgrew a bucket):
            # the ids it sampled move over on the device
            cap.tokens.copy_(self._last.tokens, non_blocking=True)
        if temps is not None:
            host[0: B].view(np.float32)[:] = np.asarray(list(temps), dtype=np.float32)
            host[B: 2 * B] = np.asarray([s & 0x7FFFFFFF for s in seeds], dtype=np.int32)
            lo = 0
        elif same_batch and moved:
            # ... and so do the temperatures and seeds, which live in each graph's own buffer
            cap.buf[0: 2 * B].copy_(self._last.buf[0: 2 * B], non_blocking=True)
        elif not same_batch:
            host[0: 2 * B] = 0          # nobody said otherwise: greedy
            lo = 0
        ops.copy_to_device(cap.buf, st["host"], lo, hi)
        stream = ops.current_stream()
        ev = st.get("own_event")
        if ev is None:
            ev = st["own_event"] = torch.cuda.Event()
        ev.record(stream)
        st["event"] = ev
        if fresh:
            # One eager run configures the kernels and fills the allocator, then the capture.
            saved = cap.tokens.clone()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self._run(cap, ctx)
            torch.cuda.current_stream().wait_stream(side)
            cap.tokens.copy_(saved)
            before = ops.COUNTER.launches
            with torch.cuda.graph(cap.graph):
                cap.logits = self._run(cap, ctx)
            cap.launches = ops.COUNTER.launches - before
            ops.COUNTER.launches = before            # captured, not yet run
            self.cached[key] = cap
            self.captures += 1
        cap.graph.replay()
        self._done.record(stream)
        ops.COUNTER.launches += cap.launches
        self.replays += 1
        return cap

    @staticmethod
    def read(ticket) -> list[int]:
        """The ids a step launched with `keep` sampled: waits for that step only."""
        buf, event, B = ticket
        event.synchronize()
        return buf[:B].tolist()

    def host_tokens(self) -> list[int]:
        """The ids the last step sampled, on the host: waits for the step (its graph ends with the
        copy into pinned memory)."""
        self._done.synchronize()
        return self._last.host_tokens.tolist()

    def last_logits(self, n_requests: int, max_kv_len: int) -> torch.Tensor:
        return self.cached[self._key(n_requests, max_kv_len)].logits
