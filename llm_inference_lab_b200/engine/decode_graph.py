"""Decode steps replayed from CUDA graphs.

A step in which every request brings exactly one token has the same launches
every time; only the metadata (positions, cache slots, block tables, lengths)
and the token ids change.  Such a step is captured once per (batch size, context
bucket) into a CUDA graph over fixed buffers; later steps copy their metadata
into those buffers and replay the graph.  The sampled tokens stay in a device
buffer that is also the next step's input, so a run of decode steps needs no
copy back to the host unless the caller wants the tokens.

Batch sizes are rounded up to a few sizes (`padded_batch`): the rows beyond
the real ones belong to requests of length zero, whose keys and values go
nowhere and whose attention reads nothing, so a batch that shrinks request by
request, as in continuous batching, walks through a handful of graphs instead
of one per size.  All graphs share one memory pool: they never run side by
side, and nothing a step leaves in the pool is read later (the sampled ids live
in buffers of their own).

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
    rows_cap: int               # rows of the captured step (the padded batch size)
    buf: torch.Tensor           # one int32 device buffer: [temps | seeds | metadata | tokens], each rows_cap wide
    dev: torch.Tensor           # view: the int32 metadata
    tokens: torch.Tensor        # view [rows_cap] int32: input ids of the step, overwritten with the sampled ids
    temps: torch.Tensor         # view [rows_cap] float32
    seeds: torch.Tensor         # view [rows_cap] int32
    rows: torch.Tensor          # [rows_cap] int32: 0..rows_cap-1, the rows whose logits are computed
    host_tokens: torch.Tensor   # [rows_cap] int32 in pinned memory: the sampled ids, copied by the graph itself
    launches: int = 0           # kernels the graph holds


def padded_batch(n: int) -> int:
    """The batch size a step of `n` requests is captured at: 1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128,
    then multiples of 64."""
    for size in (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128):
        if n <= size:
            return size
    return -(-n // 64) * 64


class DecodeGraphs:
    MAX_CACHED = 48
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
        self._pool = None                     # the memory pool all graphs share
        self._ring, self._ring_at = [], 0     # pinned buffers for the ids of steps launched with `keep`
        self._done = torch.cuda.Event()     # recorded after every replay

    # ------------------------------------------------------------------------------------
    def _key(self, n_requests: int, max_kv_len: int):
        cap = min(padded_batch(n_requests), max(self.engine.max_requests, n_requests))
        return (cap, max(256, 1 << (int(max_kv_len) - 1).bit_length()))

    def _context(self, cap: _Captured, kv_bucket: int) -> StepContext:
        eng, n = self.engine, cap.rows_cap
        widths = [eng.max_blocks] * len(eng.group_windows)
        return eng._context(cap.dev, cap.layout, widths, n, n, [1] * n, [kv_bucket] * n, [], cap.tokens)

    def _run(self, cap: _Captured, ctx: StepContext) -> None:
        # What the parts share within a step (the table of rotation angles, for one) is formed anew in
        # every run: the run that is captured must hold the kernels that fill it, not find what the
        # warm-up run before it left.
        ctx.scratch.clear()
        # position of the token being drawn = tokens held after this step; the head picks the tokens
        # itself, so a decode step writes no logits
        self.engine.model.forward(ctx, self.engine.views, cap.rows, pick=(cap.temps, cap.seeds, ctx.kv_len, cap.tokens))
        cap.host_tokens.copy_(cap.tokens, non_blocking=True)   # part of the graph: no launch of its own later

    def _new_capture(self, key):
        eng = self.engine
        n, kv_bucket = key
        n_groups = len(eng.group_windows)
        layout = eng.cache.layout(n, n, [eng.max_blocks] * n_groups)
        # Temperatures and seeds before the metadata, tokens after it: whatever a step brings from
        # the host is one contiguous piece, and one copy.
        buf = torch.zeros((3 * n + layout.total,), dtype=torch.int32, device=eng.device)
        at = 2 * n
        cap = _Captured(graph=torch.cuda.CUDAGraph(), layout=layout, rows_cap=n, buf=buf,
                        dev=buf[at: at + layout.total], tokens=buf[at + layout.total: at + layout.total + n],
                        temps=buf[0: n].view(torch.float32), seeds=buf[n: 2 * n],
                        rows=torch.arange(n, dtype=torch.int32, device=eng.device),
                        host_tokens=torch.zeros((n,), dtype=torch.int32, pin_memory=True))
        return cap, self._context(cap, kv_bucket)

    # ------------------------------------------------------------------------------------
    def step(self, requests: Sequence[int], tokens: Optional[Sequence[int]] = None,
             temps: Optional[Sequence[float]] = None, seeds: Optional[Sequence[int]] = None,
             reserved: bool = False, keep: bool = False):
        """One decode step for `requests` (each brings one token).  `tokens` are the input ids
        on the host; None means: the ids the previous step of the same requests sampled, which
        are still on the device.  `temps` and `seeds` None means: as in the previous step of the
        same requests (greedy if there was none).  Returns the device buffer [B] of sampled ids
        (valid until the next step); with `keep`, a ticket for `read` instead: the ids are also copied
        into a pinned buffer of their own, so that they can be read after later steps have been
        launched."""
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
            if not self._ring or B > self._ring[0][0].numel():
                # (buffers that were outgrown are dropped once their tickets are: a ticket holds its buffer)
                size = max(self.MAX_KEPT_BATCH, eng.max_requests, B)
                self._ring = [(torch.zeros((size,), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                              for _ in range(4)]
                self._ring_at = 0
            buf, event = self._ring[self._ring_at]
            self._ring_at = (self._ring_at + 1) % len(self._ring)
            buf[:B].copy_(cap.tokens[:B], non_blocking=True)
            event.record(ops.current_stream())
            return (buf, event, B)
        return cap.tokens[:B]

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
        n = cap.rows_cap
        st = eng._next_staging()
        n_meta = cap.layout.total
        host = st["np"]
        # rows beyond the real ones: requests of length zero (their keys go nowhere, they read none)
        eng.cache.pack(pairs, cap.layout, host[2 * n:], n, n)
        lo, hi = 2 * n, 2 * n + n_meta
        moved = cap is not self._last
        if tokens is not None:
            host[hi: hi + B] = np.asarray(tokens, dtype=np.int32)
            host[hi + B: hi + n] = 0
            hi += n
        elif moved:
            # the previous step of this batch ran from another graph (its context outgrew a bucket):
            # the ids it sampled move over on the device
            cap.tokens[:B].copy_(self._last.tokens[:B], non_blocking=True)
        if temps is not None:
            host[0: 2 * n] = 0
            host[0: B].view(np.float32)[:] = np.asarray(list(temps), dtype=np.float32)
            host[n: n + B] = np.asarray([s & 0x7FFFFFFF for s in seeds], dtype=np.int32)
            lo = 0
        elif same_batch and moved:
            # ... and so do the temperatures and seeds, which live in each graph's own buffer
            last = self._last
            cap.temps[:B].copy_(last.temps[:B], non_blocking=True)
            cap.seeds[:B].copy_(last.seeds[:B], non_blocking=True)
        elif not same_batch:
            host[0: 2 * n] = 0          # nobody said otherwise: greedy
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
            if self._pool is None:
                self._pool = torch.cuda.graph_pool_handle()
            before = ops.COUNTER.launches
            with torch.cuda.graph(cap.graph, pool=self._pool):
                self._run(cap, ctx)
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
        return self._last.host_tokens[: len(self._last_requests)].tolist()
