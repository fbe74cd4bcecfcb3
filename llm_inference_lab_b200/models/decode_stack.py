"""The layers of a decode step as one persistent kernel.

A step in which every request brings one token runs the same small operators
layer after layer; launched one by one they cost more in launches than in work.
Where a model's layers are all of the shape the fused kernel knows (pre-norm
blocks of grouped-query attention with rotary encoding over heads of 64 or 128,
a gated SiLU feed-forward and RMS norms, in bfloat16), `DecodeStack` runs the
whole stack of layer calls for such a step as one cooperative kernel
(``csrc/kernels/decode_stack.cu``).  It is an arrangement of the same parts, not
another model: it reads the parts' own tensors and sizes, follows the
blueprint's run order (a layer named twice, a call that reads another call's
cache), and any model, layer or step it does not fit runs part by part as
before.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np
import torch

from ..kernels import ops
from ..parts.attention import GQAttention
from ..parts.base import CacheView, StepContext
from ..parts.block import PreNormBlock
from ..parts.mlp import GatedMLP
from ..parts.norm import RMSNorm
from ..parts.rope import Rope

MAX_TOKENS = 64     # what the kernel takes
EAGER_TOKENS = 16   # up to where it is the faster way to run a step that is launched kernel by kernel
PHASES = 5      # per layer call: q/k/v projection, attention, output projection, gate/up, down


def _fits(block, dtype) -> bool:
    if type(block) is not PreNormBlock or dtype != torch.bfloat16:
        return False
    m, f = block.mixer, block.ffn
    if type(m) is not GQAttention or type(f) is not GatedMLP or any(type(n) is not RMSNorm for n in block.norms):
        return False
    if type(m.position) is not Rope or m.position.rotary_dim != m.d or m.d not in (64, 128) or m.b_o is not None:
        return False
    hidden, inter = m.w_qkv.shape[1], f.w_down.shape[1]
    return hidden % 8 == 0 and inter % 8 == 0 and hidden <= 2048 and m.w_o.shape == (hidden, m.n_q * m.d)


def pick_slices(tiles: int, k_tiles: int, grid: int, rows: int, work_bytes: int) -> int:
    """Into how many slices of K a product of `tiles` output tiles is cut, so that the items (tile, slice)
    spread over `grid` CTAs: the number that makes the busiest CTA's share shortest, counting a fixed
    cost per item (operand, barriers, epilogue: about what three k-tiles of weights take to arrive);
    on a near tie the fewer slices; a slice's operand (`rows` tokens) must fit the work area."""
    best, best_cost = 0, 0.0
    for s in range(1, k_tiles + 1):
        per = -(-k_tiles // s)
        if (s - 1) * per >= k_tiles:
            continue                                  # an empty slice
        if per * rows * 128 > work_bytes:
            continue
        if per < 2 and s > 1 and k_tiles >= 2:
            continue
        cost = -(-tiles * s // grid) * (per + 3.0)
        if best == 0 or cost < 0.9 * best_cost:
            best, best_cost = s, cost
    return best


class DecodeStack:
    def __init__(self, blocks, order, dtype, device):
        self.blocks, self.order, self.device = blocks, order, device
        m, f = blocks[0].mixer, blocks[0].ffn
        self.d, self.n_q, self.n_kv = m.d, m.n_q, m.n_kv
        self.hidden, self.inter = m.w_qkv.shape[1], f.w_down.shape[1]
        self.scale = m.scale
        self.lib = ops.lib("decode_stack", {"LAB_HEAD_DIM": self.d})
        self.grid = int(self.lib.lab_decode_stack_grid())
        if self.grid <= 0:
            raise ops.KernelError("the decode stack kernel does not fit this device")
        self.work_bytes = int(self.lib.lab_decode_stack_work_bytes())
        self._layers: dict = {}       # cache tensors' addresses -> device array of the layer calls' parameters
        self._plans: dict = {}
        n_qd = self.n_q * self.d
        z = lambda *shape, dt=torch.bfloat16: torch.empty(shape, dtype=dt, device=device)  # noqa: E731
        self.qbuf, self.attn, self.act = z(MAX_TOKENS, n_qd), z(MAX_TOKENS, n_qd), z(MAX_TOKENS, self.inter)
        self.counters = torch.zeros((8192,), dtype=torch.int32, device=device)
        self.barrier = torch.zeros((64,), dtype=torch.int32, device=device)
        self.stamps = None            # set to an int64 tensor [5 * calls + 1] to have CTA 0 stamp every phase's start
        self.partial = None
        self.att_scratch = None
        ops.on_device_error(self._reset)

    @staticmethod
    def build(blocks, order, dtype, device) -> Optional["DecodeStack"]:
        """The fused stack for these layer calls, or None where a layer does not fit it."""
        if not blocks or not order or not all(_fits(b, dtype) for b in blocks) or len(order) > 1024:
            return None
        first = blocks[0]
        same = lambda b: (b.mixer.d, b.mixer.n_q, b.mixer.n_kv, b.mixer.w_qkv.shape, b.ffn.w_down.shape,  # noqa: E731
                          b.mixer.position.theta, b.mixer.scale)
        if any(same(b) != same(first) for b in blocks):
            return None
        stack = DecodeStack(blocks, order, dtype, device)
        return stack if stack._plan(MAX_TOKENS, 64) is not None else None

    def _reset(self) -> None:
        """After a wait ran out the barrier's words and the counters may be left mid-count."""
        self.counters.zero_()
        self.barrier.zero_()

    def serves(self, ctx: StepContext, caches) -> bool:
        """Pure decode steps of few tokens that are launched kernel by kernel.  Measured on a B200 at the
        Qwen2.5-0.5B sizes, batch 8: the stack takes 1.29 ms a step, the same layers part by part 0.80 ms
        when replayed from a CUDA graph (programmatic dependent launch overlaps each kernel's set-up with
        its predecessor, while the stack pays a grid-wide barrier and a pass through L2 for every
        reduction), but 2.8 ms when the host launches their 190 kernels one by one.  So a step that is
        being captured into a graph runs part by part, and an eager one of up to 16 tokens runs here."""
        return (ctx.max_q_len == 1 and 0 < ctx.n_tokens <= EAGER_TOKENS and ctx.n_tokens == ctx.n_requests
                and not torch.cuda.is_current_stream_capturing()
                and ctx.dtype == torch.bfloat16 and not ops.forced_plain() and len(ctx.groups) <= 4
                and all(caches[c.cache].k is not None for c in self.order))

    # ------------------------------------------------------------------------------------
    def _plan(self, T: int, bn: int):
        """Slices of K per product for steps of up to `bn` tokens."""
        plan = self._plans.get(bn)
        if plan is None:
            width = (self.n_q + 2 * self.n_kv) * self.d
            kt = lambda k: -(-k // 64)   # noqa: E731
            shapes = [(-(-width // 128), kt(self.hidden)), (-(-self.hidden // 128), kt(self.n_q * self.d)),
                      (-(-self.inter // 64), kt(self.hidden)), (-(-self.hidden // 128), kt(self.inter))]
            slices = [pick_slices(t, k, self.grid, bn, self.work_bytes) for t, k in shapes]
            if any(s == 0 for s in slices) or any(t > 1024 for t, _ in shapes):
                return None
            need = max(t * s for (t, _), s in zip(shapes, slices)) * 128 * bn
            plan = self._plans[bn] = (slices, need)
        return plan

    def _layer_params(self, caches: list[CacheView]) -> torch.Tensor:
        key = tuple((caches[c.cache].k.data_ptr(), caches[c.cache].v.data_ptr(), c.write) for c in self.order)
        dev = self._layers.get(key)
        if dev is None:
            size = int(self.lib.lab_decode_stack_layer_bytes())
            host = np.zeros((len(self.order), size), dtype=np.uint8)
            for i, call in enumerate(self.order):
                block, view = self.blocks[call.layer], caches[call.cache]
                m, f = block.mixer, block.ffn
                if view.k.dtype != torch.bfloat16 or not view.k.is_contiguous() or view.k.shape[1:] != \
                        (self.n_kv, view.k.shape[2], self.d):
                    raise ops.KernelError("the decode stack takes contiguous bfloat16 caches [pages, kv heads, page, d]")
                rc = self.lib.lab_decode_stack_layer(
                    ctypes.c_void_p(host[i].ctypes.data), ops._ptr(m.w_qkv), ops._ptr(m.w_o), ops._ptr(f.w_gate_up),
                    ops._ptr(f.w_down), ops._ptr(block.norms[0].weight), ops._ptr(block.norms[1].weight),
                    ops._ptr(m.b_qkv), ops._ptr(view.k), ops._ptr(view.v), self.hidden, self.n_q, self.n_kv, self.inter,
                    ctypes.c_float(block.norms[0].eps), ctypes.c_float(block.norms[1].eps), int(view.group),
                    int(m.window), int(bool(call.write and view.write)))
                if rc != 0:
                    raise ops.KernelError(f"decode stack: describing layer call {i} failed (CUDA error {rc})")
            dev = self._layers[key] = torch.from_numpy(host).to(self.device)
        return dev

    def run(self, x: torch.Tensor, ctx: StepContext, caches: list[CacheView], phases: Optional[tuple[int, int]] = None):
        """Runs the layer calls on the residual rows `x` [tokens, hidden] in place (`phases`: a range of
        the 5 * calls phases, for tests)."""
        T = ctx.n_tokens
        bn = 16 if T <= 16 else (32 if T <= 32 else 64)
        slices, need = self._plan(T, bn)
        if self.partial is None or self.partial.numel() < need:
            self.partial = torch.empty((need,), dtype=torch.float32, device=self.device)
        m_tiles = -(-(self.n_q // self.n_kv) // 16)
        items = T * self.n_kv * m_tiles
        span = ctx.max_kv_len
        keys_per_round = 128 if self.d == 64 else 96
        att_splits = int(max(1, min(8, self.grid // items, -(-span // keys_per_round))))
        att_need = T * self.n_q * att_splits * (self.d + 2)
        if self.att_scratch is None or self.att_scratch.numel() < att_need:
            self.att_scratch = torch.empty((max(att_need, 1 << 20),), dtype=torch.float32, device=self.device)
        att_acc = self.att_scratch
        att_ml = self.att_scratch[T * self.n_q * att_splits * self.d:]
        first = caches[self.order[0].cache]
        num_pages, _, page_size, _ = first.k.shape
        assert x.is_contiguous() and x.shape == (T, self.hidden) and x.dtype == torch.bfloat16
        table = self.blocks[0].mixer.position.table(ctx.row_pos, ctx.scratch)
        layers = self._layer_params(caches)
        groups = ctx.groups
        ptr_list = [layers, x, self.qbuf, self.attn, self.act, self.partial, att_acc, att_ml, self.counters,
                    self.barrier, table, ctx.q_start, ctx.kv_len, self.stamps]
        ptr_list += [g.row_slot for g in groups] + [g.block_table for g in groups]
        ptrs = (ctypes.c_void_p * len(ptr_list))(*[0 if t is None else t.data_ptr() for t in ptr_list])
        int_list = [T, bn, self.hidden, self.n_q, self.n_kv, self.inter, *slices, att_splits, page_size, num_pages,
                    len(groups)] + [g.block_table.shape[1] for g in groups]
        ints = (ctypes.c_int * len(int_list))(*int_list)
        lo, hi = phases if phases is not None else (0, PHASES * len(self.order))
        ops._check(self.lib.lab_decode_stack(ptrs, ints, len(self.order), lo, hi, ctypes.c_float(self.scale),
                                             ops._stream()), "decode_stack")
        return x
