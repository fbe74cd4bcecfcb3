"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import CacheView, Mixer, StepContext, lookup, register_part
from .spec import PagedKV, PartSpec, TensorSpec


class GQAttention(Mixer):
    """q/k/v projections (optional bias), position encoding of q and k, attention of every
    row over its request's cache (causal, optionally the last `window` keys only), output
    projection.  Sizes, bias flags, window and position encoding are parameters.

    Formulas: rust/engine/src/runner/model/qwen2/engine.rs:1133-1214 (projections, rotation),
    1072-1115 (cache write, attention), 1225-1232 (output projection); kv head of query
    head h is h // (n_heads / n_kv_heads) (engine.rs:1589-1617).
    The three projection matrices are concatenated once at load time, so that one matrix
    product yields q, k and v.
    """

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, nq, nkv, d = spec["hidden"], spec["n_heads"], spec["n_kv_heads"], spec["head_dim"]
        p = spec.prefix
        out = [TensorSpec(p + "q_proj.weight", (nq * d, h)), TensorSpec(p + "k_proj.weight", (nkv * d, h)),
               TensorSpec(p + "v_proj.weight", (nkv * d, h)), TensorSpec(p + "o_proj.weight", (h, nq * d))]
        if spec["qkv_bias"]:
            out += [TensorSpec(p + "q_proj.bias", (nq * d,), init="bias"),
                    TensorSpec(p + "k_proj.bias", (nkv * d,), init="bias"),
                    TensorSpec(p + "v_proj.bias", (nkv * d,), init="bias")]
        if spec.get("out_bias"):
            out.append(TensorSpec(p + "o_proj.bias", (h,), init="bias"))
        return out

    @classmethod
    def cache_need(cls, spec: PartSpec):
        return PagedKV(spec["n_kv_heads"], spec["head_dim"], int(spec.get("window") or 0))

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.n_q, self.n_kv, self.d = spec["n_heads"], spec["n_kv_heads"], spec["head_dim"]
        if self.n_q % self.n_kv:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.window = int(spec.get("window") or 0)
        self.scale = 1.0 / math.sqrt(self.d)
        w = lambda n: self._weight(weights, n)  # noqa: E731
        self.w_qkv = torch.cat([w("q_proj.weight"), w("k_proj.weight"), w("v_proj.weight")], dim=0).contiguous()
        self.b_qkv = None
        if spec["qkv_bias"]:
            self.b_qkv = torch.cat([w("q_proj.bias"), w("k_proj.bias"), w("v_proj.bias")], dim=0).contiguous()
        self.w_o = w("o_proj.weight").contiguous()
        self.b_o = w("o_proj.bias") if spec.get("out_bias") else None
        pos = spec["position"]
        self.position = lookup("position", pos.kind)(pos, weights, dtype, device)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        group = ctx.groups[cache.group]
        # With few tokens the product may come back as split-K partial sums (bias not yet added);
        # the position encoding then sums them, adds the bias and rounds once.
        qkv = ops.linear(x, self.w_qkv, self.b_qkv, allow_partial=True)
        rotary = getattr(self.position, "rotary", None)
        if (ops.FUSE_DECODE_ATTENTION and ctx.max_q_len == 1 and cache.write and rotary is not None
                and ops.decode_fusable(qkv.dtype if qkv.dim() == 2 else cache.k.dtype, self.d, self.n_q, self.n_kv)):
            # Every request brings one token: rotation, cache write and attention run as one kernel.
            attn = ops.attention_decode_fused(
                qkv, self.b_qkv if qkv.dim() == 3 else None, rotary[0], rotary[1], group.row_slot, cache.k, cache.v,
                ctx.q_start, ctx.kv_len, group.block_table, ctx.n_requests, ctx.max_kv_len, self.n_q, self.n_kv,
                self.d, self.window, self.scale)
            return ops.linear(attn, self.w_o, self.b_o, allow_partial=self.b_o is None)
        q = self.position.rotate_and_store(qkv, ctx.row_pos, group.row_slot, cache, self.n_q, self.n_kv, self.d,
                                           bias=self.b_qkv if qkv.dim() == 3 else None, scratch=ctx.scratch)
        attn = ops.attention(q, cache.k, cache.v, ctx, group, self.n_q, self.n_kv, self.d, self.window, self.scale)
        return ops.linear(attn, self.w_o, self.b_o, allow_partial=self.b_o is None)


register_part("mixer", "gqa_attention", GQAttention)
