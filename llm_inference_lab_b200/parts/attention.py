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
        table_of = getattr(self.position, "table", None)
        if (table_of is not None and x.shape[0] > 128
                and ops.qkv_fusable(x, self.w_qkv, self.d, getattr(self.position, "rotary_dim", 0))):
            # One kernel: projection, bias, rotation of q and k from the step's table of cosines and
            # sines, k and v straight into their cache slots.  (Steps of few tokens keep the product
            # with K split over more CTAs and the rotation kernel that sums its parts: measured faster
            # there than nine CTAs that each walk the whole of K.)
            write = cache.write
            q = ops.qkv_rope_store(x, self.w_qkv, self.b_qkv, table_of(ctx.row_pos, ctx.scratch), group.row_slot,
                                   cache.k if write else None, cache.v if write else None, self.n_q, self.n_kv, self.d)
        else:
            # With few tokens the product may come back as split-K partial sums (bias not yet added), if
            # the position encoding takes them: it then sums them, adds the bias and rounds once.
            partial = bool(getattr(self.position, "takes_partials", False))
            qkv = ops.linear(x, self.w_qkv, self.b_qkv, allow_partial=partial)
            q = self.position.rotate_and_store(qkv, ctx.row_pos, group.row_slot, cache, self.n_q, self.n_kv, self.d,
                                               bias=self.b_qkv if qkv.dim() == 3 else None, scratch=ctx.scratch)
        attn = ops.attention(q, cache.k, cache.v, ctx, group, self.n_q, self.n_kv, self.d, self.window, self.scale)
        return ops.linear(attn, self.w_o, self.b_o, allow_partial=self.b_o is None)


register_part("mixer", "gqa_attention", GQAttention)
