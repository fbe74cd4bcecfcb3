"""Arrangements of a mixer and a feed-forward around the residual stream."""
from __future__ import annotations

from ..profiling import scoped_range
from .base import Block, register_part


class PreNormBlock(Block):
    """r = x + mixer(norm1(x)); out = r + ffn(norm2(r))
    (rust/engine/src/runner/model/qwen2/engine.rs:1216-1296).

    The add that closes a sub-layer is fused with the norm that opens the next one, so the
    block hands its last product to the next block (or the final norm) as `pending`.
    """
    n_norms = 2

    def forward(self, x, pending, ctx, cache):
        with scoped_range(self.mixer_range):
            h = self.norms[0].forward_add(x, pending)
            a = self.mixer.forward(h, ctx, cache)
        with scoped_range(self.ffn_range):
            h = self.norms[1].forward_add(x, a)
            return x, self.ffn.forward(h, ctx)


register_part("block", "prenorm", PreNormBlock)
