"""Token embedding and output head."""
from __future__ import annotations

from ..kernels import ops
from .base import Embedding, Head, register_part
from .spec import PartSpec, TensorSpec


class TokenEmbedding(Embedding):
    """x[t] = table[id_t], no scaling (rust/engine/src/runner/model/qwen2/kernels.rs:46-57)."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec.prefix + "weight", (spec["vocab"], spec["hidden"]), init="table")]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.table = self._weight(weights, "weight").contiguous()
        weights[spec.prefix + "weight"] = self.table   # a tied head shares this storage

    def forward(self, token_ids):
        return ops.embed(token_ids, self.table)


class LinearHead(Head):
    """logits = x W^T in 32-bit, no bias; W is the embedding table when tied
    (rust/engine/src/runner/model/qwen2/engine.rs:299-303, 1312-1319)."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        if spec.get("tied_to"):
            return []
        return [TensorSpec(spec.prefix + "weight", (spec["vocab"], spec["hidden"]))]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        tied = spec.get("tied_to")
        w = weights[tied] if tied else weights[spec.prefix + "weight"]
        self.weight = (w if w.dtype == dtype else w.to(dtype)).contiguous()

    def forward(self, x):
        return ops.linear(x, self.weight, None, out_f32=True)

    def pick(self, x, temperature, seeds, positions, out=None):
        # In one pass where the tensor-core product serves: the [rows, vocab] logits are never written.
        if ops.head_pick_fusable(x, self.weight):
            return ops.head_pick(x, self.weight, temperature, seeds, positions, out=out)
        return super().pick(x, temperature, seeds, positions, out=out)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
