"""Dense gated feed-forward."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import FeedForward, register_part
from .spec import PartSpec, TensorSpec


class GatedMLP(FeedForward):
    """down( act(x Wg^T) * (x Wu^T) ), no biases; act is SiLU
    (rust/engine/src/runner/model/qwen2/kernels.rs:1469-1486, engine.rs:1242-1293).
    Gate and up matrices are concatenated at load time; the activation and the product are
    the epilogue of their matrix product."""

    ACTS = ("silu",)

    @classmethod
    def tensors(cls, spec: PartSpec):
        h, i, p = spec["hidden"], spec["intermediate"], spec.prefix
        return [TensorSpec(p + "gate_proj.weight", (i, h)), TensorSpec(p + "up_proj.weight", (i, h)),
                TensorSpec(p + "down_proj.weight", (h, i))]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        if spec["act"] not in self.ACTS:
            raise ValueError(f"gated_mlp: activation {spec['act']!r} is not built (known: {self.ACTS})")
        self.w_gate_up = torch.cat([self._weight(weights, "gate_proj.weight"),
                                    self._weight(weights, "up_proj.weight")], dim=0).contiguous()
        self.w_down = self._weight(weights, "down_proj.weight").contiguous()

    def forward(self, x, ctx):
        act = ops.linear_gated(x, self.w_gate_up)
        return ops.linear(act, self.w_down, None, allow_partial=True)


register_part("feed_forward", "gated_mlp", GatedMLP)
