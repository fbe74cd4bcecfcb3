"""RMSNorm, fused with the residual add that precedes it."""
from __future__ import annotations

from ..kernels import ops
from .base import Norm, register_part
from .spec import PartSpec, TensorSpec


class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * w  (rust/engine/src/runner/model/qwen2/kernels.rs:546-582)."""

    @classmethod
    def tensors(cls, spec: PartSpec):
        return [TensorSpec(spec.prefix + "weight", (spec["hidden"],), init="norm")]

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.weight = self._weight(weights, "weight")
        self.eps = float(spec["eps"])

    def forward(self, x, rows=None):
        return ops.add_rmsnorm(x, self.weight, self.eps, rows=rows)

    def forward_add(self, x, delta, rows=None):
        if delta is not None and delta.dim() == 3:      # split-K partial products in 32-bit
            return ops.add_rmsnorm(x, self.weight, self.eps, partial=delta, rows=rows)
        return ops.add_rmsnorm(x, self.weight, self.eps, delta=delta, rows=rows)


register_part("norm", "rmsnorm", RMSNorm)
