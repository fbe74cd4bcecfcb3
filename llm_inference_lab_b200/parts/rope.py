"""Rotary position encoding (split-half pairing) with a theta parameter."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import PositionEncoding, register_part


class Rope(PositionEncoding):
    """inv_freq[i] = theta^(-2i/rotary_dim) held in 32-bit; the angle pos * inv_freq is formed
    in 32-bit on the device (rust/engine/src/runner/model/qwen2/engine.rs:304-311, kernels.rs:587-631).
    The rotation of q and k is fused with the write of k and v into the cache pages."""

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.rotary_dim = int(spec["rotary_dim"])
        i = np.arange(self.rotary_dim // 2, dtype=np.float64)
        inv = np.power(float(spec["theta"]), -2.0 * i / self.rotary_dim).astype(np.float32)
        self.theta = float(spec["theta"])
        self.inv_freq = torch.from_numpy(inv).to(device)
        # (inverse frequencies, rotary width): lets a mixer hand the rotation to a fused kernel
        self.rotary = (self.inv_freq, self.rotary_dim)

    def rotate_and_store(self, qkv, positions, slots, cache, n_q, n_kv, head_dim, bias=None, scratch=None):
        write = cache is not None and cache.write
        if (scratch is not None and qkv.dim() == 2 and qkv.dtype == torch.bfloat16 and qkv.shape[0] >= 128
                and self.rotary_dim % 16 == 0 and self.rotary_dim > 0 and head_dim % 8 == 0):
            # Many rows: cos and sin are formed once per step (shared by every layer that rotates
            # alike) and the rotation runs on 16-byte vectors.
            key = ("rope_table", self.rotary_dim, self.theta, positions.data_ptr())
            table = scratch.get(key)
            if table is None:
                table = scratch[key] = ops.rope_table(positions, self.inv_freq)
            return ops.rope_kv_write_table(qkv, table, self.rotary_dim, slots if write else None,
                                           cache.k if write else None, cache.v if write else None, n_q, n_kv,
                                           head_dim)
        return ops.rope_kv_write(qkv, positions, self.inv_freq, self.rotary_dim, slots if write else None,
                                 cache.k if write else None, cache.v if write else None, n_q, n_kv, head_dim,
                                 bias=bias)


class NoPosition(PositionEncoding):
    """No encoding: q and k are used as projected; k and v are still written to the cache."""

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.inv_freq = torch.zeros((0,), dtype=torch.float32, device=device)
        self.rotary = (self.inv_freq, 0)

    def rotate_and_store(self, qkv, positions, slots, cache, n_q, n_kv, head_dim, bias=None, scratch=None):
        write = cache is not None and cache.write
        return ops.rope_kv_write(qkv, positions, self.inv_freq, 0, slots if write else None,
                                 cache.k if write else None, cache.v if write else None, n_q, n_kv, head_dim,
                                 bias=bias)


register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
