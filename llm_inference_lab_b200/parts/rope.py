"""Rotary position encoding (split-half pairing) with a theta parameter."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import PositionEncoding, register_part


class Rope(PositionEncoding):
    """inv_freq[i] = theta^(-2i/rotary_dim) held in 32-bit; the angle pos * inv_freq is formed
    in 32-bit on the device (rust/engine/src/runner/model/qwen2/engine.rs:304-311, kernels.rs:587-631).
    The rotation of q and k is fused with the write of k and v into the cache pages; where the mixer's
    fused projection can take the rotation into its epilogue, it asks for the step's `table`."""
    takes_partials = True

    def __init__(self, spec, weights, dtype, device):
        super().__init__(spec, weights, dtype, device)
        self.rotary_dim = int(spec["rotary_dim"])
        i = np.arange(self.rotary_dim // 2, dtype=np.float64)
        inv = np.power(float(spec["theta"]), -2.0 * i / self.rotary_dim).astype(np.float32)
        self.theta = float(spec["theta"])
        self.inv_freq = torch.from_numpy(inv).to(device)

    def table(self, positions, scratch):
        """(cos, sin) of every row's angles [tokens, rotary_dim / 2, 2] in 32-bit, formed once per step
        and shared by every layer that rotates alike."""
        key = ("rope_table", self.rotary_dim, self.theta, positions.data_ptr())
        table = scratch.get(key)
        if table is None:
            table = scratch[key] = ops.rope_table(positions, self.inv_freq)
        return table

    def encode(self, qkv, positions, n_q, n_kv, head_dim):
        ops.rope_kv_write(qkv, positions, self.inv_freq, self.rotary_dim, None, None, None, n_q, n_kv, head_dim)

    def rotate_and_store(self, qkv, positions, slots, cache, n_q, n_kv, head_dim, bias=None, scratch=None):
        write = cache is not None and cache.write
        if (scratch is not None and qkv.dim() == 2 and qkv.dtype == torch.bfloat16 and qkv.shape[0] >= 128
                and self.rotary_dim % 16 == 0 and self.rotary_dim > 0 and head_dim % 8 == 0):
            # Many rows: the rotation runs on 16-byte vectors with cos and sin from the step's table.
            table = self.table(positions, scratch)
            return ops.rope_kv_write_table(qkv, table, self.rotary_dim, slots if write else None,
                                           cache.k if write else None, cache.v if write else None, n_q, n_kv,
                                           head_dim)
        return ops.rope_kv_write(qkv, positions, self.inv_freq, self.rotary_dim, slots if write else None,
                                 cache.k if write else None, cache.v if write else None, n_q, n_kv, head_dim,
                                 bias=bias)


class NoPosition(PositionEncoding):
    """No encoding: q and k are used as projected; k and v are still written to the cache (the
    framework's store does that)."""

    def encode(self, qkv, positions, n_q, n_kv, head_dim):
        pass


register_part("position", "rope", Rope)
register_part("position", "none", NoPosition)
