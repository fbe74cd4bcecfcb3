"""Per-request sampling options and the on-GPU pick of the next token.

Option names follow the reference's `SamplingConfig = GenerationConfig`
(rust/engine/src/runner/loader.rs:30-44): ``do_sample``, ``temperature``,
``top_k``, ``top_p``, ``max_new_tokens`` (default 1), ``eos_token_id`` (one id
or several).  The reference accepts pure greedy only and refuses the rest
(rust/engine/src/runner/model_runner.rs:612-625); this engine adds temperature
sampling with a seed, and still refuses ``top_k`` / ``top_p``.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence, Union

import torch

from ..kernels import ops


@dataclasses.dataclass
class SamplingConfig:
    max_new_tokens: int = 1
    do_sample: bool = False
    temperature: Optional[float] = None
    top_k: Optional[int] = None
    top_p: Optional[float] = None
    seed: int = 0
    eos_token_id: Union[None, int, Sequence[int]] = None    # overrides the model's own list
    ignore_eos: bool = False

    def validate(self) -> None:
        if self.top_k is not None or self.top_p is not None:
            raise ValueError("only greedy and temperature sampling are supported: top_k / top_p are not built")
        if self.max_new_tokens < 0:
            raise ValueError("max_new_tokens must not be negative")
        if self.temperature is not None and self.temperature < 0:
            raise ValueError("temperature must not be negative")

    def effective_temperature(self) -> float:
        """0 means greedy.  A temperature only takes effect with do_sample, as in generation configs."""
        if self.do_sample and self.temperature is None:
            return 1.0
        if self.temperature is None or not self.do_sample:
            return 0.0
        return float(self.temperature)

    def eos_ids(self, model_eos: Sequence[int]) -> list[int]:
        if self.eos_token_id is None:
            return list(model_eos)
        if isinstance(self.eos_token_id, int):
            return [self.eos_token_id]
        return [int(t) for t in self.eos_token_id]


class Sampler:
    """Picks one token per row of 32-bit logits on the GPU (`csrc/kernels/sampling.cu`)."""

    def __init__(self, device):
        self.device = device

    def pick(self, logits: torch.Tensor, temperatures: Sequence[float], seeds: Sequence[int],
             positions: Sequence[int]) -> list[int]:
        rows = logits.shape[0]
        if any(t > 0 for t in temperatures):
            meta = torch.tensor([list(temperatures)], dtype=torch.float32).to(self.device, non_blocking=True)
            ints = torch.tensor([[s & 0x7FFFFFFF for s in seeds], list(positions)], dtype=torch.int32).to(
                self.device, non_blocking=True)
            out = ops.sample(logits, meta[0], ints[0], ints[1])
        else:
            out = ops.sample(logits)
        tokens = self.check(out.cpu().tolist(), logits.shape[1])
        assert len(tokens) == rows
        return tokens

    def device_args(self, temperatures: Sequence[float], seeds: Sequence[int], positions: Sequence[int]):
        """(temperatures, seeds, positions) on the device for a step that picks its own tokens
        (`Engine.step(..., pick=...)`); three Nones when every row is greedy."""
        if not any(t > 0 for t in temperatures):
            return (None, None, None)
        meta = torch.tensor([list(temperatures)], dtype=torch.float32).to(self.device, non_blocking=True)
        ints = torch.tensor([[s & 0x7FFFFFFF for s in seeds], list(positions)], dtype=torch.int32).to(
            self.device, non_blocking=True)
        return (meta[0], ints[0], ints[1])

    @staticmethod
    def check(tokens: list[int], vocab: int) -> list[int]:
        """A row without any finite candidate comes back as INT32_MAX (sampling.cu)."""
        for r, t in enumerate(tokens):
            if not 0 <= t < vocab:
                raise RuntimeError(f"row {r}: non-finite logits or invalid argmax")
        return tokens
