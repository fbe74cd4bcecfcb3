"""Weights by tensor name.

The loader is given the list of tensors the model's parts want (`TensorSpec`)
and checks the whole folder against it before a single byte moves: tensors
that are wanted but absent, present but not wanted, or of another shape are
reported together in one `WeightsError`.  Stored precision is kept: bfloat16
stays bfloat16, a tensor stored in 32-bit stays 32-bit, float16 is widened to
float32 (exact; narrowing it to bfloat16 here would cost a 32-bit engine three
bits of every weight), float64 is narrowed to float32, integer tables become
int32.  A part then casts what its kernels need (a float32 engine
widens everything; a bfloat16 engine narrows matrices that were stored wider,
round to nearest even) unless the tensor is marked ``keep_f32``.
Names and shapes are the checkpoint's own; nothing is renamed
(rust/engine/src/runner/model/qwen2/engine.rs:291-400, 2223-2241;
dtype conversion: rust/engine/src/runner/loader.rs:57-133).
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..parts.spec import TensorSpec
from .safetensors_io import ModelFiles, SafetensorsError


class WeightsError(ValueError):
    """The folder does not hold the tensors the model wants."""

    def __init__(self, model_dir, missing, unexpected, wrong_shape):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        lines = [f"weights in {model_dir} do not fit the model:"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} is {list(got)}, wanted {list(want)}" for n, got, want in self.wrong_shape))
        super().__init__("\n".join(lines))


def kept_dtype(stored: torch.dtype) -> torch.dtype:
    if stored == torch.bfloat16:
        return torch.bfloat16
    if stored in (torch.float16, torch.float32, torch.float64):
        return torch.float32
    if stored in (torch.int64, torch.int32, torch.int16, torch.int8, torch.uint8, torch.bool):
        return torch.int32
    raise SafetensorsError(f"unsupported stored dtype {stored}")


def check_folder(files: ModelFiles, specs: Sequence[TensorSpec], model_dir: str, optional=()) -> None:
    wanted = {s.name: s for s in specs}
    present = set(files.names())
    missing = sorted(n for n in wanted if n not in present)
    unexpected = sorted(n for n in present if n not in wanted and n not in optional)
    wrong = [(n, files.shape(n), wanted[n].shape) for n in sorted(wanted)
             if n in present and tuple(files.shape(n)) != tuple(wanted[n].shape)]
    if missing or unexpected or wrong:
        raise WeightsError(model_dir, missing, unexpected, wrong)


def load_weights(model_dir: str, specs: Sequence[TensorSpec], device, optional=()) -> dict[str, torch.Tensor]:
    """Check the folder, then bring every wanted tensor to `device` in its kept dtype."""
    files = ModelFiles(model_dir)
    check_folder(files, specs, model_dir, optional)
    out = {}
    for spec in specs:
        t = files.get(spec.name)
        out[spec.name] = t.to(device=device, dtype=kept_dtype(t.dtype), copy=True)
    return out
