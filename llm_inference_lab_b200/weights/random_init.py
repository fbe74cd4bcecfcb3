"""Random-weights mode: a model folder from a configuration and a seed.

The reference makes random models only inside its tests
(rust/engine/src/runner/model/qwen2/engine.rs:2360-2454); here it is a mode of
the loader, so benchmarks and tests run without a checkpoint.  Every tensor
draws from its own stream keyed by (seed, CRC32 of its name), so the values do
not depend on the order or on which other tensors exist.
"""
from __future__ import annotations

import os
import zlib
from concurrent.futures import ThreadPoolExecutor
from typing import Sequence

import numpy as np
import torch

from ..parts.spec import TensorSpec
from .safetensors_io import save_file


def random_tensor(spec: TensorSpec, seed: int, std: float, norm_std: float, scales: dict[str, float]) -> torch.Tensor:
    rng = np.random.default_rng([seed & 0xFFFFFFFF, zlib.crc32(spec.name.encode())])
    values = rng.standard_normal(size=spec.shape, dtype=np.float32)
    # in place: a model of billions of values is made of tensors of hundreds of megabytes
    if spec.init == "norm":
        values *= np.float32(norm_std)
        values += np.float32(1.0)
    else:
        values *= np.float32(std)
    for pattern, scale in scales.items():
        if pattern in spec.name:
            values *= np.float32(scale)
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32))


def write_random_model(config, folder: str, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                       std: float = 0.02, norm_std: float = 0.1, scales: dict[str, float] | None = None) -> str:
    """Write ``config.json`` and ``model.safetensors`` for `config` under `folder`.

    `scales` multiplies tensors whose name contains a key, e.g. ``{"q_proj.weight": 8}``
    to make attention peaky in tests.
    """
    from ..models.builder import expected_tensors
    from ..registry import resolve

    arch = resolve(config.to_dict())
    specs: Sequence[TensorSpec] = expected_tensors(arch.blueprint(config))

    def make(spec: TensorSpec) -> torch.Tensor:
        t = random_tensor(spec, seed, std, norm_std, scales or {})
        return t if spec.keep_f32 else t.to(dtype)

    # Every tensor has a stream of its own, so they can be drawn side by side (NumPy's generator
    # releases the interpreter lock); the values do not depend on the number of threads.
    with ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as pool:
        tensors = dict(zip((spec.name for spec in specs), pool.map(make, specs)))
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt", "seed": str(seed)})
    return folder
