"""Reading and writing safetensors files, without any helper library.

Layout of a file: an 8-byte little-endian header length N, N bytes of JSON
(``name -> {dtype, shape, data_offsets: [begin, end]}`` plus an optional
``__metadata__``), then the tensors' bytes.  A model folder holds either one
``model.safetensors`` or a ``model.safetensors.index.json`` whose
``weight_map`` names the shard of every tensor; a broken index is an error and
never falls back to the single file (rust/engine/src/runner/loader.rs:151-192).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Iterable

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One memory-mapped safetensors file; tensors are views of the mapping."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except FileNotFoundError:
            raise SafetensorsError(f"weight file not found: {path}") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._fh.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} exceeds the file")
        try:
            header = json.loads(self._fh.read(hlen))
        except json.JSONDecodeError as exc:
            raise SafetensorsError(f"{path}: header is not JSON: {exc}") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: dict[str, dict] = {}
        for name, info in header.items():
            dtype = info.get("dtype")
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dtype!r}")
            begin, end = info["data_offsets"]
            shape = tuple(int(s) for s in info["shape"])
            numel = 1
            for s in shape:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[dtype]).element_size()
            if end - begin != want or self._base + end > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} holds {end - begin} bytes, its shape {shape} wants {want}")
            self.entries[name] = {"dtype": _DTYPES[dtype], "shape": shape, "begin": begin, "numel": numel}

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name]["shape"]

    def get(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e["numel"] == 0:
            return torch.empty(e["shape"], dtype=e["dtype"])
        with warnings.catch_warnings():
            # The mapping is read-only on purpose; every consumer copies (to the device or to a cast).
            warnings.simplefilter("ignore", UserWarning)
            t = torch.frombuffer(self._map, dtype=e["dtype"], count=e["numel"], offset=self._base + e["begin"])
        return t.reshape(e["shape"])


class ModelFiles:
    """All tensors of a model folder, by name, across shards."""

    def __init__(self, model_dir: str):
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: dict[str, SafetensorsFile] = {}
        self._where: dict[str, str] = {}
        if os.path.exists(index):
            try:
                with open(index) as fh:
                    weight_map = json.load(fh)["weight_map"]
            except (json.JSONDecodeError, KeyError, TypeError) as exc:
                raise SafetensorsError(f"{index}: broken index ({exc!r})") from None
            for name, shard in weight_map.items():
                if (not isinstance(shard, str) or os.path.basename(shard) != shard
                        or not shard.endswith(".safetensors")):
                    raise SafetensorsError(f"{index}: shard name {shard!r} is not a plain *.safetensors file name")
                if shard not in self._files:
                    self._files[shard] = SafetensorsFile(os.path.join(model_dir, shard))
                if name not in self._files[shard].entries:
                    raise SafetensorsError(f"{index}: tensor {name!r} is not in shard {shard}")
                self._where[name] = shard
        elif os.path.exists(single):
            self._files["model.safetensors"] = SafetensorsFile(single)
            for name in self._files["model.safetensors"].names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"no model.safetensors (or index) in {model_dir}")

    def names(self) -> list[str]:
        return list(self._where)

    def shape(self, name: str) -> tuple[int, ...]:
        return self._files[self._where[name]].shape(name)

    def get(self, name: str) -> torch.Tensor:
        if name not in self._where:
            raise SafetensorsError(f"tensor {name!r} not found")
        return self._files[self._where[name]].get(name)


def save_file(tensors: dict[str, torch.Tensor], path: str, metadata: dict[str, str] | None = None) -> None:
    """Write CPU tensors to one safetensors file, names in sorted order."""
    header: dict[str, object] = {}
    if metadata:
        header["__metadata__"] = metadata
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} of tensor {name!r}")
        # a view of the tensor's own bytes: nothing is copied before the write
        raw = memoryview(t.reshape(-1).view(torch.uint8).numpy()) if t.numel() else memoryview(b"")
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + raw.nbytes]}
        offset += raw.nbytes
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((8 - len(text) % 8) % 8)
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)
