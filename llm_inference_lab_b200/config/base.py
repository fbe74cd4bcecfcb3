"""Typed model configuration: the common machinery.

A model family declares a dataclass whose fields are the keys of its own
``config.json``.  `ConfigField` metadata says which keys are required and how a
value is checked, so that an absent or ill-typed key is reported by name
instead of surfacing later as a shape error.  This mirrors the reference's
serde schema, where a key without a default is required
(rust/engine/src/runner/model/qwen2/engine.rs:197-216).
"""
from __future__ import annotations

import dataclasses
import json
import math
import os
from typing import Any, ClassVar


class ConfigError(ValueError):
    """A config.json that the engine refuses, with the key named."""


_MISSING = dataclasses.MISSING


def required(kind, check=None, doc=""):
    """A key that must be present in config.json."""
    return dataclasses.field(default=_MISSING, metadata={"kind": kind, "check": check, "doc": doc})


def optional(kind, default, check=None, doc=""):
    """A key with a default when config.json leaves it out."""
    if isinstance(default, (list, dict)):
        return dataclasses.field(default_factory=lambda: type(default)(default),
                                 metadata={"kind": kind, "check": check, "doc": doc})
    return dataclasses.field(default=default, metadata={"kind": kind, "check": check, "doc": doc})


def positive(name, value):
    if not (value > 0):
        raise ConfigError(f"config key {name!r} must be positive, got {value!r}")


def finite_positive(name, value):
    if not (isinstance(value, (int, float)) and math.isfinite(value) and value > 0):
        raise ConfigError(f"config key {name!r} must be finite and positive, got {value!r}")


def _coerce(name: str, kind, value):
    if value is None:
        return None
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            if isinstance(value, float) and value.is_integer():
                return int(value)
            raise ConfigError(f"config key {name!r} must be an integer, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config key {name!r} must be a number, got {value!r}")
        return float(value)
    if kind is bool:
        if not isinstance(value, bool):
            raise ConfigError(f"config key {name!r} must be true or false, got {value!r}")
        return value
    if kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config key {name!r} must be a string, got {value!r}")
        return value
    return value  # "any": lists, nested objects


@dataclasses.dataclass
class ModelConfig:
    """Base of every family's typed configuration."""

    #: the value ``architectures[0]`` of config.json that selects this family
    architecture: ClassVar[str] = ""

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "ModelConfig":
        values = {}
        for f in dataclasses.fields(cls):
            kind = f.metadata.get("kind", "any")
            if f.name in raw:
                value = _coerce(f.name, kind, raw[f.name])
            elif f.default is not _MISSING:
                value = f.default
            elif f.default_factory is not _MISSING:  # type: ignore[misc]
                value = f.default_factory()  # type: ignore[misc]
            else:
                raise ConfigError(
                    f"config.json of {cls.architecture or cls.__name__} lacks the required key {f.name!r}")
            check = f.metadata.get("check")
            if check is not None and value is not None:
                check(f.name, value)
            values[f.name] = value
        cfg = cls(**values)
        cfg.validate()
        return cfg

    @classmethod
    def from_json_file(cls, path: str) -> "ModelConfig":
        return cls.from_dict(read_config_json(path))

    def validate(self) -> None:  # relations between keys
        pass

    def to_dict(self) -> dict[str, Any]:
        out = {"architectures": [self.architecture]}
        out.update(dataclasses.asdict(self))
        return out

    def save(self, folder: str) -> None:
        os.makedirs(folder, exist_ok=True)
        with open(os.path.join(folder, "config.json"), "w") as fh:
            json.dump(self.to_dict(), fh, indent=2)


def read_config_json(path: str) -> dict[str, Any]:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path) as fh:
            raw = json.load(fh)
    except FileNotFoundError:
        raise ConfigError(f"no config.json at {path}") from None
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return raw


def read_generation_eos(model_dir: str) -> tuple[int, ...] | None:
    """End-of-sequence ids from an optional ``generation_config.json`` beside ``config.json``.

    The reference reads that file if it exists and lets its ``eos_token_id`` (one id or a
    list) replace the model configuration's single id
    (rust/engine/src/runner/loader.rs:199-205; rust/engine/src/runner/model/qwen2/engine.rs:403-407).
    Its other keys (do_sample, temperature, top_k, top_p, max_new_tokens) are per-request
    options there and are not taken from the file.  Returns None if the file is absent or
    names no id.
    """
    path = os.path.join(model_dir, "generation_config.json")
    if not os.path.exists(path):
        return None
    try:
        with open(path) as fh:
            raw = json.load(fh)
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from None
    if not isinstance(raw, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    eos = raw.get("eos_token_id")
    if eos is None:
        return None
    ids = [eos] if isinstance(eos, int) and not isinstance(eos, bool) else eos
    if not isinstance(ids, list) or not all(isinstance(t, int) and not isinstance(t, bool) and t >= 0 for t in ids):
        raise ConfigError(f"{path}: 'eos_token_id' must be a non-negative integer or a list of them")
    return tuple(ids)
