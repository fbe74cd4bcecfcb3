"""One registry from an architecture's name to its model.

``config.json`` names its architecture in ``architectures[0]``; the registry
maps that name to a typed configuration class and to the function that turns
the configuration into a `ModelBlueprint`.  The reference has no registry (its
engine type is picked at compile time, rust/engine/examples/qwen2.rs:78-83);
the fallback on ``model_type`` keeps its check of that key (engine.rs:260).
"""
from __future__ import annotations

import dataclasses
from typing import Callable

from .config.base import ConfigError, ModelConfig, read_config_json
from .parts.spec import ModelBlueprint


@dataclasses.dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    blueprint: Callable[[ModelConfig], ModelBlueprint]
    model_types: tuple[str, ...] = ()


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, blueprint, model_types=()) -> Architecture:
    arch = Architecture(name, config_class, blueprint, tuple(model_types))
    _ARCHITECTURES[name] = arch
    return arch


def architectures() -> tuple[str, ...]:
    return tuple(sorted(_ARCHITECTURES))


def resolve(raw_config: dict) -> Architecture:
    """The architecture a raw config.json names."""
    names = raw_config.get("architectures")
    if isinstance(names, list) and names:
        if names[0] in _ARCHITECTURES:
            return _ARCHITECTURES[names[0]]
        raise ConfigError(f"architecture {names[0]!r} is not registered; known: {', '.join(architectures())}")
    model_type = raw_config.get("model_type")
    for arch in _ARCHITECTURES.values():
        if model_type in arch.model_types:
            return arch
    raise ConfigError("config.json names no architecture: 'architectures' is absent and "
                      f"'model_type' is {model_type!r}; known: {', '.join(architectures())}")


def load_config(model_dir: str) -> tuple[Architecture, ModelConfig]:
    raw = read_config_json(model_dir)
    arch = resolve(raw)
    return arch, arch.config_class.from_dict(raw)


def _register_builtin() -> None:
    from .config.qwen2 import Qwen2Config, qwen2_blueprint
    register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_blueprint, model_types=("qwen2",))


_register_builtin()
