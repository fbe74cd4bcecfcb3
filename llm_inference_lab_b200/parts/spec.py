"""Descriptions of parts: what a model is made of, as data.

An architecture turns its typed configuration into a `ModelBlueprint`: the
embedding, a list of layers (each naming its mixer, feed-forward, norms and
block arrangement by *kind* with their sizes and constants as parameters), the
order in which layers run, the final norm and the output head.  The generic
model builder looks each kind up in the part registries, so a part never knows
which model it is in, and one model may hold different mixers and feed-forwards
in different layers.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """One tensor a part wants from the checkpoint."""
    name: str                 # full tensor name in the safetensors file
    shape: tuple[int, ...]
    init: str = "matrix"      # random-weights mode: "matrix" | "bias" | "norm" | "table"
    keep_f32: bool = False    # kept in 32-bit even in a bfloat16 engine


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part chosen by kind, with its sizes and constants."""
    kind: str
    params: dict[str, Any]
    prefix: str = ""          # tensor-name prefix of this part's weights

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward."""
    block: str                     # arrangement kind, e.g. "prenorm"
    mixer: PartSpec
    ffn: PartSpec
    norms: tuple[PartSpec, ...]    # as many as the arrangement wants
    hidden: int = 0


@dataclasses.dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes `ModelBlueprint.layers` (a layer may be named twice);
    ``cache`` names the cache this call uses (calls that give the same number
    share one cache); ``write`` is False for a call that only reads a cache
    another call has filled.
    """
    layer: int
    cache: int
    write: bool = True


@dataclasses.dataclass(frozen=True)
class ModelBlueprint:
    hidden: int
    vocab: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    eos_token_ids: tuple[int, ...] = ()


# ----------------------------------------------------------------------------------------
# What a mixer keeps per request between steps.
# ----------------------------------------------------------------------------------------

@dataclasses.dataclass(frozen=True)
class PagedKV:
    """Keys and values for every position (window == 0) or for the last ``window`` ones."""
    n_kv_heads: int
    head_dim: int
    window: int = 0

    def group_key(self):
        # Layers whose pages live and die together share a block table.
        return ("paged_kv", self.window)


@dataclasses.dataclass(frozen=True)
class FixedState:
    """A state of fixed size per request (recurrent mixers), kept in 32-bit."""
    shape: tuple[int, ...]

    def group_key(self):
        return ("fixed_state",)


CacheNeed = Optional[PagedKV | FixedState]
