"""Interfaces of the parts a model is put together from, and their registries.

A part is built from a `PartSpec` (its sizes and constants), the tensors it
named in `tensors(spec)`, the engine's storage type and the device.  Parts are
looked up by kind:

=================  ==========================================================
registry           interface
=================  ==========================================================
``MIXERS``         `Mixer`: ``cache_need(spec)``, ``forward(x, ctx, cache)``
``FEED_FORWARDS``  `FeedForward`: ``forward(x, ctx)``
``NORMS``          `Norm`: ``forward(x, rows=None)``, ``forward_add(x, delta, rows=None)``
``POSITIONS``      `PositionEncoding`: ``rotate_and_store(...)``
``BLOCKS``         `Block`: ``forward(x, pending, ctx, cache)``
``EMBEDDINGS``     `Embedding`: ``forward(token_ids)``
``HEADS``          `Head`: ``forward(x)`` giving 32-bit logits
=================  ==========================================================

`x` is the packed batch ``[tokens, hidden]``: rows of all requests of the step,
one after the other.  `ctx` (`StepContext`) says which request and position
each row belongs to and where the cache of each request lies.
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch

from .spec import CacheNeed, PartSpec, TensorSpec


@dataclasses.dataclass
class GroupView:
    """Per-step metadata of one cache group (layers whose pages live and die together)."""
    page_size: int
    window: int
    row_slot: torch.Tensor      # [tokens] int32: page * page_size + offset where each row's K/V go
    block_table: torch.Tensor   # [requests, width] int32: page of each logical block, -1 if none


@dataclasses.dataclass
class StepContext:
    """What a step's kernels need to know about the packed batch."""
    dtype: torch.dtype
    device: torch.device
    n_tokens: int
    n_requests: int
    token_ids: torch.Tensor     # [tokens] int32
    row_req: torch.Tensor       # [tokens] int32: index of the row's request within the step
    row_pos: torch.Tensor       # [tokens] int32: absolute position of the row
    q_start: torch.Tensor       # [requests + 1] int32: first row of each request
    kv_len: torch.Tensor        # [requests] int32: tokens held after this step
    pos0: torch.Tensor          # [requests] int32: position of the request's first row
    state_slot: torch.Tensor    # [requests] int32: slot of the request's fixed-size state
    groups: list[GroupView]
    # host copies, for launch decisions only
    q_lens: list[int]
    kv_lens: list[int]
    state_slots: list[int]
    max_q_len: int = 0
    max_kv_len: int = 0
    scratch: dict = dataclasses.field(default_factory=dict)   # per-step buffers shared between layers


@dataclasses.dataclass
class CacheView:
    """The cache one layer call works on."""
    need: CacheNeed
    group: int = -1                         # index into StepContext.groups (paged caches)
    write: bool = True                      # False: the call only reads what another call wrote
    k: Optional[torch.Tensor] = None        # [pages, n_kv, page_size, head_dim]
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None    # [max_requests, *shape] float32


class Part:
    kind = ""

    @classmethod
    def tensors(cls, spec: PartSpec) -> list[TensorSpec]:
        return []

    def __init__(self, spec: PartSpec, weights: dict[str, torch.Tensor], dtype: torch.dtype, device):
        self.spec, self.dtype, self.device = spec, dtype, device

    def _weight(self, weights, name, keep_f32=False):
        t = weights[self.spec.prefix + name]
        want = torch.float32 if keep_f32 else self.dtype
        return t if t.dtype == want else t.to(want)


class Mixer(Part):
    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def forward_add(self, x: torch.Tensor, delta: Optional[torch.Tensor],
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x += delta in place (32-bit add), then the norm of the sum.  With `rows`, only
        those rows are computed and x is left as it is."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Encodes positions into q and k.  A new encoding defines `encode`; the paged store of k and v is
    the framework's (`rotate_and_store` below), so an encoding never touches the cache.  An encoding
    that brings a fused kernel of its own may override `rotate_and_store` as a whole, take the
    projection's 32-bit split-K partial sums (`takes_partials`), or offer per-step cosines and sines
    to the mixer's fused projection (`table`, see `Rope`)."""
    takes_partials = False      # rotate_and_store accepts [splits, tokens, width] partial sums plus the bias

    def encode(self, qkv: torch.Tensor, positions: torch.Tensor, n_q: int, n_kv: int, head_dim: int) -> None:
        """Encodes, in place, the q heads (columns [0, n_q * d)) and the k heads (the next n_kv * d
        columns) of the fused projection `qkv` [tokens, (n_q + 2 n_kv) * d]; `positions` [tokens] int32."""
        raise NotImplementedError

    def rotate_and_store(self, qkv, positions, slots, cache: CacheView, n_q: int, n_kv: int, head_dim: int,
                         bias=None, scratch=None) -> torch.Tensor:
        """Encodes q and k of the fused projection `qkv`, writes k and v to the cache slots when the
        call may write, and returns the encoded q.  `scratch` is the step's dictionary for buffers that
        layers may share (e.g. a table of angles)."""
        from ..kernels import ops
        self.encode(qkv, positions, n_q, n_kv, head_dim)
        write = cache is not None and cache.write
        return ops.kv_store(qkv, slots if write else None, cache.k if write else None, cache.v if write else None,
                            n_q, n_kv, head_dim)


class Block:
    kind = ""

    def __init__(self, mixer: Mixer, ffn: FeedForward, norms: list[Norm]):
        self.mixer, self.ffn, self.norms = mixer, ffn, norms
        # names of the profiling ranges around the two halves of a block
        self.mixer_range = "mixer." + str(getattr(getattr(mixer, "spec", None), "kind", type(mixer).__name__))
        self.ffn_range = "feed_forward." + str(getattr(getattr(ffn, "spec", None), "kind", type(ffn).__name__))

    def forward(self, x, pending, ctx: StepContext, cache: CacheView):
        """`pending` is what the previous block still owes the residual stream (or None)."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def pick(self, x: torch.Tensor, temperature, seeds, positions, out=None) -> torch.Tensor:
        """One token per row (int32): greedy where `temperature` is None or 0, else sampled with the
        row's seed at its position.  The default forms the logits and lets the sampling kernel pick; a
        head may do both in one pass."""
        from ..kernels import ops
        return ops.sample(self.forward(x), temperature, seeds, positions, out=out)


MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITIONS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}
EMBEDDINGS: dict[str, type] = {}
HEADS: dict[str, type] = {}
_REGISTRIES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS, "position": POSITIONS,
               "block": BLOCKS, "embedding": EMBEDDINGS, "head": HEADS}


def register_part(family: str, kind: str, cls: type) -> type:
    """Make `cls` available under `kind` in one of the part registries."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family {family!r}; known: {', '.join(_REGISTRIES)}")
    cls.kind = kind
    _REGISTRIES[family][kind] = cls
    return cls


def lookup(family: str, kind: str) -> type:
    try:
        return _REGISTRIES[family][kind]
    except KeyError:
        raise KeyError(f"no {family} of kind {kind!r} is registered; known: "
                       f"{', '.join(sorted(_REGISTRIES[family]))}") from None
