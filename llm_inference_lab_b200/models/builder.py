"""The generic model: a `ModelBlueprint` turned into parts, and its forward pass.

Nothing here knows Qwen2.  The blueprint names the parts by kind; the registries
of `parts.base` supply the classes; the run order is the blueprint's list of
`LayerCall`s, which may name a layer twice or let a call read the cache another
call fills.  The data flow of one step follows the reference's
`submit_forward_kernels` (rust/engine/src/runner/model/qwen2/engine.rs:916-1130):
embedding, the layers in order, then the final norm and the head only at the
rows whose logits are wanted (engine.rs:1298-1341).
"""
from __future__ import annotations

import dataclasses

import torch

from ..parts.base import CacheView, StepContext, lookup
from ..profiling import scoped_range
from ..parts.spec import CacheNeed, ModelBlueprint, PagedKV, TensorSpec


# False: pure decode steps run part by part as every other step does (tests compare the two).
USE_DECODE_STACK = True


def _part_classes(bp: ModelBlueprint):
    yield lookup("embedding", bp.embedding.kind), bp.embedding
    for layer in bp.layers:
        yield lookup("mixer", layer.mixer.kind), layer.mixer
        yield lookup("feed_forward", layer.ffn.kind), layer.ffn
        for n in layer.norms:
            yield lookup("norm", n.kind), n
    yield lookup("norm", bp.final_norm.kind), bp.final_norm
    yield lookup("head", bp.head.kind), bp.head


def expected_tensors(bp: ModelBlueprint) -> list[TensorSpec]:
    """Every tensor the model's parts want from the checkpoint, each name once."""
    seen: dict[str, TensorSpec] = {}
    for cls, spec in _part_classes(bp):
        for t in cls.tensors(spec):
            if t.name in seen and seen[t.name].shape != t.shape:
                raise ValueError(f"two parts want tensor {t.name!r} with different shapes")
            seen.setdefault(t.name, t)
    return list(seen.values())


@dataclasses.dataclass(frozen=True)
class CachePlan:
    """What the caches of a model look like: one need per cache id, gathered in groups."""
    needs: tuple[CacheNeed, ...]            # by cache id
    group_of: tuple[int, ...]               # cache id -> group index (-1: no paged group)
    group_windows: tuple[int, ...]          # per paged group: 0 or the window


def cache_plan(bp: ModelBlueprint) -> CachePlan:
    n_caches = 1 + max((c.cache for c in bp.order), default=-1)
    needs: list = [None] * n_caches
    writers = [0] * n_caches
    for call in bp.order:
        layer = bp.layers[call.layer]
        need = lookup("mixer", layer.mixer.kind).cache_need(layer.mixer)
        if needs[call.cache] is not None and needs[call.cache] != need:
            raise ValueError(f"cache {call.cache} is used by layers with different needs: "
                             f"{needs[call.cache]} and {need}")
        needs[call.cache] = need
        writers[call.cache] += bool(call.write)
    for cid, n in enumerate(writers):
        if needs[cid] is not None and n == 0:
            raise ValueError(f"cache {cid} is read but no layer call writes it")
    keys: list = []
    group_of = []
    for need in needs:
        if isinstance(need, PagedKV):
            key = need.group_key()
            if key not in keys:
                keys.append(key)
            group_of.append(keys.index(key))
        else:
            group_of.append(-1)
    return CachePlan(tuple(needs), tuple(group_of), tuple(k[1] for k in keys))


class CausalLM:
    """Embedding, blocks in the blueprint's order, final norm, head."""

    decode_stack = None     # the one kernel that runs all layer calls of a small decode step, where the layers fit it

    def __init__(self, bp: ModelBlueprint, weights: dict[str, torch.Tensor], dtype: torch.dtype, device):
        self.blueprint, self.dtype, self.device = bp, dtype, device
        weights = dict(weights)
        self.embedding = lookup("embedding", bp.embedding.kind)(bp.embedding, weights, dtype, device)
        self.blocks = []
        for layer in bp.layers:
            mixer = lookup("mixer", layer.mixer.kind)(layer.mixer, weights, dtype, device)
            ffn = lookup("feed_forward", layer.ffn.kind)(layer.ffn, weights, dtype, device)
            norms = [lookup("norm", n.kind)(n, weights, dtype, device) for n in layer.norms]
            self.blocks.append(lookup("block", layer.block)(mixer, ffn, norms))
        self.final_norm = lookup("norm", bp.final_norm.kind)(bp.final_norm, weights, dtype, device)
        self.head = lookup("head", bp.head.kind)(bp.head, weights, dtype, device)
        self.order = bp.order
        # pure decode steps of few tokens run all layer calls as one kernel where the layers fit it
        from .decode_stack import DecodeStack
        self.decode_stack = DecodeStack.build(self.blocks, bp.order, dtype, device) if str(device) != "cpu" else None
        self.range_names = [f"layer.{call.layer}" for call in bp.order]     # profiling ranges
        self.cache_plan = cache_plan(bp)

    def forward(self, ctx: StepContext, caches: list[CacheView], logit_rows: torch.Tensor | None, pick=None):
        """Runs the rows of `ctx`; returns 32-bit logits [len(logit_rows), vocab] or None.  With
        `pick` = (temperatures, seeds, positions, out), each [len(logit_rows)] on the device, it returns one
        token per wanted row instead (`Head.pick`)."""
        with scoped_range("embedding"):
            x = self.embedding.forward(ctx.token_ids)
        pending = None
        stack = self.decode_stack
        if stack is not None and USE_DECODE_STACK and stack.serves(ctx, caches):
            with scoped_range("decode_stack"):
                stack.run(x, ctx, caches)
            calls = ()
        else:
            calls = zip(self.order, self.range_names)
        for call, name in calls:
            view = caches[call.cache]
            if not call.write:
                view = dataclasses.replace(view, write=False)
            with scoped_range(name):
                x, pending = self.blocks[call.layer].forward(x, pending, ctx, view)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        with scoped_range("final_norm+head"):
            h = self.final_norm.forward_add(x, pending, rows=logit_rows)
            if pick is not None:
                return self.head.pick(h, *pick)
            return self.head.forward(h)


def load_model(model_dir: str, dtype: torch.dtype, device) -> tuple[CausalLM, object]:
    """config.json picks the architecture; weights come by tensor name."""
    from ..registry import load_config
    from ..weights.loader import load_weights

    arch, config = load_config(model_dir)
    bp = arch.blueprint(config)
    weights = load_weights(model_dir, expected_tensors(bp), device, optional=_tied_extras(bp))
    return CausalLM(bp, weights, dtype, device), config


def _tied_extras(bp: ModelBlueprint) -> tuple[str, ...]:
    # A checkpoint with tied embeddings may still carry a copy of the head; it is ignored.
    if bp.head.get("tied_to"):
        return (bp.head.prefix + "weight",)
    return ()
