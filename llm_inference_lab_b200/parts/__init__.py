"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, CacheView, Embedding,
                   FeedForward, GroupView, Head, Mixer, Norm, Part, PositionEncoding, StepContext, lookup,
                   register_part)
from .spec import FixedState, LayerCall, LayerSpec, ModelBlueprint, PagedKV, PartSpec, TensorSpec

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheView",
           "Embedding", "FeedForward", "GroupView", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "StepContext", "lookup", "register_part", "FixedState", "LayerCall", "LayerSpec", "ModelBlueprint",
           "PagedKV", "PartSpec", "TensorSpec"]
