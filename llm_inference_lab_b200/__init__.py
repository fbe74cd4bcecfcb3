"""A small, whole, single-GPU inference engine for B200 (sm_100a).

Everything between a request's tokens and its next token for the Qwen2 dense
GQA decoder: typed configuration and registry, weights by tensor name, layers
put together from parts, a paged cache manager, one packed step function, a
scheduler, sampling, and hand-written CUDA kernels with a true 32-bit path.
"""
from . import parts as _parts  # noqa: F401  (registers the built-in part kinds)
from .registry import architectures, load_config, register_architecture

__all__ = ["architectures", "load_config", "register_architecture"]
__version__ = "0.1.0"
