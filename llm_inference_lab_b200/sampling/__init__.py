from .sampler import Sampler, SamplingConfig

__all__ = ["Sampler", "SamplingConfig"]
