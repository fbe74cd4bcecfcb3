from .builder import CachePlan, CausalLM, cache_plan, expected_tensors, load_model

__all__ = ["CachePlan", "CausalLM", "cache_plan", "expected_tensors", "load_model"]
