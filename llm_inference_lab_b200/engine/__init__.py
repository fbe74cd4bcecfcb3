from .engine import Engine, EngineStats, Entry, InvalidInput, parse_dtype

__all__ = ["Engine", "EngineStats", "Entry", "InvalidInput", "parse_dtype"]
