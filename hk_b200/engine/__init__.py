from .context import StepContext
from .engine import (BatchTooLarge, Engine, EngineError, StepEntry, TokenOutOfRange, UnknownRequest, parse_dtype)

__all__ = ["BatchTooLarge", "Engine", "EngineError", "StepContext", "StepEntry", "TokenOutOfRange",
           "UnknownRequest", "parse_dtype"]
