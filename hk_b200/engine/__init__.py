from .context import StepContext
from .engine import (BatchTooLarge, DeviceToken, Engine, EngineError, KernelTimeout, StepEntry, TokenOutOfRange, UnknownRequest, parse_dtype)

__all__ = ["BatchTooLarge", "DeviceToken", "Engine", "EngineError", "KernelTimeout", "StepContext", "StepEntry", "TokenOutOfRange",
           "UnknownRequest", "parse_dtype"]
