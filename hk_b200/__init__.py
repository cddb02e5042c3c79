"""hk_b200: a small, whole inference engine for the Qwen3 dense decoder on one B200."""
from . import models  # noqa: F401  (registers the architectures)
from .api import HKForCausalLM, NativeHKEngine, generate, generate_with_engine
from .engine import Engine, StepEntry
from .sampling import SamplingParams

__version__ = "0.1.0"
__all__ = ["Engine", "HKForCausalLM", "NativeHKEngine", "SamplingParams", "StepEntry", "generate",
           "generate_with_engine"]
