from . import qwen3  # noqa: F401  (registers the architecture)
from .spec import LayerCall, ModelSpec

__all__ = ["LayerCall", "ModelSpec"]
