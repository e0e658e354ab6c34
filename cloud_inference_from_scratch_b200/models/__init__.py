from . import lodalix, qwen2, zisesun  # noqa: F401  (register Qwen2ForCausalLM, Zisesun and Lodalix)
from .decoder import CacheNeed, DecoderModel, LayerParts

__all__ = ["CacheNeed", "DecoderModel", "LayerParts"]
