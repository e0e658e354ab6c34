from . import qwen2, zisesun  # noqa: F401  (register Qwen2ForCausalLM and Zisesun)
from .decoder import CacheNeed, DecoderModel, LayerParts

__all__ = ["CacheNeed", "DecoderModel", "LayerParts"]
