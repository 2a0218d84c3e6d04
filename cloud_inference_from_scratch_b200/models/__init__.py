from . import qwen2  # noqa: F401  (registers Qwen2ForCausalLM)
from .decoder import CacheNeed, DecoderModel, LayerParts

__all__ = ["CacheNeed", "DecoderModel", "LayerParts"]
