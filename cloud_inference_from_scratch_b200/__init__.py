"""A small, whole inference engine for the Qwen2 dense decoder on one B200 (sm_100a).

    from cloud_inference_from_scratch_b200 import InferenceEngine, GenerationConfig, build_config, generate
"""

from . import models, parts  # noqa: F401  (fills the registries)
from .config import EngineConfig, build_config, with_overrides
from .engine import GenerationConfig, GenerationResult, InferenceEngine, RequestHandle, generate

__version__ = "0.1.0"

__all__ = [
    "EngineConfig", "GenerationConfig", "GenerationResult", "InferenceEngine", "RequestHandle",
    "build_config", "generate", "with_overrides",
]
