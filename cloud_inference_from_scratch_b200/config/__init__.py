from .engine_config import EngineConfig, build_config, validate_config, with_overrides
from .model_config import ConfigError, Qwen2Config, read_config_json
from .registry import (
    Architecture,
    architecture_for,
    register_architecture,
    registered_architectures,
    resolve_config,
    resolve_model,
)
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

__all__ = [
    "Architecture", "ConfigError", "EngineConfig", "LayerSpec", "ModelSpec", "PartSpec",
    "Qwen2Config", "ScheduleEntry", "architecture_for", "build_config", "read_config_json",
    "register_architecture", "registered_architectures", "resolve_config", "resolve_model",
    "validate_config", "with_overrides",
]
