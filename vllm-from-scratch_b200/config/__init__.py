"""Configuration: the model's own config.json as a typed object, the engine's
knobs, and the registry from an architecture's name to what builds it."""

from .engine_config import (CacheConfig, EngineConfig, ModelConfig, SchedulerConfig,
                            VllmConfig, canonical_dtype)
from .model_config import ConfigError, Qwen3Config
from .registry import (ArchitectureEntry, get_architecture, load_model_config,
                       register_architecture, registered_architectures)

__all__ = [
    "ArchitectureEntry", "CacheConfig", "ConfigError", "EngineConfig", "ModelConfig",
    "Qwen3Config", "SchedulerConfig", "VllmConfig", "canonical_dtype", "get_architecture",
    "load_model_config", "register_architecture", "registered_architectures",
]
