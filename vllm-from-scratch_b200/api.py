"""The public interface, re-exported by the importable package."""

from .cache import CacheManager, CacheStorage
from .config import (CacheConfig, ConfigError, EngineConfig, ModelConfig, Qwen3Config,
                     SchedulerConfig, VllmConfig, get_architecture, load_model_config,
                     register_architecture, registered_architectures)
from .engine.llm_engine import LLM, EngineDeadError, LLMEngine
from .engine.request import FinishReason, Logprob, Request, RequestOutput, RequestStatus
from .engine.runner import ModelRunner
from .engine.scheduler import Scheduler, SchedulerOutput
from .sampling import Sampler, SamplingParams
from .engine.step import StepEntry, StepFunction
from .parts import DecoderModel, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .weights import WeightLoadError, load_weights, write_random_model

__all__ = [
    "LLM", "LLMEngine", "EngineDeadError", "FinishReason", "Logprob", "Request", "RequestOutput", "RequestStatus",
    "Sampler", "SamplingParams", "Scheduler", "SchedulerOutput",
    "CacheConfig", "CacheManager", "CacheStorage", "ConfigError", "DecoderModel", "EngineConfig",
    "LayerSpec", "ModelConfig", "ModelRunner", "ModelSpec", "PartSpec", "Qwen3Config",
    "ScheduleEntry", "SchedulerConfig", "StepEntry", "StepFunction", "VllmConfig", "WeightLoadError",
    "get_architecture", "load_model_config", "load_weights", "register_architecture",
    "registered_architectures", "write_random_model",
]
