"""Engine-side configuration: which model and precision, how many pages, how
many tokens a step may carry.

Names and meanings follow the reference's ``ModelConfig`` / ``CacheConfig`` /
``SchedulerConfig`` / ``VllmConfig`` (minivllm/config.py:125-166, 220-240,
243-262, 1898-1913) so that a user of that engine finds the same knobs.
"""

from __future__ import annotations

from dataclasses import dataclass, field

_DTYPES = {
    # minivllm/model_loader/base_loader.py:21-30
    "float32": "float32", "fp32": "float32",
    "bfloat16": "bfloat16", "bf16": "bfloat16",
}


def canonical_dtype(name: str) -> str:
    try:
        return _DTYPES[str(name).lower().replace("torch.", "")]
    except KeyError:
        raise ValueError(
            f"dtype {name!r} is not built: choose 'bfloat16' (serving kernels) or "
            f"'float32' (true 32-bit arithmetic everywhere)") from None


@dataclass(frozen=True)
class ModelConfig:
    model: str                      # folder with config.json and model.safetensors
    dtype: str = "bfloat16"
    max_model_len: int = 4096       # longest request (prompt + generated)
    enforce_eager: bool = False     # True: no CUDA-graph replay of decode steps
    seed: int = 0                   # engine-level seed for requests that bring none

    def __post_init__(self) -> None:
        object.__setattr__(self, "dtype", canonical_dtype(self.dtype))
        if self.max_model_len < 2:
            raise ValueError(f"max_model_len must be at least 2, got {self.max_model_len}")


@dataclass(frozen=True)
class CacheConfig:
    block_size: int = 16            # tokens per page
    num_gpu_blocks: int = 64        # pages in each group's pool (no memory profiling)
    enable_prefix_caching: bool = False

    def __post_init__(self) -> None:
        if self.block_size <= 0:
            raise ValueError(f"block_size must be positive, got {self.block_size}")
        if self.num_gpu_blocks <= 0:
            raise ValueError(f"num_gpu_blocks must be positive, got {self.num_gpu_blocks}")


@dataclass(frozen=True)
class SchedulerConfig:
    max_num_seqs: int = 8               # most requests running at once
    max_num_batched_tokens: int = 64    # token budget of one step
    policy: str = "fcfs"                # or "priority"
    # Queue the next decode step on the GPU before the tokens of the running one have
    # come back to the host (they are fed on the device); what a stopped request
    # computed one step too far is thrown away.  The reference has no such mode.
    async_scheduling: bool = False

    def __post_init__(self) -> None:
        if self.max_num_seqs <= 0:
            raise ValueError(f"max_num_seqs must be positive, got {self.max_num_seqs}")
        if self.max_num_batched_tokens <= 0:
            raise ValueError(
                f"max_num_batched_tokens must be positive, got {self.max_num_batched_tokens}")
        if self.policy not in ("fcfs", "priority"):
            raise ValueError(f"policy must be 'fcfs' or 'priority', got {self.policy!r}")


@dataclass(frozen=True)
class EngineConfig:
    model_config: ModelConfig
    cache_config: CacheConfig = field(default_factory=CacheConfig)
    scheduler_config: SchedulerConfig = field(default_factory=SchedulerConfig)
    device: str = "cuda"


# The reference's name for the same object.
VllmConfig = EngineConfig
