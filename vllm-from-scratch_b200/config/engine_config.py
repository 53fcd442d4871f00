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
    # Pages in each group's pool.  None: as many as fit into ``gpu_memory_utilization`` of the
    # device memory that is free once the weights are loaded (the reference always takes a number).
    num_gpu_blocks: int | None = 64
    enable_prefix_caching: bool = False
    gpu_memory_utilization: float = 0.9

    def __post_init__(self) -> None:
        if self.block_size <= 0:
            raise ValueError(f"block_size must be positive, got {self.block_size}")
        if self.num_gpu_blocks is not None and self.num_gpu_blocks <= 0:
            raise ValueError(f"num_gpu_blocks must be positive, got {self.num_gpu_blocks}")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError(f"gpu_memory_utilization must be in (0, 1], got {self.gpu_memory_utilization}")


@dataclass(frozen=True)
class SchedulerConfig:
    max_num_seqs: int = 8               # most requests running at once
    max_num_batched_tokens: int = 64    # token budget of one step
    policy: str = "fcfs"                # or "priority"
    # Queue the next decode step on the GPU before the tokens of the running one have
    # come back to the host (they are fed on the device); what a stopped request
    # computed one step too far is thrown away.  On by default: the same tokens, a fifth
    # more of them a second at batch 8 (the host's part of a step hides behind the GPU's).
    # It takes effect where decode steps are graph replays on a CUDA device and falls back
    # step by step otherwise.  The reference has no such mode.
    async_scheduling: bool = True

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
