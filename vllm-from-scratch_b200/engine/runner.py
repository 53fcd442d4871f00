"""Everything below the scheduler in one object: the model with its weights, the
cache's memory and books, and the step function over them.  The replay program
and the generating engine both build this and nothing else; the reference's
counterpart is the chain ``Worker.load_model`` -> ``GPUModelRunner`` ->
``initialize_kv_cache`` (minivllm/worker/worker.py:76-103, minivllm/worker/
gpu_model_runner.py:342-371, 585-660)."""

from __future__ import annotations

from pathlib import Path
from typing import Mapping

import torch

from ..cache import CacheManager, CacheStorage
from ..config.registry import load_model_config
from ..parts.model import DecoderModel
from ..parts.spec import ModelSpec
from ..weights.loader import load_weights, load_weights_from_tensors
from .step import StepEntry, StepFunction

_TORCH_DTYPE = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def require_device(device: str | torch.device) -> torch.device:
    device = torch.device(device)
    if device.type == "cuda" and not torch.cuda.is_available():
        raise RuntimeError(
            "no CUDA device is visible: the engine runs its own sm_100a kernels and has no CPU path")
    return device


class ModelRunner:
    """``num_pages=None`` sizes the pool from the device memory that is free once the weights are
    loaded: ``gpu_memory_utilization`` of it, less ``reserve_bytes`` for the activations and graphs
    of the steps to come, divided by what a page costs over all layers (the reference takes the
    number from its caller, ``--num-kv-blocks``, minivllm/demo.py:110; it profiles nothing)."""

    def __init__(self, spec: ModelSpec, weights: str | Path | Mapping[str, torch.Tensor], dtype: str,
                 page_size: int, num_pages: int | None, max_requests: int, device: str | torch.device = "cuda",
                 enable_prefix_caching: bool = False, model_config=None, gpu_memory_utilization: float = 0.9,
                 reserve_bytes: int = 4 << 30) -> None:
        self.device = require_device(device)
        self.dtype = _TORCH_DTYPE[dtype]
        self.model_config = model_config
        if self.dtype == torch.float32:
            # The 32-bit mode is 32-bit everywhere: nothing may route a product
            # through a reduced-precision tensor-core mode.
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        self.model = DecoderModel(spec, self.dtype, self.device)
        if isinstance(weights, Mapping):
            load_weights_from_tensors(self.model, weights)
        else:
            load_weights(self.model, weights)
        self.spec = spec
        self.max_requests = max_requests
        self.enable_prefix_caching = enable_prefix_caching
        if num_pages is None:
            num_pages = self.pages_that_fit(page_size, gpu_memory_utilization, reserve_bytes)
        self.rebuild_cache(page_size, num_pages)

    def rebuild_cache(self, page_size: int, num_pages: int) -> None:
        """A new, empty cache of ``num_pages`` pages (memory, books and step function); what the
        old one held is gone.  For a caller that sizes the pool after it has let go of memory
        of its own: ``runner.rebuild_cache(page, runner.pages_that_fit(page))``."""
        self.storage = self.manager = self.step_function = None
        cache_from = [entry.cache_from for entry in self.spec.schedule]
        self.storage = CacheStorage(self.model.cache_needs(), cache_from, page_size, num_pages,
                                    self.max_requests, self.dtype, self.device)
        self.manager = CacheManager(self.storage.group_windows, page_size, num_pages, self.max_requests,
                                    self.enable_prefix_caching, has_state=self.storage.has_state)
        self.step_function = StepFunction(self.model, self.storage, self.manager)

    def pages_that_fit(self, page_size: int, gpu_memory_utilization: float = 0.9,
                       reserve_bytes: int = 4 << 30) -> int:
        """How many pages the free memory of the device holds now (call it after the weights are
        loaded and whatever else must stay has been allocated)."""
        if self.device.type != "cuda":
            raise ValueError("the pool can be sized from free memory on a CUDA device only: give num_pages")
        if not 0.0 < gpu_memory_utilization <= 1.0:
            raise ValueError(f"gpu_memory_utilization must be in (0, 1], got {gpu_memory_utilization}")
        torch.cuda.synchronize(self.device)
        torch.cuda.empty_cache()
        free, _ = torch.cuda.mem_get_info(self.device)
        per_page = CacheStorage.bytes_per_page(self.model.cache_needs(), page_size, self.dtype)
        if per_page == 0:
            return 1
        pages = int((free * gpu_memory_utilization - reserve_bytes) // per_page)
        if pages < 1:
            raise RuntimeError(f"{free / 2**30:.1f} GiB are free on {self.device}: no room for a cache page of "
                               f"{per_page / 2**20:.2f} MiB beside the reserve of {reserve_bytes / 2**30:.1f} GiB")
        return pages

    @classmethod
    def from_folder(cls, folder: str | Path, dtype: str, page_size: int, num_pages: int | None,
                    max_requests: int, device: str | torch.device = "cuda",
                    enable_prefix_caching: bool = False, gpu_memory_utilization: float = 0.9) -> "ModelRunner":
        require_device(device)
        entry, config = load_model_config(folder)
        return cls(entry.build_spec(config), folder, dtype, page_size, num_pages, max_requests, device,
                   enable_prefix_caching, model_config=config, gpu_memory_utilization=gpu_memory_utilization)

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        return self.step_function.run(entries)

    def write_status(self, out: torch.Tensor) -> None:
        """The error words of the steps so far into ``out`` (int32 ``[kernels.STATUS_WORDS]`` on the
        device), without waiting; read them on the host with ``kernels.status_problem``."""
        from .. import kernels
        kernels.collect_status(self.model._token_error, out)

    def clear_device_errors(self) -> None:
        """Reset the error words (after their content has been reported)."""
        from .. import kernels
        self.model._token_error.zero_()
        kernels.device_error()

    def check_device(self) -> None:
        """Raise if a step since the last check fed a token id outside the vocabulary or
        a kernel gave up a bounded wait (waits for the device; not for every step)."""
        from .. import kernels
        self.model.check_token_ids()
        problem = kernels.device_error()        # None where no kernel library is loaded
        if problem:
            raise RuntimeError(f"a kernel reported an error, results since the last check are void: {problem}")
