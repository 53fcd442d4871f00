"""The generating engine: requests in, tokens out.

``LLMEngine`` keeps the reference's interface (minivllm/engine/llm_engine.py:
24-118): ``add_request``, ``step() -> list[RequestOutput]``, ``abort_request``,
``has_unfinished_requests``, ``shutdown``.  One ``step`` is one round of
schedule -> run the batch -> sample -> commit (minivllm/engine/core.py:251-280).
After an exception in a step the engine refuses further steps
(minivllm/engine/core.py:282-294): its cache and scheduler may disagree.

``LLM`` is the short way: ``LLM(model_folder).generate(prompts, params)``.
"""

from __future__ import annotations

import random
import time
from pathlib import Path
from typing import Sequence

import torch

from ..config.engine_config import CacheConfig, EngineConfig, ModelConfig, SchedulerConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .request import Request, RequestOutput, RequestStatus
from .runner import ModelRunner
from .scheduler import Scheduler, SchedulerOutput
from .step import StepEntry


class EngineDeadError(RuntimeError):
    pass


class LLMEngine:
    def __init__(self, config: EngineConfig, runner: ModelRunner | None = None) -> None:
        self.config = config
        model, cache, sched = config.model_config, config.cache_config, config.scheduler_config
        self.runner = runner or ModelRunner.from_folder(
            model.model, model.dtype, cache.block_size, cache.num_gpu_blocks, sched.max_num_seqs,
            device=config.device, enable_prefix_caching=cache.enable_prefix_caching)
        self.scheduler = Scheduler(sched, self.runner.manager, model.max_model_len)
        self.sampler = Sampler(self.runner.model.vocab_size, self.runner.device)
        self._seed_source = random.Random(model.seed)
        self._failure: BaseException | None = None
        self._first_inputs: dict | None = None
        self.num_steps = 0
        self.decode_graphs = None
        if not model.enforce_eager and self.runner.device.type == "cuda":
            from .decode_graph import DecodeGraphs
            self.decode_graphs = DecodeGraphs(self.runner, sched.max_num_seqs, model.max_model_len)

    # ----------------------------------------------------------------- requests
    def add_request(self, request_id: str, prompt_token_ids: Sequence[int],
                    sampling_params: SamplingParams | None = None, arrival_time: float | None = None,
                    priority: int = 0) -> None:
        params = sampling_params or SamplingParams()
        prompt = [int(t) for t in prompt_token_ids]
        vocab = self.runner.model.vocab_size
        bad = [t for t in prompt if not 0 <= t < vocab]
        if bad:
            raise ValueError(f"prompt token id {bad[0]} lies outside the vocabulary [0, {vocab})")
        room = self.config.model_config.max_model_len - len(prompt)
        if 0 < room < params.max_tokens:
            # minivllm/engine/core.py:122-125: no more tokens than the context has room for.
            params = SamplingParams(**{**params.__dict__, "max_tokens": room,
                                       "min_tokens": min(params.min_tokens, room)})
        seed = params.seed if params.seed is not None else self._seed_source.getrandbits(62)
        self.scheduler.add_request(Request(
            str(request_id), prompt, params, arrival_time if arrival_time is not None else time.monotonic(),
            priority, seed=seed))

    def abort_request(self, request_ids) -> None:
        self.scheduler.finish_requests(request_ids, RequestStatus.FINISHED_ABORTED)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_requests()

    # --------------------------------------------------------------------- step
    def step(self) -> list[RequestOutput]:
        if self._failure is not None:
            raise EngineDeadError(
                f"an earlier step failed ({self._failure!r}); build a new engine") from self._failure
        try:
            return self._step()
        except BaseException as error:
            self._failure = error
            raise

    def _step(self) -> list[RequestOutput]:
        plan = self.scheduler.schedule()
        self.num_steps += 1
        if not plan.scheduled:
            return []
        sampled = self._execute(plan)
        return self.scheduler.update(plan, sampled)

    def _execute(self, plan: SchedulerOutput) -> dict[str, int]:
        entries = []
        sampling = []
        for item in plan.scheduled:
            request = item.request
            tokens = request.all_token_ids[item.start:item.start + item.num_tokens]
            entries.append(StepEntry(request.request_id, tokens, item.start,
                                     [item.num_tokens - 1] if item.samples else []))
            if item.samples:
                sampling.append(request)
        if self.decode_graphs is not None and self.decode_graphs.accepts(entries):
            logits = self.decode_graphs.run(entries)
        else:
            logits = self.runner.step(entries)
        if self._first_inputs is None:
            self._first_inputs = self._describe_inputs(plan)
        if not sampling:
            return {}
        tokens = self.sampler.sample(
            logits, [r.sampling_params for r in sampling], [r.seed for r in sampling],
            [r.prompt_token_ids for r in sampling], [r.output_token_ids for r in sampling])
        return {request.request_id: token for request, token in zip(sampling, tokens)}

    # -------------------------------------------------------------------- trace
    def _describe_inputs(self, plan: SchedulerOutput) -> dict | None:
        ctx = self.runner.step_function.last_context
        if ctx is None:
            return None
        return {
            "num_scheduled_tokens": {i.request.request_id: i.num_tokens for i in plan.scheduled},
            "positions": ctx.positions.tolist(),
            "query_start": ctx.query_start.tolist(),
            "seq_lens": ctx.seq_lens.tolist(),
            "slot_mapping": {g: c.slot_mapping.tolist() for g, c in ctx.groups.items()},
            "block_table": {g: c.block_table.tolist() for g, c in ctx.groups.items()},
        }

    @property
    def first_step_inputs(self) -> dict | None:
        """What the first step fed to the model (the demo's ``--trace``)."""
        return self._first_inputs

    def shutdown(self) -> None:
        self.decode_graphs = None


class LLM:
    """``LLM(folder, dtype="bfloat16").generate([[1, 2, 3], ...], SamplingParams(...))``."""

    def __init__(self, model: str | Path, dtype: str = "bfloat16", max_model_len: int = 4096,
                 block_size: int = 16, num_gpu_blocks: int | None = None, max_num_seqs: int = 8,
                 max_num_batched_tokens: int = 2048, enable_prefix_caching: bool = False,
                 enforce_eager: bool = False, seed: int = 0, device: str = "cuda") -> None:
        if num_gpu_blocks is None:
            num_gpu_blocks = max_num_seqs * -(-max_model_len // block_size)
        self.engine = LLMEngine(EngineConfig(
            ModelConfig(str(model), dtype, max_model_len, enforce_eager, seed),
            CacheConfig(block_size, num_gpu_blocks, enable_prefix_caching),
            SchedulerConfig(max_num_seqs, max_num_batched_tokens), device))
        self._counter = 0

    def generate(self, prompt_token_ids: Sequence[Sequence[int]],
                 sampling_params: SamplingParams | Sequence[SamplingParams] | None = None
                 ) -> list[RequestOutput]:
        """Generate for every prompt; results come back in the order of the prompts."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompt_token_ids)
        if len(sampling_params) != len(prompt_token_ids):
            raise ValueError("one SamplingParams per prompt, or one for all")
        ids = []
        for prompt, params in zip(prompt_token_ids, sampling_params):
            request_id = f"gen-{self._counter}"
            self._counter += 1
            self.engine.add_request(request_id, prompt, params)
            ids.append(request_id)
        latest: dict[str, RequestOutput] = {}
        while self.engine.has_unfinished_requests():
            for output in self.engine.step():
                latest[output.request_id] = output
        return [latest[request_id] for request_id in ids]
