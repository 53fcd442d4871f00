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

import numpy as np
import torch

from .. import kernels
from ..config.engine_config import CacheConfig, EngineConfig, ModelConfig, SchedulerConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .request import Request, RequestOutput, RequestStatus
from .runner import ModelRunner
from .scheduler import Scheduler, SchedulerOutput
from .step import StepEntry


class EngineDeadError(RuntimeError):
    pass


class _InFlight:
    """A step whose work is queued on the GPU: the plan, the requests that sample (in
    row order), their ids on the device (followed by the step's status words when
    ``has_status``), and the pinned copy on its way to the host."""

    def __init__(self, plan: SchedulerOutput, sampling: list[Request], tokens: torch.Tensor | None,
                 host: torch.Tensor | None, has_status: bool = False, logprob_width: int = 0) -> None:
        self.plan, self.sampling, self.tokens, self.host = plan, sampling, tokens, host
        self.has_status = has_status
        self.logprob_width = logprob_width          # columns of log-probabilities per row behind ids and status (0: none)
        self.status: list[int] | None = None        # filled by wait()
        self.logprobs: dict[str, tuple[list[int], list[float], int]] | None = None
        self.arrived: torch.cuda.Event | None = None
        if tokens is not None and host is not None:
            host[:tokens.shape[0]].copy_(tokens, non_blocking=True)
            self.arrived = torch.cuda.Event()
            self.arrived.record()

    def wait(self) -> dict[str, int]:
        if self.tokens is None:
            return {}
        if self.arrived is not None:
            self.arrived.synchronize()
            words = self.host[:self.tokens.shape[0]].numpy()
        else:
            words = self.tokens.cpu().numpy()
        rows = len(self.sampling)
        extra = kernels.STATUS_WORDS if self.has_status else 0
        values = words[:rows + extra].tolist()
        if self.has_status:
            self.status = values[rows:]
        if self.logprob_width:
            ids, bits, places = Sampler.logprob_views(words[rows + extra:], rows, self.logprob_width)
            ids, numbers, places = ids.tolist(), bits.view(np.float32).tolist(), places.tolist()
            self.logprobs = {request.request_id: (ids[row], numbers[row], places[row])
                             for row, request in enumerate(self.sampling) if request.sampling_params.logprobs is not None}
        return {request.request_id: token for request, token in zip(self.sampling, values)}


class LLMEngine:
    def __init__(self, config: EngineConfig, runner: ModelRunner | None = None, tokenizer=None) -> None:
        """``tokenizer``: anything with ``decode(ids, skip_special_tokens=True)``; outputs then carry
        ``text`` (minivllm/engine/llm_engine.py:25, minivllm/outputs.py:198)."""
        self.config = config
        self.tokenizer = tokenizer
        model, cache, sched = config.model_config, config.cache_config, config.scheduler_config
        self.runner = runner or ModelRunner.from_folder(
            model.model, model.dtype, cache.block_size, cache.num_gpu_blocks, sched.max_num_seqs,
            device=config.device, enable_prefix_caching=cache.enable_prefix_caching,
            gpu_memory_utilization=cache.gpu_memory_utilization)
        trained = getattr(self.runner.model_config, "max_position_embeddings", None)
        if trained is not None and model.max_model_len > trained:
            # minivllm/worker/worker.py:140: positions past the range the position encoding was
            # trained for are refused (rotation angles are computed on the fly here, so nothing
            # else would stop them).
            raise ValueError(f"max_model_len={model.max_model_len} exceeds the model's "
                             f"max_position_embeddings={trained}")
        self.scheduler = Scheduler(sched, self.runner.manager, model.max_model_len)
        self.sampler = Sampler(self.runner.model.vocab_size, self.runner.device)
        self._seed_source = random.Random(model.seed)
        self._failure: BaseException | None = None
        self._first_inputs: dict | None = None
        self.num_steps = 0
        self.num_steps_ahead = 0            # steps queued before their input tokens reached the host
        self._pending: _InFlight | None = None
        self._host_tokens: list[torch.Tensor] = []
        # Every step that samples brings the kernels' error words to the host beside its ids.
        self._carry_status = self.runner.device.type == "cuda"
        self.decode_graphs = None
        self.mixed_graphs = None
        # Steps are replayed as CUDA graphs only if every part of the model says that it reads
        # what differs between steps from device data (``Part.graph_safe``): a part that looks
        # at the batch from the host would have its first step's values baked into a graph.
        self.graphs_refused_by_parts = (not model.enforce_eager and self.runner.device.type == "cuda"
                                        and not self.runner.model.graph_safe())
        if not model.enforce_eager and self.runner.device.type == "cuda" and self.runner.model.graph_safe():
            from .decode_graph import DecodeGraphs, MixedGraphs
            self.decode_graphs = DecodeGraphs(self.runner, sched.max_num_seqs, model.max_model_len)
            if not self.runner.storage.has_state:
                # Prompt steps of models with per-request state stay on the ordinary path: the
                # padding requests of a replayed prompt step bring no tokens at all, which a
                # state-keeping part would have to know how to skip.
                self.mixed_graphs = MixedGraphs(self.runner, model.max_model_len)

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
        request_ids = [request_ids] if isinstance(request_ids, str) else list(request_ids)
        self.scheduler.finish_requests(request_ids, RequestStatus.FINISHED_ABORTED)
        for request_id in request_ids:
            self.sampler.forget(request_id)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished_requests()

    def get_num_unfinished_requests(self) -> int:
        """Running and waiting requests (minivllm/engine/llm_engine.py:83-86)."""
        return len(self.scheduler.running) + len(self.scheduler.waiting)

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
        current, self._pending = self._pending, None
        if current is None:
            plan = self.scheduler.schedule()
            self.num_steps += 1
            if not plan.scheduled:
                return []
            current = self._execute(plan)
        if self._overlaps():
            # Queue the step after this one before waiting for this one's tokens.
            ahead = self.scheduler.schedule_ahead(current.plan)
            if ahead is not None:
                self.num_steps += 1
                self.num_steps_ahead += 1
                self._pending = self._execute(ahead, previous=current)
        sampled = current.wait()
        if current.status is not None:
            # The step's error words came with its ids: a step that fed a bad token id, or in which
            # a kernel gave up a bounded wait, is refused before anything of it is committed,
            # handed out or published to the prefix cache.
            problem = kernels.status_problem(current.status, self.runner.model.vocab_size)
            if problem:
                self.runner.clear_device_errors()
                raise RuntimeError(f"the step is void: {problem}")
        outputs = self.scheduler.update(current.plan, sampled, current.logprobs)
        for output in outputs:
            if output.finished:
                self.sampler.forget(output.request_id)
            if self.tokenizer is not None:
                output.text = self.tokenizer.decode(output.token_ids, skip_special_tokens=True)
        idle = not self.scheduler.has_unfinished_requests()
        if self._pending is not None and idle:
            self._pending = None            # everyone stopped: what was queued ahead is of no use
        if idle:
            self.runner.check_device()      # steps that sampled nothing (prompt portions) carry no words
        return outputs

    def _overlaps(self) -> bool:
        return (self.config.scheduler_config.async_scheduling and self.decode_graphs is not None
                and self.runner.device.type == "cuda")

    def _pinned(self, rows: int) -> torch.Tensor | None:
        """One of two pinned buffers for the sampled ids (two steps may be in flight)."""
        if self.runner.device.type != "cuda":
            return None
        if not self._host_tokens:
            most = self.config.scheduler_config.max_num_seqs
            size = max(rows, most + kernels.STATUS_WORDS + Sampler.logprob_words(most, kernels.MAX_LOGPROBS + 1))
            self._host_tokens = [torch.empty(size, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._host_tokens.reverse()
        buffer = self._host_tokens[0]
        return buffer if buffer.shape[0] >= rows else None

    def _execute(self, plan: SchedulerOutput, previous: _InFlight | None = None) -> _InFlight:
        """Queue the plan's batch and its sampling.  With ``previous`` the plan was made
        ahead: every request's token is the one ``previous`` sampled, taken on the device."""
        entries = []
        sampling = []
        for item in plan.scheduled:
            request = item.request
            if previous is None:
                tokens = request.all_token_ids[item.start:item.start + item.num_tokens]
            else:
                tokens = [0]                    # replaced on the device
            entries.append(StepEntry(request.request_id, tokens, item.start,
                                     [item.num_tokens - 1] if item.samples else []))
            if item.samples:
                sampling.append(request)
        last = None
        if previous is not None:
            row_of = {request.request_id: row for row, request in enumerate(previous.sampling)}
            rows = [row_of[item.request.request_id] for item in plan.scheduled]
            logits = self.decode_graphs.run(entries, device_tokens=(previous.tokens, rows))
            last = (previous.tokens, [row_of[request.request_id] for request in sampling])
        elif self.decode_graphs is not None and self.decode_graphs.accepts(entries):
            logits = self.decode_graphs.run(entries)
        elif self.mixed_graphs is not None:
            logits = self.mixed_graphs.run(entries)
        else:
            logits = self.runner.step(entries)
        if self._first_inputs is None:
            self._first_inputs = self._describe_inputs(plan)
        if not sampling:
            return _InFlight(plan, [], None, None)
        on_gpu = self._carry_status
        tokens = self.sampler.sample_device(
            logits, [r.sampling_params for r in sampling], [r.seed for r in sampling],
            [r.prompt_token_ids for r in sampling], [r.output_token_ids for r in sampling],
            ahead=0 if previous is None else 1, extra=kernels.STATUS_WORDS if on_gpu else 0,
            keys=[r.request_id for r in sampling], last=last)
        if on_gpu:
            self.runner.write_status(tokens[len(sampling):len(sampling) + kernels.STATUS_WORDS])
        return _InFlight(plan, sampling, tokens, self._pinned(tokens.shape[0]), has_status=on_gpu,
                         logprob_width=Sampler.logprob_width([r.sampling_params for r in sampling]))

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
        self.mixed_graphs = None


class LLM:
    """``LLM(folder, dtype="bfloat16").generate([[1, 2, 3], ...], SamplingParams(...))``."""

    def __init__(self, model: str | Path, dtype: str = "bfloat16", max_model_len: int = 4096,
                 block_size: int = 16, num_gpu_blocks: int | None = None, max_num_seqs: int = 8,
                 max_num_batched_tokens: int = 2048, enable_prefix_caching: bool = False,
                 enforce_eager: bool = False, seed: int = 0, device: str = "cuda",
                 async_scheduling: bool = True, tokenizer=None) -> None:
        if num_gpu_blocks is None:
            num_gpu_blocks = max_num_seqs * -(-max_model_len // block_size)
        self.engine = LLMEngine(EngineConfig(
            ModelConfig(str(model), dtype, max_model_len, enforce_eager, seed),
            CacheConfig(block_size, num_gpu_blocks, enable_prefix_caching),
            SchedulerConfig(max_num_seqs, max_num_batched_tokens, async_scheduling=async_scheduling), device),
            tokenizer=tokenizer)
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
