"""A request as the scheduler sees it, and what the engine hands back.

State and names follow minivllm/request.py:67-258 (status values, the single
place where output tokens are appended, ``num_computed_tokens``) and
minivllm/outputs.py:36-201 (``RequestOutput``, ``FinishReason``).
"""

from __future__ import annotations

import enum
from dataclasses import dataclass, field

from ..sampling.params import SamplingParams


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    PREEMPTED = "preempted"
    FINISHED_STOPPED = "finished_stopped"
    FINISHED_LENGTH_CAPPED = "finished_length_capped"
    FINISHED_ABORTED = "finished_aborted"

    @property
    def finished(self) -> bool:
        return self.name.startswith("FINISHED")


class FinishReason(enum.Enum):
    STOP = "stop"
    LENGTH = "length"
    ABORT = "abort"


@dataclass
class Logprob:
    """What is reported of one token at one generated position (minivllm/logprobs.py:30-37):
    its log-probability and its place among all tokens (1: the most likely)."""

    logprob: float
    rank: int | None = None
    decoded_token: str | None = None


_REASON = {
    RequestStatus.FINISHED_STOPPED: FinishReason.STOP,
    RequestStatus.FINISHED_LENGTH_CAPPED: FinishReason.LENGTH,
    RequestStatus.FINISHED_ABORTED: FinishReason.ABORT,
}


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling_params: SamplingParams
    arrival_time: float = 0.0
    priority: int = 0
    seed: int = 0                                   # resolved: the request's own or drawn by the engine
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    num_computed_tokens: int = 0
    num_preemptions: int = 0
    stop_reason: int | None = None
    # With SamplingParams.logprobs: per generated token a dict from token id to Logprob, the
    # generated token and the most likely ones (minivllm/logprobs.py:50-76), and the sum of the
    # generated tokens' log-probabilities.
    logprobs: list[dict[int, Logprob]] | None = None
    cumulative_logprob: float | None = None

    def append_output(self, token: int, reported: tuple[list[int], list[float], int] | None = None) -> None:
        """The one place where a generated token is added.  ``reported``: the columns of the
        sampler's log-probabilities for it (ids and values, the generated token first, and its
        place)."""
        self.output_token_ids.append(int(token))
        wanted = self.sampling_params.logprobs
        if wanted is None:
            return
        if reported is None:
            raise RuntimeError(f"request {self.request_id!r} asked for log-probabilities and the step brought none")
        ids, values, place = reported
        if self.logprobs is None:
            self.logprobs, self.cumulative_logprob = [], 0.0
        # the generated token first, then the list with places 1, 2, ...: a token that is both keeps
        # the later entry, as in the reference's dict
        entry = {int(ids[0]): Logprob(float(values[0]), int(place))}
        for position in range(1, wanted + 1):
            if ids[position] >= 0:
                entry[int(ids[position])] = Logprob(float(values[position]), position)
        self.logprobs.append(entry)
        self.cumulative_logprob += float(values[0])

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def finish_reason(self) -> FinishReason | None:
        return _REASON.get(self.status)


@dataclass
class RequestOutput:
    """Cumulative result of one request after a step."""

    request_id: str
    prompt_token_ids: list[int]
    token_ids: list[int]
    finished: bool
    finish_reason: FinishReason | None = None
    stop_reason: int | None = None
    num_preemptions: int = 0
    logprobs: list[dict[int, Logprob]] | None = None        # aligned with token_ids
    cumulative_logprob: float | None = None
    text: str | None = None                                 # of token_ids, where the engine has a tokenizer


def check_stop(request: Request, max_model_len: int) -> bool:
    """Decide after a new token whether the request is over
    (minivllm/core/sched/utils.py:18-47): too few tokens yet -> go on; eos (unless
    ignored) or a stop id -> stopped; context or ``max_tokens`` reached -> capped."""
    params = request.sampling_params
    produced = len(request.output_token_ids)
    if produced < params.min_tokens:
        return False
    last = request.output_token_ids[-1]
    if not params.ignore_eos and params.eos_token_id is not None and last == params.eos_token_id:
        request.status = RequestStatus.FINISHED_STOPPED
        return True
    if last in params.stop_token_ids:
        request.status = RequestStatus.FINISHED_STOPPED
        request.stop_reason = last
        return True
    if request.num_tokens >= max_model_len or produced >= params.max_tokens:
        request.status = RequestStatus.FINISHED_LENGTH_CAPPED
        return True
    return False
