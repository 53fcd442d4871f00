"""The scheduler: which requests run in the next step and with how many tokens.

Policy as in the reference (minivllm/core/sched/scheduler.py:214-421):

* one token budget per step, shared by everything in it; a request gets
  ``min(tokens it still has to compute, budget left)``, so a long prompt is cut
  into portions by the budget alone and portions share steps with decoding
  requests (:423-445);
* running requests first, in their order, then waiting ones while there is
  budget, a free place among ``max_num_seqs`` and no preemption in this step
  (:307-351);
* when the pages run out for a running request, a victim is preempted: the last
  of the running list (policy "fcfs") or the one of lowest urgency (policy
  "priority"); it loses its pages and its progress, goes to the front of the
  waiting queue and is computed again from its first token when readmitted; a
  victim already planned for this step is unplanned and its tokens are refunded
  (:247-281, 483-515);
* two steps in a row that schedule nothing while requests remain raise, with the
  reason (:519-543).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..config.engine_config import SchedulerConfig
from .request import Request, RequestOutput, RequestStatus, check_stop


@dataclass
class ScheduledRequest:
    request: Request
    start: int              # tokens already in the cache before this step
    num_tokens: int         # tokens computed in this step
    samples: bool           # True when this step reaches the request's last known token
    resumed: bool = False   # readmitted after a preemption (or admitted for the first time)


@dataclass
class SchedulerOutput:
    scheduled: list[ScheduledRequest] = field(default_factory=list)
    preempted_ids: list[str] = field(default_factory=list)
    finished_ids: list[str] = field(default_factory=list)

    @property
    def total_num_scheduled_tokens(self) -> int:
        return sum(item.num_tokens for item in self.scheduled)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager, max_model_len: int,
                 trace_length: int = 256) -> None:
        self.config, self.cache, self.max_model_len = config, cache, max_model_len
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.requests: dict[str, Request] = {}
        self._finished_since_last: list[str] = []
        self._idle_steps = 0
        self.num_preemptions = 0
        self.step_count = 0
        self.trace: deque[dict] = deque(maxlen=trace_length)

    # ----------------------------------------------------------------- requests
    def add_request(self, request: Request) -> None:
        if request.request_id in self.requests:
            raise ValueError(f"request id {request.request_id!r} is already in use")
        if request.request_id in self._finished_since_last:
            # minivllm/core/sched/scheduler.py:163-170: an id may be used again only after the
            # notice that its last holder has finished went out with a step's plan; until then
            # one plan would name the id both as finished and as new.
            raise ValueError(f"request id {request.request_id!r} has just finished and its notice has not "
                             f"gone out with a step yet: use it again after the next step")
        if not request.prompt_token_ids:
            raise ValueError("a request needs at least one prompt token")
        if len(request.prompt_token_ids) >= self.max_model_len:
            raise ValueError(f"prompt of {len(request.prompt_token_ids)} tokens does not fit "
                             f"max_model_len={self.max_model_len}")
        pages = -(-(len(request.prompt_token_ids) + 1) // self.cache.page_size)
        smallest = min((pool.num_pages for pool in self.cache.pools), default=pages)
        if pages > smallest and all(w is None for w in self.cache.group_windows):
            raise ValueError(f"request {request.request_id!r} needs {pages} pages for its prompt alone; "
                             f"the pool has {smallest}")
        request.status = RequestStatus.WAITING
        self.requests[request.request_id] = request
        self._enqueue(request, front=False)

    def _enqueue(self, request: Request, front: bool) -> None:
        if self.config.policy == "priority":
            items = sorted([*self.waiting, request], key=lambda r: (r.priority, r.arrival_time))
            self.waiting = deque(items)
        elif front:
            self.waiting.appendleft(request)
        else:
            self.waiting.append(request)

    def has_unfinished_requests(self) -> bool:
        return bool(self.waiting or self.running)

    def finish_requests(self, request_ids, status: RequestStatus = RequestStatus.FINISHED_ABORTED) -> None:
        for request_id in ([request_ids] if isinstance(request_ids, str) else list(request_ids)):
            request = self.requests.get(request_id)
            if request is None or request.status.finished:
                continue
            if request in self.running:
                self.running.remove(request)
            else:
                self.waiting = deque(r for r in self.waiting if r is not request)
            request.status = status
            self._free(request)

    def _free(self, request: Request) -> None:
        if self.cache.is_admitted(request.request_id):
            self.cache.release(request.request_id)
        self.requests.pop(request.request_id, None)
        self._finished_since_last.append(request.request_id)

    # ----------------------------------------------------------------- schedule
    def _new_tokens(self, request: Request, start: int, budget: int) -> int:
        return max(0, min(request.num_tokens - start, budget))

    def _pick_victim(self) -> Request:
        if self.config.policy == "priority":
            return max(self.running, key=lambda r: (r.priority, r.arrival_time))
        return self.running[-1]

    def _preempt(self, request: Request, output: SchedulerOutput) -> None:
        self.cache.release(request.request_id)
        request.status = RequestStatus.PREEMPTED
        request.num_computed_tokens = 0
        request.num_preemptions += 1
        self.num_preemptions += 1
        output.preempted_ids.append(request.request_id)
        self._enqueue(request, front=True)

    def schedule(self) -> SchedulerOutput:
        output = SchedulerOutput(finished_ids=self._finished_since_last)
        self._finished_since_last = []
        budget = self.config.max_num_batched_tokens
        planned: dict[str, ScheduledRequest] = {}

        for request in list(self.running):
            if budget <= 0:
                break
            if request not in self.running:          # preempted earlier in this loop
                continue
            start = request.num_computed_tokens
            count = self._new_tokens(request, start, budget)
            if count == 0:
                continue
            allocated = False
            while True:
                if self.cache.allocate(request.request_id, start + count):
                    allocated = True
                    break
                victim = self._pick_victim()
                self.running.remove(victim)
                plan = planned.pop(victim.request_id, None)
                if plan is not None:
                    budget += plan.num_tokens
                self._preempt(victim, output)
                if victim is request:
                    break
            if not allocated:
                break
            planned[request.request_id] = ScheduledRequest(
                request, start, count, samples=start + count == request.num_tokens)
            budget -= count

        while (self.waiting and budget > 0 and not output.preempted_ids
               and len(self.running) < self.config.max_num_seqs):
            request = self.waiting[0]
            if self.cache.num_free_slots == 0:
                break
            self.cache.admit(request.request_id)
            tokens = request.all_token_ids
            start = self.cache.match_prefix(request.request_id, tokens)
            count = self._new_tokens(request, start, budget)
            if count == 0 or not self.cache.allocate(request.request_id, start + count):
                self.cache.release(request.request_id)       # nothing changed for this request
                break
            self.waiting.popleft()
            request.status = RequestStatus.RUNNING
            request.num_computed_tokens = start
            self.running.append(request)
            planned[request.request_id] = ScheduledRequest(
                request, start, count, samples=start + count == request.num_tokens, resumed=True)
            budget -= count

        # Keep the running list's order in the batch.
        output.scheduled = [planned[r.request_id] for r in self.running if r.request_id in planned]
        for item in output.scheduled:
            item.request.num_computed_tokens = item.start + item.num_tokens
        self._check_progress(output)
        self.step_count += 1
        self.trace.append({
            "step": self.step_count,
            "scheduled": {item.request.request_id: item.num_tokens for item in output.scheduled},
            "preempted": list(output.preempted_ids),
            "running": len(self.running), "waiting": len(self.waiting),
            "free_pages": [pool.num_free for pool in self.cache.pools],
        })
        return output

    def schedule_ahead(self, previous: SchedulerOutput) -> SchedulerOutput | None:
        """The decode step after ``previous``, planned while ``previous`` still runs: every
        request of it that cannot end by length goes on with the one token that
        ``previous`` samples, which the host does not know yet.  Declines (``None``)
        whenever that is not plainly the next step: something waits, ``previous`` was not
        a pure decode step or preempted, or a page is missing (no preemption on a guess)."""
        if self.waiting or previous.preempted_ids or not previous.scheduled:
            return None
        if len(previous.scheduled) != len(self.running):
            return None
        chosen: list[Request] = []
        for item in previous.scheduled:
            request = item.request
            if (not item.samples or item.num_tokens != 1 or request.status is not RequestStatus.RUNNING
                    or request.num_computed_tokens != request.num_tokens):
                return None
            produced = len(request.output_token_ids) + 1            # with the token in flight
            if produced >= request.sampling_params.max_tokens or request.num_tokens + 1 >= self.max_model_len:
                continue                                            # ends by length when that token arrives
            chosen.append(request)
        if not chosen:
            return None
        for request in chosen:
            if not self.cache.allocate(request.request_id, request.num_computed_tokens + 1):
                return None             # pages taken so far stay with their requests for the next step
        output = SchedulerOutput(finished_ids=[])
        for request in chosen:
            output.scheduled.append(ScheduledRequest(request, request.num_computed_tokens, 1, samples=True))
            request.num_computed_tokens += 1
        self.step_count += 1
        self.trace.append({
            "step": self.step_count,
            "scheduled": {item.request.request_id: 1 for item in output.scheduled},
            "preempted": [], "running": len(self.running), "waiting": 0,
            "free_pages": [pool.num_free for pool in self.cache.pools], "ahead": True,
        })
        return output

    def _check_progress(self, output: SchedulerOutput) -> None:
        if output.total_num_scheduled_tokens or not self.has_unfinished_requests():
            self._idle_steps = 0
            return
        self._idle_steps += 1
        if self._idle_steps >= 2:
            head = self.waiting[0] if self.waiting else None
            detail = ""
            if head is not None:
                need = -(-(head.num_tokens + 1) // self.cache.page_size)
                detail = (f"; the first waiting request {head.request_id!r} has {head.num_tokens} tokens "
                          f"({need} pages) and the pools have "
                          f"{[pool.num_free for pool in self.cache.pools]} pages free of "
                          f"{[pool.num_pages for pool in self.cache.pools]}")
            raise RuntimeError(
                f"the scheduler made no progress in two consecutive steps with "
                f"{len(self.running)} running and {len(self.waiting)} waiting requests{detail}")

    # ------------------------------------------------------------------- update
    def update(self, output: SchedulerOutput, sampled: dict[str, int],
               logprobs: dict[str, tuple[list[int], list[float], int]] | None = None) -> list[RequestOutput]:
        """Commit the step's results: append sampled tokens (with their log-probabilities where
        a request asked for them), decide who is over, give their pages back, publish full pages
        (minivllm/core/sched/scheduler.py:596-733)."""
        results: list[RequestOutput] = []
        for item in output.scheduled:
            request = item.request
            if request.status is not RequestStatus.RUNNING:
                continue                        # aborted between schedule and update
            finished = False
            if item.samples:
                if request.request_id not in sampled:
                    raise RuntimeError(f"no token was sampled for request {request.request_id!r}")
                request.append_output(sampled[request.request_id], (logprobs or {}).get(request.request_id))
                finished = check_stop(request, self.max_model_len)
            # Publish full pages first: they stay hittable after the request is gone.
            self.cache.commit(request.request_id, request.num_computed_tokens, request.all_token_ids)
            if finished:
                self.running.remove(request)
                self._free(request)
            if item.samples:
                results.append(RequestOutput(
                    request.request_id, request.prompt_token_ids, list(request.output_token_ids), finished,
                    request.finish_reason, request.stop_reason, request.num_preemptions,
                    None if request.logprobs is None else list(request.logprobs), request.cumulative_logprob))
        return results

    # -------------------------------------------------------------------- trace
    def format_trace(self) -> str:
        lines = ["step  running waiting  free_pages  scheduled (request: tokens)  preempted"]
        for row in self.trace:
            plan = ", ".join(f"{rid}: {n}" for rid, n in row["scheduled"].items()) or "-"
            lines.append(f"{row['step']:>4}  {row['running']:>7} {row['waiting']:>7}  "
                         f"{str(row['free_pages']):>10}  {plan}  {','.join(row['preempted']) or '-'}")
        return "\n".join(lines)
