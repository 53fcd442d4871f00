"""The scheduler's decisions, driven without a model: a scripted "runner" hands
back tokens.  Budget, portions, order, preemption with refund, the guard against
standing still, stop conditions."""

from __future__ import annotations

import pytest

from vllm_from_scratch_b200 import (CacheManager, Request, RequestStatus, SamplingParams, Scheduler,
                                    SchedulerConfig)
from vllm_from_scratch_b200.engine.request import check_stop


def make(pages=16, page_size=4, seqs=4, budget=16, policy="fcfs", max_len=64, prefix=False, windows=(None,)):
    cache = CacheManager(list(windows), page_size, pages, seqs, enable_prefix_caching=prefix)
    return Scheduler(SchedulerConfig(seqs, budget, policy), cache, max_len), cache


def request(name, prompt_len, max_tokens=4, priority=0, arrival=0.0, **params):
    return Request(name, list(range(1, prompt_len + 1)),
                   SamplingParams(temperature=0.0, max_tokens=max_tokens, **params),
                   arrival_time=arrival, priority=priority)


def run_step(scheduler, token=9):
    plan = scheduler.schedule()
    sampled = {item.request.request_id: token for item in plan.scheduled if item.samples}
    return plan, scheduler.update(plan, sampled)


def planned(plan):
    return {item.request.request_id: (item.start, item.num_tokens, item.samples) for item in plan.scheduled}


def test_budget_cuts_prompts_into_portions_and_shares_steps():
    scheduler, cache = make(budget=16)
    scheduler.add_request(request("a", 10))
    scheduler.add_request(request("b", 20))
    plan, outs = run_step(scheduler)
    assert planned(plan) == {"a": (0, 10, True), "b": (0, 6, False)}
    assert [o.request_id for o in outs] == ["a"]
    plan, outs = run_step(scheduler)
    # running requests first: a decodes one token, b takes what is left of the budget
    assert planned(plan) == {"a": (10, 1, True), "b": (6, 14, True)}
    plan, outs = run_step(scheduler)
    assert planned(plan) == {"a": (11, 1, True), "b": (20, 1, True)}
    cache.check_invariants()


def test_max_num_seqs_and_fcfs_order():
    scheduler, _ = make(seqs=2, budget=64)
    for name in "abc":
        scheduler.add_request(request(name, 3, max_tokens=2))
    plan, _ = run_step(scheduler)
    assert list(planned(plan)) == ["a", "b"]
    plan, outs = run_step(scheduler)            # a and b reach max_tokens = 2 and finish
    assert all(o.finished and o.finish_reason.name == "LENGTH" for o in outs)
    plan, _ = run_step(scheduler)
    assert list(planned(plan)) == ["c"]
    assert plan.finished_ids == ["a", "b"]


def test_preemption_takes_the_last_running_and_recomputes_it():
    scheduler, cache = make(pages=6, page_size=4, budget=64)
    scheduler.add_request(request("a", 8, max_tokens=12))
    scheduler.add_request(request("b", 8, max_tokens=12))
    run_step(scheduler)                          # 2 + 2 pages; 2 left
    for _ in range(4):
        plan, _ = run_step(scheduler)            # positions 8..11 fit in the third page of each
    assert cache.num_free_pages() == 0
    plan, _ = run_step(scheduler)                # a needs a fourth page: b is preempted
    assert plan.preempted_ids == ["b"] and list(planned(plan)) == ["a"]
    victim = scheduler.waiting[0]
    assert victim.request_id == "b" and victim.status is RequestStatus.PREEMPTED
    assert victim.num_computed_tokens == 0 and len(victim.output_token_ids) == 5
    assert not cache.is_admitted("b")
    cache.check_invariants()
    # a runs on; b comes back only when pages are free, and then from its first token
    resumed = None
    for _ in range(20):
        plan, _ = run_step(scheduler)
        if "b" in planned(plan):
            resumed = planned(plan)["b"]
            break
    assert resumed is not None and resumed[0] == 0 and resumed[1] == 8 + 5
    assert scheduler.num_preemptions == 1


def test_preempted_plan_is_refunded_under_priority_policy():
    scheduler, cache = make(pages=5, page_size=4, budget=10, policy="priority")
    scheduler.add_request(request("low", 8, max_tokens=8, priority=5))
    run_step(scheduler)                           # low: 2 pages
    scheduler.add_request(request("high", 8, max_tokens=8, priority=0))
    run_step(scheduler)                           # low decodes (pos 8: third page), high prefills 2 pages
    assert cache.num_free_pages() == 0
    for _ in range(3):
        run_step(scheduler)                       # both decode inside their pages (high: pos 8 needs a page!)
    # by now one of them had to be preempted: it must be the low-priority one
    assert scheduler.num_preemptions >= 1
    assert all(r.request_id != "high" for r in scheduler.waiting)
    cache.check_invariants()


def test_no_progress_raises_with_a_reason():
    scheduler, _ = make(pages=2, page_size=4, budget=64, windows=(8,))
    # a windowed pool is not checked at admission; a prompt of 12 needs 3 pages at once
    scheduler.add_request(request("big", 12))
    scheduler.schedule()
    with pytest.raises(RuntimeError, match="no progress"):
        scheduler.schedule()


def test_admission_checks():
    scheduler, _ = make(pages=2, page_size=4, max_len=16)
    with pytest.raises(ValueError, match="at least one"):
        scheduler.add_request(request("e", 0))
    with pytest.raises(ValueError, match="max_model_len"):
        scheduler.add_request(request("l", 16))
    with pytest.raises(ValueError, match="pages"):
        scheduler.add_request(request("p", 12))
    scheduler.add_request(request("ok", 4))
    with pytest.raises(ValueError, match="already"):
        scheduler.add_request(request("ok", 4))


def test_stop_conditions():
    def outcome(tokens, **params):
        r = request("s", 3, **params)
        for t in tokens:
            r.output_token_ids.append(t)
            if check_stop(r, max_model_len=10):
                return r.status, r.stop_reason, len(r.output_token_ids)
        return None
    assert outcome([5, 7], max_tokens=8, eos_token_id=7) == (RequestStatus.FINISHED_STOPPED, None, 2)
    assert outcome([5, 7, 1], max_tokens=3, eos_token_id=7, ignore_eos=True)[0] is RequestStatus.FINISHED_LENGTH_CAPPED
    assert outcome([5, 6], max_tokens=8, stop_token_ids=[6]) == (RequestStatus.FINISHED_STOPPED, 6, 2)
    assert outcome([7, 7, 7], max_tokens=8, eos_token_id=7, min_tokens=3) == (RequestStatus.FINISHED_STOPPED, None, 3)
    assert outcome([1] * 9, max_tokens=50)[2] == 7          # 3 prompt + 7 = max_model_len 10


def test_abort_and_trace():
    scheduler, cache = make()
    scheduler.add_request(request("a", 5))
    scheduler.add_request(request("b", 5))
    run_step(scheduler)
    scheduler.finish_requests("a")
    assert not cache.is_admitted("a")
    plan, _ = run_step(scheduler)
    assert "a" in plan.finished_ids and list(planned(plan)) == ["b"]
    assert "b: 1" in scheduler.format_trace()
    cache.check_invariants()


def test_prefix_hit_shortens_the_second_prompt():
    scheduler, cache = make(pages=16, page_size=4, budget=64, prefix=True)
    scheduler.add_request(request("a", 13, max_tokens=1))
    run_step(scheduler)
    scheduler.add_request(request("b", 13, max_tokens=1))
    plan, _ = run_step(scheduler)
    assert planned(plan)["b"] == (12, 1, True)


# --------------------------------------------------------- a step planned ahead
def _decoding(scheduler, names_and_lengths, **params):
    for name, length in names_and_lengths:
        scheduler.add_request(request(name, length, **params))
    run_step(scheduler)                          # prompts
    return scheduler.schedule()                  # the first pure decode step, not yet updated


def test_schedule_ahead_continues_every_request_with_the_token_in_flight():
    scheduler, cache = make(budget=16)
    plan = _decoding(scheduler, [("a", 3), ("b", 5)], max_tokens=10)
    assert planned(plan) == {"a": (3, 1, True), "b": (5, 1, True)}
    ahead = scheduler.schedule_ahead(plan)
    # the token that `plan` samples is the input: it sits at the next position
    assert planned(ahead) == {"a": (4, 1, True), "b": (6, 1, True)}
    outs = scheduler.update(plan, {"a": 7, "b": 7})
    assert [len(o.token_ids) for o in outs] == [2, 2]
    again = scheduler.schedule_ahead(ahead)
    assert planned(again) == {"a": (5, 1, True), "b": (7, 1, True)}
    scheduler.update(ahead, {"a": 8, "b": 8})
    scheduler.update(again, {"a": 9, "b": 9})
    assert scheduler.requests["a"].output_token_ids == [9, 7, 8, 9]
    # nothing in flight any more: the ordinary schedule goes on from the same place
    assert planned(scheduler.schedule()) == {"a": (6, 1, True), "b": (8, 1, True)}
    cache.check_invariants()


def test_schedule_ahead_leaves_out_what_ends_by_length_and_declines_when_unsure():
    scheduler, cache = make(budget=16)
    scheduler.add_request(request("short", 3, max_tokens=2))
    scheduler.add_request(request("long", 3, max_tokens=9))
    run_step(scheduler)
    plan = scheduler.schedule()
    ahead = scheduler.schedule_ahead(plan)       # "short" gets its second and last token from `plan`
    assert planned(ahead) == {"long": (4, 1, True)}
    outs = scheduler.update(plan, {"short": 5, "long": 5})
    assert [o.finished for o in outs] == [True, False]
    # a request that stops on a token while its next step is queued: that step's result is dropped
    stopper, _ = make(budget=16)
    stopper.add_request(request("s", 3, max_tokens=9, stop_token_ids=[42]))
    run_step(stopper)
    plan = stopper.schedule()
    ahead = stopper.schedule_ahead(plan)
    outs = stopper.update(plan, {"s": 42})
    assert outs[0].finished and outs[0].finish_reason.name == "STOP"
    assert stopper.update(ahead, {"s": 1}) == [] and not stopper.has_unfinished_requests()
    stopper.cache.check_invariants()
    assert stopper.cache.stats()["requests"] == 0

    # declines: someone waits; a prompt portion was in the step; no page left
    waiting, _ = make(seqs=1, budget=16)
    plan = _decoding(waiting, [("a", 3), ("b", 3)], max_tokens=9)
    assert waiting.schedule_ahead(plan) is None
    portion, _ = make(budget=4)
    portion.add_request(request("a", 3, max_tokens=9))
    portion.add_request(request("b", 9, max_tokens=9))
    run_step(portion)
    assert portion.schedule_ahead(portion.schedule()) is None
    # penalties do not keep a step from being planned ahead: the sampler counts the token in flight on the device
    penal, _ = make(budget=16)
    assert penal.schedule_ahead(_decoding(penal, [("a", 3)], max_tokens=9, repetition_penalty=1.2)) is not None
    full, cache = make(pages=2, page_size=4, budget=16)
    plan = _decoding(full, [("a", 7)], max_tokens=9)         # 8 tokens fill both pages
    assert full.schedule_ahead(plan) is None
    cache.check_invariants()


def test_an_id_is_free_again_only_after_its_finished_notice_went_out():
    """minivllm/core/sched/scheduler.py:163-170: between the end of a request and the next plan
    (which carries the notice that it finished) its id is refused."""
    scheduler, _ = make(pages=16)
    scheduler.add_request(request("r", 5, max_tokens=1))
    plan = scheduler.schedule()
    scheduler.update(plan, {"r": 7})
    assert not scheduler.has_unfinished_requests()
    with pytest.raises(ValueError, match="has just finished"):
        scheduler.add_request(request("r", 3))
    assert scheduler.schedule().finished_ids == ["r"]
    scheduler.add_request(request("r", 3))
    with pytest.raises(ValueError, match="already in use"):
        scheduler.add_request(request("r", 3))


def test_logprobs_travel_with_the_tokens():
    """``SamplingParams.logprobs`` within what is built; a step's columns of log-probabilities become
    one dict per generated token (minivllm/logprobs.py:50-76): the generated token with its place,
    then the list with places 1, 2, ..., a token that is both keeping the list's entry."""
    from vllm_from_scratch_b200.engine.request import Logprob
    for bad in (-1, 33):
        with pytest.raises(NotImplementedError):
            SamplingParams(logprobs=bad)
    scheduler, _ = make(budget=16)
    scheduler.add_request(request("a", 3, max_tokens=3, logprobs=2))
    scheduler.add_request(request("b", 3, max_tokens=3))
    plan = scheduler.schedule()
    outputs = scheduler.update(plan, {"a": 7, "b": 8}, {"a": ([7, 9, 7], [-1.5, -0.25, -1.5], 2)})
    by_id = {o.request_id: o for o in outputs}
    assert by_id["b"].logprobs is None and by_id["b"].cumulative_logprob is None
    assert by_id["a"].logprobs == [{7: Logprob(-1.5, 2), 9: Logprob(-0.25, 1)}]
    assert by_id["a"].cumulative_logprob == -1.5
    plan = scheduler.schedule()
    outputs = scheduler.update(plan, {"a": 4, "b": 8}, {"a": ([4, 9, 1], [-3.0, -0.5, -1.0], 5)})
    a = {o.request_id: o for o in outputs}["a"]
    assert a.logprobs[1] == {4: Logprob(-3.0, 5), 9: Logprob(-0.5, 1), 1: Logprob(-1.0, 2)}
    assert a.cumulative_logprob == -4.5 and len(a.logprobs) == len(a.token_ids) == 2
    with pytest.raises(RuntimeError, match="log-probabilities"):
        scheduler.update(scheduler.schedule(), {"a": 1, "b": 2})
