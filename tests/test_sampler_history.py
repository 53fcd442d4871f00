"""What the sampler hands to the penalties kernel: the distinct tokens a request has seen and how
often each was generated (minivllm/sample/ops/penalties.py:51-72 counts them anew every step),
counted anew or kept up from step to step under the request's key."""

from __future__ import annotations

import random
from collections import Counter

import numpy as np
import torch

from vllm_from_scratch_b200 import kernels
from vllm_from_scratch_b200.sampling import SamplingParams
from vllm_from_scratch_b200.sampling.sampler import Sampler


def expected(prompts, outputs, with_penalties):
    offsets, seen, counts = [0], [], []
    for prompt, output, on in zip(prompts, outputs, with_penalties):
        if on:
            generated = Counter(output)
            for token in sorted(set(prompt) | set(generated)):
                seen.append(token)
                counts.append(generated.get(token, 0))
        offsets.append(len(seen))
    return offsets, seen, counts


def test_seen_tokens_kept_up_or_counted_anew(monkeypatch):
    calls = []
    monkeypatch.setattr(kernels, "apply_penalties",
                        lambda logits, offsets, seen, counts, *rest: calls.append(
                            (offsets.tolist(), seen.tolist(), counts.tolist())))
    monkeypatch.setattr(kernels, "sample", lambda *args: None)
    vocab = 97
    rng = random.Random(5)
    sampler = Sampler(vocab, "cpu")
    params = [SamplingParams(repetition_penalty=1.2), SamplingParams(), SamplingParams(frequency_penalty=0.5),
              SamplingParams(presence_penalty=0.3)]
    on = [p.has_penalties for p in params]
    prompts = [[rng.randrange(vocab) for _ in range(n)] for n in (40, 7, 1, 90)]
    outputs = [[], [], [rng.randrange(vocab) for _ in range(50)], []]       # one joins with a history (a resumed request)
    keys = ["a", "b", "c", "d"]
    logits = torch.zeros(4, vocab)
    for step in range(60):
        for use_keys in (True, False):
            calls.clear()
            sampler.sample_device(logits, params, [1, 2, 3, 4], prompts, outputs, keys=keys if use_keys else None)
            assert calls == [expected(prompts, outputs, on)], (step, use_keys)
        for output in outputs:
            output.append(rng.randrange(vocab))
        if step == 30:
            # "d" ends and its key names a new request with another prompt
            sampler.forget("d")
            prompts[3] = [rng.randrange(vocab) for _ in range(12)]
            outputs[3] = []
    # a key whose request was never forgotten but whose output is shorter than what was counted
    outputs[0] = outputs[0][:3]
    calls.clear()
    sampler.sample_device(logits, params, [1, 2, 3, 4], prompts, outputs, keys=keys)
    assert calls == [expected(prompts, outputs, on)]


def test_no_penalties_no_call(monkeypatch):
    monkeypatch.setattr(kernels, "apply_penalties", lambda *args: (_ for _ in ()).throw(AssertionError("called")))
    monkeypatch.setattr(kernels, "sample", lambda *args: None)
    sampler = Sampler(11, "cpu")
    sampler.sample_device(torch.zeros(1, 11), [SamplingParams()], [0], [[1, 2]], [[3]], keys=["x"])
    assert not sampler._seen
