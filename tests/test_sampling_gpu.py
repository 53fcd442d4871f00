"""The sampling kernels against the reference's formulas written in plain tensor
code (minivllm/sample/ops/topk_topp_sampler.py:48-90, minivllm/sample/sampler.py:
290-303, minivllm/sample/ops/penalties.py:51-72)."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def plain_keep_mask(logits, temperature, top_k, top_p, min_p):
    """Which tokens survive temperature -> min_p -> top-k -> top-p, one row."""
    x = logits.double() / temperature
    keep = torch.ones_like(x, dtype=torch.bool)
    if min_p > 0:
        probs = torch.softmax(x, dim=-1)
        keep &= probs >= probs.max() * min_p
        x = x.masked_fill(~keep, float("-inf"))
    if top_k > 0 and top_k < x.numel():
        kth = torch.topk(x, top_k).values[-1]
        keep &= x >= kth
        x = x.masked_fill(~keep, float("-inf"))
    if top_p < 1.0:
        order = torch.argsort(x)                       # ascending
        probs = torch.softmax(x, dim=-1)[order]
        drop = torch.cumsum(probs, dim=-1) <= 1 - top_p
        drop[-1] = False
        keep[order[drop]] = False
    return keep


def draw(logits_row, n, temperature, top_k=0, top_p=1.0, min_p=0.0, seed0=0):
    import vllm_from_scratch_b200.kernels as k
    vocab = logits_row.numel()
    logits = logits_row.float().cuda().unsqueeze(0).repeat(n, 1).contiguous()
    f = lambda v, dt: torch.full((n,), v, dtype=dt, device="cuda")
    seeds = torch.arange(seed0, seed0 + n, dtype=torch.int64, device="cuda")
    index = torch.arange(n, dtype=torch.int64, device="cuda") % 7
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    k.sample(logits, f(temperature, torch.float32), f(top_k, torch.int32), f(top_p, torch.float32),
             f(min_p, torch.float32), seeds, index, out, 1e-5)
    return out.cpu().long()


@pytest.mark.parametrize("vocab", [256, 503, 151936])
def test_greedy_is_first_argmax(vocab):
    g = torch.Generator().manual_seed(vocab)
    row = torch.randn(vocab, generator=g)
    row[vocab // 3] = row[vocab // 2] = row.max() + 1.0       # a tie: the first index wins
    tokens = draw(row, 3, temperature=0.0)
    assert tokens.tolist() == [vocab // 3] * 3


@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [
    (1.0, 5, 1.0, 0.0), (0.7, 0, 0.9, 0.0), (1.3, 0, 1.0, 0.05), (0.8, 20, 0.8, 0.01), (1.0, 1, 1.0, 0.0),
    (1.0, 0, 0.3, 0.0),
])
def test_filters_keep_the_reference_set(temperature, top_k, top_p, min_p):
    g = torch.Generator().manual_seed(7)
    row = torch.randn(503, generator=g) * 2.0
    keep = plain_keep_mask(row, temperature, top_k, top_p, min_p)
    tokens = draw(row, 4096, temperature, top_k, top_p, min_p)
    assert bool(keep[tokens].all()), "a token outside the reference's candidate set was drawn"
    kept = int(keep.sum())
    if kept <= 8:
        assert set(tokens.tolist()) == set(keep.nonzero().flatten().tolist())


def test_distribution_follows_softmax():
    g = torch.Generator().manual_seed(3)
    row = torch.randn(311, generator=g) * 1.5
    n = 1 << 16
    tokens = draw(row, n, temperature=0.9)
    expected = torch.softmax(row.double() / 0.9, dim=-1)
    counts = torch.bincount(tokens, minlength=311).double()
    sigma = torch.sqrt(expected * (1 - expected) * n)
    z = (counts - expected * n).abs() / sigma.clamp(min=1.0)
    assert float(z.max()) < 5.0, f"worst deviation {float(z.max()):.2f} sigma"


def test_same_key_same_token_and_large_vocabulary():
    g = torch.Generator().manual_seed(1)
    row = torch.randn(151936, generator=g) * 3
    a = draw(row, 64, temperature=1.0, top_k=50, top_p=0.95)
    b = draw(row, 64, temperature=1.0, top_k=50, top_p=0.95)
    assert torch.equal(a, b)
    assert len(set(a.tolist())) > 3
    keep = plain_keep_mask(row, 1.0, 50, 0.95, 0.0)
    assert bool(keep[a].all())


@pytest.mark.parametrize("vocab,n", [(503, 12), (4096, 12), (151936, 12), (151936, 24), (50257, 70)])
def test_rows_with_and_without_filters_draw_alike(vocab, n):
    """Rows without a filter and rows with one run in different kernels.  A filter that keeps
    every token (top-k of the whole vocabulary) must give the token of the row without it, in
    one call with rows of both kinds and in calls that launch one kernel only.  (The number of
    rows decides how many blocks share a row with a filter: eight, four or two.)"""
    import vllm_from_scratch_b200.kernels as k
    g = torch.Generator().manual_seed(vocab)
    logits = (torch.randn(n, vocab, generator=g) * 2).cuda()
    logits[5] = float("-inf")                            # nothing to draw from: the first token
    seeds = torch.arange(100, 100 + n, dtype=torch.int64, device="cuda")
    index = torch.arange(n, dtype=torch.int64, device="cuda") % 5
    temperature = torch.full((n,), 0.8, device="cuda")
    temperature[3] = 0.0                                 # a greedy row among them
    ones, zeros = torch.ones(n, device="cuda"), torch.zeros(n, device="cuda")
    none = torch.zeros(n, dtype=torch.int32, device="cuda")
    whole = torch.full((n,), vocab, dtype=torch.int32, device="cuda")
    mixed = torch.where(torch.arange(n, device="cuda") % 2 == 0, none, whole)

    def run(top_k, kinds):
        out = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        k.sample(logits, temperature, top_k, ones, zeros, seeds, index, out, 1e-5, kinds)
        return out.cpu().tolist()

    plain, filtered = run(none, 1), run(whole, 3)
    assert plain == filtered == run(mixed, 3) == run(none, 3)
    assert plain[3] == int(logits[3].argmax()) and plain[5] == 0
    assert len(set(plain)) > 3
    with pytest.raises(k.KernelError):
        run(none, 0)


def test_a_rows_token_does_not_depend_on_the_batch():
    """Few rows get eight blocks each, many rows four or two: thresholds and draws are exact
    functions of the row, so a row's token is the same whichever company it keeps."""
    import vllm_from_scratch_b200.kernels as k
    vocab = 32003
    g = torch.Generator().manual_seed(8)
    many = (torch.randn(70, vocab, generator=g) * 2.5).cuda()
    settings = [(0.8, 40, 0.9, 0.0), (1.0, 0, 0.7, 0.0), (1.2, 7, 1.0, 0.0), (0.9, 0, 1.0, 0.03), (0.7, 0, 1.0, 0.0), (0.0, 0, 1.0, 0.0)]

    def run(rows):
        n = rows.shape[0]
        column = lambda j, kind: torch.tensor([settings[i % len(settings)][j] for i in range(n)], dtype=kind, device="cuda")
        out = torch.empty(n, dtype=torch.int32, device="cuda")
        k.sample(rows, column(0, torch.float32), column(1, torch.int32), column(2, torch.float32), column(3, torch.float32),
                 torch.arange(n, dtype=torch.int64, device="cuda") + 50, torch.arange(n, dtype=torch.int64, device="cuda") % 3,
                 out, 1e-5)
        return out.cpu().tolist()

    whole = run(many)
    assert run(many[:6].contiguous()) == whole[:6]
    assert run(many[:24].contiguous()) == whole[:24]
    assert len(set(whole)) > 20


def test_filters_refuse_a_vocabulary_beyond_their_counters():
    import vllm_from_scratch_b200.kernels as k
    row = torch.zeros(1 << 20)
    with pytest.raises(k.KernelError, match="vocabulary"):
        draw(row, 2, temperature=1.0, top_k=5)
    # rows without a filter take any size, when the caller says that there are no others
    logits = row.cuda().unsqueeze(0).contiguous()
    logits[0, 77] = 30.0
    one = lambda v, dt: torch.full((1,), v, dtype=dt, device="cuda")
    out = torch.empty(1, dtype=torch.int32, device="cuda")
    k.sample(logits, one(1.0, torch.float32), one(0, torch.int32), one(1.0, torch.float32), one(0.0, torch.float32),
             one(5, torch.int64), one(0, torch.int64), out, 1e-5, 1)
    assert int(out[0]) == 77


def _large_rows():
    g = torch.Generator().manual_seed(21)
    vocab = 151936
    spread = torch.randn(vocab, generator=g) * 3                 # thresholds fall into sparse coarse bins
    crowd = torch.randn(vocab, generator=g) * 0.01               # every token within 0.05: one crowded bin
    tail = torch.full((vocab,), -60.0)                           # all but a hundred tokens far below the maximum
    tail[torch.randperm(vocab, generator=g)[:100]] = torch.randn(100, generator=g)
    peaked = torch.randn(vocab, generator=g)
    peaked[torch.randperm(vocab, generator=g)[:6]] += torch.tensor([9.0, 8.5, 8.0, 7.5, 7.0, 6.5])
    flat = torch.randn(vocab, generator=g)                       # thousands of tokens in the bin of a top-p threshold
    ties = torch.zeros(vocab)                                    # no division of a bin tells these apart
    ties[torch.randperm(vocab, generator=g)[:3]] = torch.tensor([0.5, 0.25, 0.125])
    return {"spread": spread, "crowd": crowd, "tail": tail, "peaked": peaked, "flat": flat, "ties": ties}


@pytest.mark.parametrize("name,temperature,top_k,top_p,min_p", [
    ("spread", 1.0, 5, 1.0, 0.0), ("spread", 0.8, 300, 0.9, 0.0), ("spread", 1.0, 0, 0.999, 0.0),
    ("crowd", 1.0, 6, 1.0, 0.0), ("crowd", 1.0, 70000, 1.0, 0.0), ("crowd", 1.0, 0, 0.5, 0.0),
    ("crowd", 1.0, 50000, 0.7, 0.0), ("tail", 1.0, 500, 1.0, 0.0), ("tail", 1.0, 40, 0.9, 0.0),
    ("tail", 1.0, 0, 0.999999, 0.0), ("peaked", 1.0, 0, 0.6, 0.0), ("peaked", 1.3, 4, 0.95, 0.001),
    ("flat", 0.8, 0, 0.9, 0.0), ("flat", 0.8, 20000, 0.5, 0.0), ("flat", 1.0, 0, 0.999, 0.02),
    ("ties", 1.0, 3, 1.0, 0.0), ("ties", 1.0, 10, 1.0, 0.0), ("ties", 1.0, 0, 1.0, 0.9),
])
def test_filters_on_a_large_vocabulary(name, temperature, top_k, top_p, min_p):
    """The threshold search looks at the row coarsely first, divides a crowded bin again and
    then selects among the keys of one bin held in shared memory; a threshold in the far tail
    or among thousands of equal logits takes the path over the whole row.  All of them must
    keep the reference's set."""
    row = _large_rows()[name]
    keep = plain_keep_mask(row, temperature, top_k, top_p, min_p)
    tokens = draw(row, 2048, temperature, top_k, top_p, min_p)
    assert bool(keep[tokens].all()), "a token outside the reference's candidate set was drawn"
    kept = int(keep.sum())
    if kept <= 8:
        assert set(tokens.tolist()) == set(keep.nonzero().flatten().tolist())
    else:
        # a kept set that large cannot be hit by so few distinct tokens if the cut were far too high
        assert len(set(tokens.tolist())) >= min(kept, 64) // 2


def test_penalties_and_masks_follow_the_formula():
    import vllm_from_scratch_b200.kernels as k
    vocab = 503
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(3, vocab, generator=g)
    prompts = [[1, 2, 2, 400], [5], [7, 8]]
    outputs = [[2, 9, 9, 9], [], [8, 8, 502]]
    rep, freq, pres = [1.3, 1.0, 0.7], [0.2, 0.0, 0.5], [0.1, 0.0, 0.4]
    expected = logits.clone()
    for r in range(3):
        seen = set(prompts[r]) | set(outputs[r])
        for t in seen:
            v = expected[r, t]
            expected[r, t] = v / rep[r] if v > 0 else v * rep[r]
        for t in set(outputs[r]):
            expected[r, t] -= freq[r] * outputs[r].count(t) + pres[r]
    offsets, seen_tokens, counts = [0], [], []
    for r in range(3):
        for t in sorted(set(prompts[r]) | set(outputs[r])):
            seen_tokens.append(t)
            counts.append(outputs[r].count(t))
        offsets.append(len(seen_tokens))
    device = logits.cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device="cuda")
    k.apply_penalties(device, i32(offsets), i32(seen_tokens), i32(counts), f32(rep), f32(freq), f32(pres))
    assert torch.allclose(device.cpu(), expected, atol=1e-6)
    k.mask_tokens(device, i32([0, 2]), i32([17, 502]))
    assert device[0, 17] == float("-inf") and device[2, 502] == float("-inf")
    assert torch.isfinite(device[1]).all()


def test_penalties_count_a_token_that_is_still_on_the_device():
    """A step sampled ahead of the one before it lacks that step's token in its lists; the kernel
    takes it from the device.  Bit for bit what the lists with the token in them give: a token
    that was listed before (prompt only, or generated), one that is new, a row without penalties,
    a row without such a token."""
    import vllm_from_scratch_b200.kernels as k
    vocab = 311
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(5, vocab, generator=g) * 3
    prompts = [[1, 2, 2, 300], [5, 6], [7, 8], [3], [10, 11]]
    outputs = [[2, 9, 9], [6], [8, 8, 310], [], [12]]
    last = [9, 5, 44, 77, None]                     # generated again; from the prompt; new; a row without penalties; none
    rep, freq, pres = [1.3, 0.8, 1.0, 1.0, 1.1], [0.3, 0.7, 0.11, 0.0, 0.2], [0.1, 0.0, 0.4, 0.0, 0.3]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    f32 = lambda v: torch.tensor(v, dtype=torch.float32, device="cuda")

    def lists(generated):
        offsets, seen_tokens, counts = [0], [], []
        for r in range(5):
            for t in sorted(set(prompts[r]) | set(generated[r])):
                seen_tokens.append(t)
                counts.append(generated[r].count(t))
            offsets.append(len(seen_tokens))
        return i32(offsets), i32(seen_tokens), i32(counts)

    whole = logits.cuda()
    k.apply_penalties(whole, *lists([o + ([t] if t is not None else []) for o, t in zip(outputs, last)]),
                      f32(rep), f32(freq), f32(pres))
    ahead = logits.cuda()
    on_device = i32([0, 77, 44, 5, 9, 123])          # in another order than the rows, with a word behind them
    k.apply_penalties(ahead, *lists(outputs), f32(rep), f32(freq), f32(pres), on_device, i32([4, 3, 2, 1, -1]))
    assert torch.equal(ahead, whole)
    assert not torch.equal(ahead.cpu()[:3], logits[:3])
    assert torch.equal(ahead.cpu()[3], logits[3])


@pytest.mark.parametrize("vocab", [503, 4096, 151936])
def test_logprobs_follow_log_softmax_top_k_and_rank(vocab):
    """minivllm/sample/sampler.py:313-349: log_softmax of the row at the sampled token, how many
    logits are at least as large, and the largest tokens in order; rows that ask for lists of
    different lengths or for none; ties; a token masked to -inf."""
    import vllm_from_scratch_b200.kernels as k
    g = torch.Generator().manual_seed(vocab)
    rows = 6
    logits = torch.randn(rows, vocab, generator=g) * 4
    logits[1, 7] = logits[1, 300] = logits[1].max() + 1.0          # a tie at the top
    logits[2, 5] = float("-inf")
    tokens = torch.tensor([3, 300, 5, 11, vocab - 1, 0], dtype=torch.int32)
    wanted = torch.tensor([5, 2, 0, -1, 32, 1], dtype=torch.int32)
    width = 33
    ids = torch.full((rows, width), -7, dtype=torch.int32, device="cuda")
    values = torch.full((rows, width), 7.0, device="cuda")
    place = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    k.logprobs(logits.cuda(), tokens.cuda(), wanted.cuda(), ids, values, place)
    ids, values, place = ids.cpu(), values.cpu(), place.cpu()
    expected = torch.log_softmax(logits.double(), dim=-1)
    for r in range(rows):
        n = int(wanted[r])
        if n < 0:
            assert (ids[r] == -7).all() and place[r] == -7
            continue
        t = int(tokens[r])
        assert ids[r, 0] == t and place[r] == int((logits[r] >= logits[r, t]).sum())
        if logits[r, t] == float("-inf"):
            assert values[r, 0] == float("-inf")
        else:
            assert abs(float(values[r, 0]) - float(expected[r, t])) < 1e-4
        order = sorted(range(vocab), key=lambda i: (-float(logits[r, i]), i))[:n]
        assert ids[r, 1:1 + n].tolist() == order
        assert torch.allclose(values[r, 1:1 + n].double(), expected[r, order], atol=1e-4)
        assert (ids[r, 1 + n:] == -7).all()
    with pytest.raises(k.KernelError):
        k.logprobs(logits.cuda(), tokens.cuda(), wanted.cuda(), torch.zeros((rows, 40), dtype=torch.int32, device="cuda"),
                   torch.zeros((rows, 40), device="cuda"), place.cuda())


def test_min_tokens_masks_stop_ids_even_for_greedy_rows():
    import vllm_from_scratch_b200 as engine
    sampler = engine.Sampler(64, "cuda")
    logits = torch.zeros(2, 64, device="cuda")
    logits[:, 10] = 5.0
    logits[:, 11] = 4.0
    params = [engine.SamplingParams(temperature=0.0, min_tokens=3, max_tokens=8, eos_token_id=10),
              engine.SamplingParams(temperature=0.0, min_tokens=0, max_tokens=8, eos_token_id=10)]
    tokens = sampler.sample(logits, params, [1, 2], [[1], [1]], [[], []])
    assert tokens == [11, 10]
