"""Generation through the entry point, the scheduler under pressure, the sampler's
kernels, long decoding and the first tokens of a sequence."""

from __future__ import annotations

import pytest
import torch

import helpers
import tiny_configs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("engine_models")
    return {"A": helpers.make_model_folder(base, tiny_configs.TINY_A, seed=11),
            "B": helpers.make_model_folder(base, tiny_configs.TINY_B, seed=12),
            "C": helpers.make_model_folder(base, tiny_configs.TINY_C, seed=13),
            "D": helpers.make_model_folder(base, tiny_configs.TINY_D, seed=14),
            "E": helpers.make_model_folder(base, tiny_configs.TINY_E, seed=15)}


def plain_greedy(folder, prompt, new_tokens):
    """Greedy continuation by the plain implementation: the whole sequence is run
    again for every token.  Also returns the margin between the best and the
    second-best logit at each step (a near-tie may legitimately flip)."""
    tokens = list(prompt)
    margins = []
    for _ in range(new_tokens):
        logits = helpers.plain_logits(folder, tokens)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        tokens.append(int(logits.argmax()))
    return tokens[len(prompt):], margins


def assert_same_until_near_tie(got, expected, margins, what, tie=1e-4):
    for index, (a, b) in enumerate(zip(got, expected)):
        if a != b:
            assert margins[index] < tie, f"{what}: token {index} is {a}, expected {b} (margin {margins[index]:.2e})"
            return
    assert len(got) == len(expected), what


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("name,lengths,page", [("A", [5, 17, 33, 1], 16), ("B", [1, 7, 40, 64, 3, 100], 8)])
def test_greedy_generation_matches_plain(folders, name, lengths, page, eager):
    import vllm_from_scratch_b200 as engine
    raw = tiny_configs.TINY_A if name == "A" else tiny_configs.TINY_B
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=50 + i) for i, n in enumerate(lengths)]
    llm = engine.LLM(folders[name], dtype="float32", max_model_len=128, block_size=page,
                     max_num_seqs=4, max_num_batched_tokens=32, enforce_eager=eager)
    outputs = llm.generate(prompts, engine.SamplingParams(temperature=0.0, max_tokens=8))
    for prompt, output in zip(prompts, outputs):
        expected, margins = plain_greedy(folders[name], prompt, 8)
        assert output.finished and output.finish_reason.name == "LENGTH"
        assert_same_until_near_tie(output.token_ids, expected, margins, f"{name} prompt of {len(prompt)}")
    if not eager:
        assert llm.engine.decode_graphs.replays > 0, "decode steps must go through the captured graphs"
    llm.engine.runner.manager.check_invariants()
    assert llm.engine.runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("eager", [True, False])
@pytest.mark.parametrize("name,page", [("D", 16), ("E", 16), ("E", 48)])
def test_bfloat16_greedy_generation_matches_plain(folders, name, page, eager):
    """bfloat16 through the entry point at head sizes 64 and 128 (the tensor-core attention
    kernels, the few-rows products, for 128 the decode kernel that also rotates and stores and
    the tcgen05 kernel for the prompts), with and without graphs, against the plain model with
    weights rounded to bfloat16.  A token may differ only where the plain model's two best
    logits lie closer than the rounding of bfloat16 activations can move them."""
    import vllm_from_scratch_b200 as engine
    raw = getattr(tiny_configs, f"TINY_{name}")
    lengths = [5, 70, 33, 1, 150, 64]
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=150 + i) for i, n in enumerate(lengths)]
    llm = engine.LLM(folders[name], dtype="bfloat16", max_model_len=256, block_size=page,
                     max_num_seqs=4, max_num_batched_tokens=96, enforce_eager=eager)
    outputs = llm.generate(prompts, engine.SamplingParams(temperature=0.0, max_tokens=12))
    same = 0
    for prompt, output in zip(prompts, outputs):
        tokens, flipped = list(prompt), False
        for place, got in enumerate(output.token_ids):
            logits = helpers.plain_logits(folders[name], tokens, round_weights_to=torch.bfloat16)[-1]
            top = torch.topk(logits, 2)
            if got != int(top.indices[0]):
                margin = float(top.values[0] - top.values[1])
                assert margin < 2 * tiny_configs.BF16_REL[name] * float(logits.abs().max()), (
                    f"{name} prompt of {len(prompt)}: token {place} is {got}, plain says {int(top.indices[0])} "
                    f"(margin {margin:.3e})")
                flipped = True
                break
            tokens.append(got)
        same += not flipped
    assert same >= len(prompts) - 2, "most requests must generate the plain model's tokens throughout"
    if not eager:
        assert llm.engine.decode_graphs.replays > 0
    llm.engine.runner.manager.check_invariants()
    assert llm.engine.runner.manager.stats()["requests"] == 0


def test_demo_command_line_prints_the_tokens_of_the_entry_point(tmp_path, capsys):
    """The command line (``demo.main``) with ``--random-weights`` in both precisions: the tokens
    it prints are those ``LLM.generate`` gives for the same model folder, prompts and options."""
    import json
    import re
    import vllm_from_scratch_b200 as engine
    from vllm_from_scratch_b200 import demo
    config_file = tmp_path / "tiny_b.json"
    config_file.write_text(json.dumps(tiny_configs.TINY_B))
    questions = ["1 2 3 4 5 6 7 8 9", "11, 12, 13", " ".join(str(7 * i % 503) for i in range(40))]
    for dtype in ("float32", "bfloat16"):
        code = demo.main([*questions, "--random-weights", str(config_file), "--random-seed", "4", "--dtype", dtype,
                          "--max-model-len", "128", "--max-new-tokens", "9", "--block-size", "8",
                          "--num-kv-blocks", "48", "--max-num-seqs", "2", "--max-num-batched-tokens", "32",
                          "--trace", "--scheduler-trace", "--logprobs", "2"])
        assert code == 0
        printed = capsys.readouterr().out
        assert printed.count("cumulative logprob") == 3 and "(rank 1)" in printed
        answers = {int(m.group(1)): json.loads(m.group(2)) for m in re.finditer(r"answer\[q(\d+)\]: (\[.*\])", printed)}
        assert sorted(answers) == [0, 1, 2] and all(len(a) == 9 for a in answers.values())
        assert "finish reason LENGTH" in printed and "first step (num_scheduled_tokens=" in printed
        assert "Qwen3ForCausalLM" in printed and "prefix caching: on" in printed
        folder = engine.write_random_model(tiny_configs.TINY_B, 4, tmp_path / f"model_{dtype}",
                                           dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32)
        llm = engine.LLM(folder, dtype=dtype, max_model_len=128, block_size=8, num_gpu_blocks=48, max_num_seqs=2,
                         max_num_batched_tokens=32, enable_prefix_caching=True)
        prompts = [demo.parse_prompt(q) for q in questions]
        expected = llm.generate(prompts, engine.SamplingParams(temperature=0.0, max_tokens=9))
        assert [answers[i] for i in range(3)] == [out.token_ids for out in expected], dtype
    with pytest.raises(SystemExit, match="not a list of token ids"):
        demo.parse_prompt("hello there")


def test_small_pool_preempts_and_gives_the_same_tokens(folders):
    """A pool too small for all requests at once: some are preempted and computed
    again; every request still ends with the tokens it gets from a large pool."""
    import vllm_from_scratch_b200 as engine
    raw = tiny_configs.TINY_B
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=70 + i) for i, n in enumerate([30, 41, 18, 25])]
    params = engine.SamplingParams(temperature=0.0, max_tokens=20)
    results = {}
    for label, blocks in (("large", 64), ("small", 14)):
        llm = engine.LLM(folders["B"], dtype="float32", max_model_len=128, block_size=8,
                         num_gpu_blocks=blocks, max_num_seqs=4, max_num_batched_tokens=64,
                         enforce_eager=True)
        results[label] = llm.generate(prompts, params)
        if label == "small":
            assert llm.engine.scheduler.num_preemptions > 0, "the small pool was meant to run out"
        llm.engine.runner.manager.check_invariants()
    for big, small in zip(results["large"], results["small"]):
        assert big.token_ids == small.token_ids


def test_temperature_sampling_is_reproducible_and_batch_independent(folders):
    import vllm_from_scratch_b200 as engine
    raw = tiny_configs.TINY_B
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=90 + i) for i, n in enumerate([1, 7, 40, 64, 3, 100])]
    def run(order, budget):
        llm = engine.LLM(folders["B"], dtype="float32", max_model_len=256, block_size=8,
                         max_num_seqs=4, max_num_batched_tokens=budget, enforce_eager=True)
        params = [engine.SamplingParams(temperature=0.8, max_tokens=12, seed=1000 + i) for i in order]
        outs = llm.generate([prompts[i] for i in order], params)
        return {i: out.token_ids for i, out in zip(order, outs)}
    first = run(list(range(6)), 32)
    again = run(list(range(6)), 32)
    other = run([5, 3, 1, 0, 2, 4], 200)
    assert first == again, "same seeds, same tokens"
    # float32 logits differ only by rounding between batchings; a seeded draw keyed by
    # position gives the same token unless two candidates are within that rounding.
    same = sum(first[i] == other[i] for i in range(6))
    assert same >= 5, (first, other)
    assert any(len(set(tokens)) > 1 for tokens in first.values())


def test_windowed_model_generates_and_returns_pages(folders):
    import vllm_from_scratch_b200 as engine
    raw = tiny_configs.TINY_C
    prompt = helpers.random_tokens(raw["vocab_size"], 90, seed=5)
    llm = engine.LLM(folders["C"], dtype="float32", max_model_len=256, block_size=16,
                     max_num_seqs=2, max_num_batched_tokens=64, enforce_eager=True)
    llm.engine.add_request("w", prompt, engine.SamplingParams(temperature=0.0, max_tokens=40))
    least_free = None
    tokens = []
    while llm.engine.has_unfinished_requests():
        for out in llm.engine.step():
            tokens = out.token_ids
        stats = llm.engine.runner.manager.stats()
        if stats["requests"]:
            # group 1 is the windowed one (window 24, pages of 16)
            least_free = stats["group1_free_pages"] if least_free is None else min(least_free, stats["group1_free_pages"])
    expected, margins = plain_greedy(folders["C"], prompt, 40)
    assert_same_until_near_tie(tokens, expected, margins, "windowed generation")
    total = llm.engine.runner.manager.pools[1].num_pages
    # a 64-token portion holds 4 pages plus the window's 2 before them; never the 9 of all 130 positions
    assert total - least_free <= 6, "the windowed group must give pages back while the request runs"


def test_long_decoding_and_first_tokens(folders):
    """One request decoded token by token from its second token on, far past
    several page edges, in both precisions."""
    from vllm_from_scratch_b200 import ModelRunner
    raw = tiny_configs.TINY_B
    tokens = helpers.random_tokens(raw["vocab_size"], 230, seed=77)
    for dtype, rounding in (("float32", None), ("bfloat16", torch.bfloat16)):
        reference = helpers.plain_logits(folders["B"], tokens, round_weights_to=rounding)
        runner = ModelRunner.from_folder(folders["B"], dtype, 8, 32, 2, device="cuda")
        steps = [[("r", 1)] for _ in range(len(tokens))]
        result = helpers.run_schedule(runner, {"r": tokens}, steps)["r"]
        diff = (result - reference).abs().max(dim=1).values
        bound = tiny_configs.F32_ATOL if dtype == "float32" else tiny_configs.BF16_REL["B"] * float(reference.abs().max())
        assert float(diff.max()) <= bound, (dtype, int(diff.argmax()), float(diff.max()))
        assert float(diff[:4].max()) <= bound


def test_failed_step_latches(folders):
    import vllm_from_scratch_b200 as engine
    llm = engine.LLM(folders["A"], dtype="float32", max_model_len=64, block_size=16, max_num_seqs=2,
                     enforce_eager=True)
    llm.engine.add_request("x", [1, 2, 3], engine.SamplingParams(max_tokens=2, temperature=0.0))

    def broken(entries):
        raise RuntimeError("host-side failure injected by the test")

    original = llm.engine.runner.step
    llm.engine.runner.step = broken
    with pytest.raises(RuntimeError, match="injected"):
        llm.engine.step()
    llm.engine.runner.step = original
    with pytest.raises(engine.EngineDeadError):
        llm.engine.step()


def _generate_with_arrivals(llm, prompts, params, arrivals):
    """Requests join at the given step numbers; returns the final output of each."""
    engine_ = llm.engine
    latest, step, added = {}, 0, 0
    while added < len(prompts) or engine_.has_unfinished_requests():
        while added < len(prompts) and arrivals[added] <= step:
            engine_.add_request(f"r{added}", prompts[added], params[added])
            added += 1
        for output in engine_.step():
            latest[output.request_id] = output
        step += 1
        assert step < 2000
    return [latest[f"r{i}"] for i in range(len(prompts))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_queued_ahead_give_the_same_tokens(folders, dtype):
    """With ``async_scheduling`` the engine queues a decode step before the one before it
    has reported its tokens.  Every request must end with the same tokens, finish for the
    same reason and at the same length as without it: greedy and seeded rows, a stop id
    that ends a request while its next step is already queued, ``max_tokens``,
    ``min_tokens``, requests with penalties (whose token in flight the sampler counts on the
    device), and requests that join while others decode."""
    import vllm_from_scratch_b200 as engine
    raw = tiny_configs.TINY_B
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=300 + i) for i, n in enumerate([9, 33, 17, 5, 21])]
    arrivals = [0, 0, 0, 12, 30]
    results = {}
    for mode in (False, True):
        llm = engine.LLM(folders["B"], dtype=dtype, max_model_len=160, block_size=8, max_num_seqs=4,
                         max_num_batched_tokens=48, async_scheduling=mode)
        if not mode:
            # a stop id that a greedy request really produces, so that it ends "early"
            probe = llm.generate([prompts[1]], engine.SamplingParams(temperature=0.0, max_tokens=24))[0]
            stop_id = probe.token_ids[10]
        params = [
            engine.SamplingParams(temperature=0.0, max_tokens=40),
            engine.SamplingParams(temperature=0.0, max_tokens=64, stop_token_ids=[stop_id]),
            engine.SamplingParams(temperature=0.9, top_k=12, top_p=0.9, seed=5, max_tokens=33, min_tokens=4,
                                  stop_token_ids=[stop_id]),
            engine.SamplingParams(temperature=0.0, max_tokens=25, repetition_penalty=1.3, presence_penalty=0.2),
            engine.SamplingParams(temperature=0.7, seed=11, max_tokens=50, frequency_penalty=0.4, repetition_penalty=0.9),
        ]
        results[mode] = _generate_with_arrivals(llm, prompts, params, arrivals)
        llm.engine.runner.manager.check_invariants()
        assert llm.engine.runner.manager.stats()["requests"] == 0
        if mode:
            assert llm.engine.num_steps_ahead > 20, "most decode steps should have been queued ahead"
        else:
            assert llm.engine.num_steps_ahead == 0
    for index, (sync, ahead) in enumerate(zip(results[False], results[True])):
        assert ahead.token_ids == sync.token_ids, f"request {index}"
        assert ahead.finish_reason == sync.finish_reason and ahead.stop_reason == sync.stop_reason
    assert results[True][1].finish_reason.name == "STOP" and len(results[True][1].token_ids) <= 11


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_requests_with_random_options_the_same_with_and_without_steps_queued_ahead(folders, dtype):
    """Twenty requests with options drawn at random (greedy or seeded, filters, penalties, stop
    ids, ``min_tokens``, log-probabilities) that join at random steps: queueing steps ahead changes
    nothing of what any of them gets."""
    import random
    import vllm_from_scratch_b200 as engine
    raw = tiny_configs.TINY_B
    rng = random.Random(11)
    prompts, params, arrivals = [], [], []
    for index in range(20):
        prompts.append(helpers.random_tokens(raw["vocab_size"], rng.randint(1, 60), seed=900 + index))
        options = {"max_tokens": rng.randint(1, 40), "temperature": rng.choice([0.0, 0.0, 0.7, 1.0, 1.3])}
        if options["temperature"] > 0:
            options["seed"] = rng.randrange(1000)
            options.update(rng.choice([{}, {"top_k": rng.randint(1, 50)}, {"top_p": rng.uniform(0.3, 0.99)},
                                       {"min_p": rng.uniform(0.01, 0.2)}, {"top_k": 30, "top_p": 0.8, "min_p": 0.02}]))
        options.update(rng.choice([{}, {}, {"repetition_penalty": rng.uniform(0.8, 1.5)},
                                   {"frequency_penalty": rng.uniform(0.1, 1.0), "presence_penalty": rng.uniform(0.0, 0.5)}]))
        options.update(rng.choice([{}, {}, {"logprobs": rng.randint(0, 4)}]))
        options.update(rng.choice([{}, {}, {"stop_token_ids": [rng.randrange(raw["vocab_size"]) for _ in range(40)]}]))
        if rng.random() < 0.3:
            options["min_tokens"] = rng.randint(0, options["max_tokens"])
        params.append(engine.SamplingParams(**options))
        arrivals.append(rng.randint(0, 45))
    arrivals.sort()
    results = {}
    for mode in (False, True):
        llm = engine.LLM(folders["B"], dtype=dtype, max_model_len=128, block_size=8, max_num_seqs=6,
                         max_num_batched_tokens=40, async_scheduling=mode)
        results[mode] = _generate_with_arrivals(llm, prompts, params, arrivals)
        llm.engine.runner.manager.check_invariants()
        assert llm.engine.runner.manager.stats()["requests"] == 0 and not llm.engine.sampler._seen
    assert llm.engine.num_steps_ahead > 20
    for index, (sync, ahead) in enumerate(zip(results[False], results[True])):
        assert ahead.token_ids == sync.token_ids, f"request {index}: {params[index]}"
        assert ahead.finish_reason == sync.finish_reason and ahead.stop_reason == sync.stop_reason
        if dtype == "float32":
            assert ahead.logprobs == sync.logprobs and ahead.cumulative_logprob == sync.cumulative_logprob
        elif sync.logprobs is not None:
            # a request that stops while its next step is queued keeps its row for that step: the
            # others' logits are then those of a batch of another size, equal up to bfloat16 rounding
            for token, one, other in zip(ahead.token_ids, ahead.logprobs, sync.logprobs):
                assert abs(one[token].logprob - other[token].logprob) < 0.05


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logprobs_of_generated_tokens_match_plain(folders, dtype):
    """``SamplingParams.logprobs``: every generated token comes with its log-probability under the
    model's own logits (before temperature and penalties, minivllm/sample/sampler.py:86-95), its
    place, and the most likely tokens; the plain model gives the same numbers, with and without
    steps queued ahead, and a request without the option gets none."""
    import vllm_from_scratch_b200 as engine
    name = "B" if dtype == "float32" else "E"
    raw = getattr(tiny_configs, f"TINY_{name}")
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=700 + i) for i, n in enumerate([12, 40, 7])]
    params = [engine.SamplingParams(temperature=0.0, max_tokens=10, logprobs=3),
              engine.SamplingParams(temperature=0.8, top_k=20, seed=3, max_tokens=14, logprobs=0, repetition_penalty=1.2, min_tokens=2),
              engine.SamplingParams(temperature=0.0, max_tokens=9)]
    results = {}
    for mode in (False, True):
        llm = engine.LLM(folders[name], dtype=dtype, max_model_len=128, block_size=16, max_num_seqs=4,
                         max_num_batched_tokens=64, async_scheduling=mode)
        results[mode] = llm.generate(prompts, params)
    bound = 1e-4 if dtype == "float32" else 2 * tiny_configs.BF16_REL[name]
    for index, (prompt, out) in enumerate(zip(prompts, results[True])):
        other = results[False][index]
        assert out.token_ids == other.token_ids
        if params[index].logprobs is None:
            assert out.logprobs is None and out.cumulative_logprob is None
            continue
        assert len(out.logprobs) == len(out.token_ids)
        assert [{t: (round(v.logprob, 5), v.rank) for t, v in entry.items()} for entry in out.logprobs] == \
               [{t: (round(v.logprob, 5), v.rank) for t, v in entry.items()} for entry in other.logprobs]
        weights = torch.bfloat16 if dtype == "bfloat16" else None
        logits = helpers.plain_logits(folders[name], list(prompt) + out.token_ids[:-1], round_weights_to=weights)
        total = 0.0
        for place, (token, entry) in enumerate(zip(out.token_ids, out.logprobs)):
            row = logits[len(prompt) - 1 + place]
            expected = torch.log_softmax(row.double(), dim=-1)
            scale = 1.0 if dtype == "float32" else float(row.abs().max())
            assert abs(entry[token].logprob - float(expected[token])) < bound * scale, (index, place)
            total += entry[token].logprob
            wanted = params[index].logprobs
            assert len(entry) in (wanted, wanted + 1)
            if dtype == "float32":
                assert entry[token].rank == int((row >= row[token]).sum())
                best = torch.topk(row, wanted).indices.tolist() if wanted else []
                listed = [t for t, v in sorted(entry.items(), key=lambda kv: kv[1].rank) if v.rank <= wanted]
                assert listed == best, (index, place)
        assert abs(out.cumulative_logprob - total) < 1e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_repeated_mixed_steps_replay_graphs_with_the_same_tokens(folders, dtype):
    """Prompts cut under a small token budget give steps of the same shape again and again
    (a portion that fills the budget beside the decoding requests); from the second time on
    such a step is a graph replay.  Tokens must equal those of the engine without graphs."""
    import vllm_from_scratch_b200 as engine
    raw = tiny_configs.TINY_B
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=400 + i) for i, n in enumerate([150, 97, 140, 33, 120])]
    params = engine.SamplingParams(temperature=0.0, max_tokens=12)
    results = {}
    for eager in (True, False):
        llm = engine.LLM(folders["B"], dtype=dtype, max_model_len=192, block_size=8, max_num_seqs=3,
                         max_num_batched_tokens=24, enforce_eager=eager)
        results[eager] = [o.token_ids for o in llm.generate(prompts, params)]
        llm.engine.runner.manager.check_invariants()
        if not eager:
            assert llm.engine.mixed_graphs.replays >= 8, "steps of a repeated shape must be replayed"
            assert llm.engine.decode_graphs.replays > 0
    assert results[False] == results[True]


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_every_engine_setting_gives_the_same_tokens(folders, name):
    """Ten requests of mixed lengths (some sharing a prefix), greedy and seeded, joining at
    random steps: without graphs, with graphs, with steps queued ahead, with prefix caching,
    and with a pool so small that requests are preempted.  In float32 every setting must
    give every request the very same tokens."""
    import random
    import vllm_from_scratch_b200 as engine
    raw = getattr(tiny_configs, f"TINY_{name}")

    def run(eager, ahead, prefix, blocks, seed):
        rng = random.Random(seed)
        shared = helpers.random_tokens(raw["vocab_size"], 40, seed=seed)
        prompts = []
        for i in range(10):
            prompt = helpers.random_tokens(raw["vocab_size"], rng.choice([1, 3, 9, 17, 33, 50, 70]), seed=seed * 100 + i)
            prompts.append(shared[:rng.choice([16, 24, 40])] + prompt if i % 3 == 0 else prompt)
        params = [engine.SamplingParams(temperature=0.0 if i % 2 == 0 else 0.8, seed=i, top_k=0 if i % 4 else 20,
                                        max_tokens=rng.choice([1, 5, 20, 40])) for i in range(10)]
        arrivals = sorted(rng.randrange(0, 30) for _ in prompts)
        llm = engine.LLM(folders[name], dtype="float32", max_model_len=min(160, raw["max_position_embeddings"]),
                         block_size=8, max_num_seqs=4, max_num_batched_tokens=32, enforce_eager=eager, async_scheduling=ahead,
                         enable_prefix_caching=prefix, num_gpu_blocks=blocks)
        core, latest, step, added = llm.engine, {}, 0, 0
        while added < len(prompts) or core.has_unfinished_requests():
            while added < len(prompts) and arrivals[added] <= step:
                core.add_request(f"r{added}", prompts[added], params[added])
                added += 1
            for output in core.step():
                latest[output.request_id] = output
            step += 1
            assert step < 5000
        core.runner.manager.check_invariants()
        assert core.runner.manager.stats()["requests"] == 0
        return [latest[f"r{i}"].token_ids for i in range(len(prompts))], core

    for seed in (1, 2):
        expected, _ = run(True, False, False, None, seed)
        settings = [(False, False, False, None), (False, True, False, None), (False, True, False, 30)]
        if name != "C":                                     # a windowed group has no prefix caching
            settings += [(False, True, True, None), (True, False, True, None), (False, False, True, 30)]
        for eager, ahead, prefix, blocks in settings:
            got, core = run(eager, ahead, prefix, blocks, seed)
            assert got == expected, (seed, eager, ahead, prefix, blocks)
            if blocks is not None:
                assert core.scheduler.num_preemptions > 0, "the small pool was meant to force preemption"
            if ahead:
                assert core.num_steps_ahead > 0


@pytest.mark.parametrize("eager", [True, False])
def test_decode_attention_in_one_kernel_gives_the_same_tokens(folders, eager, monkeypatch):
    """bfloat16, head size 128, one layer with a window: decode steps whose attention kernel also
    normalises and rotates the heads and stores the new key and value give the tokens of the steps
    that run the two kernels one after the other (their arithmetic is the same), while pages of
    the windowed layer come back and are used again."""
    import vllm_from_scratch_b200 as engine
    from vllm_from_scratch_b200 import kernels
    from vllm_from_scratch_b200.kernels import attention_bf16
    raw = tiny_configs.TINY_E
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=70 + i) for i, n in enumerate([3, 60, 17, 130, 64])]
    params = engine.SamplingParams(temperature=0.0, max_tokens=70)
    results, launches = {}, {}
    for fused in (True, False):
        monkeypatch.setattr(attention_bf16, "USE_FUSED_DECODE", fused)
        llm = engine.LLM(folders["E"], dtype="bfloat16", max_model_len=256, block_size=16, max_num_seqs=4,
                         max_num_batched_tokens=64, enforce_eager=eager)
        before = kernels.launch_count
        results[fused] = [output.token_ids for output in llm.generate(prompts, params)]
        launches[fused] = kernels.launch_count - before
        llm.engine.runner.manager.check_invariants()
        assert llm.engine.runner.manager.stats()["requests"] == 0
        assert kernels.device_error() is None
    assert results[True] == results[False]
    if eager:
        assert launches[True] < launches[False], "the decode steps must have run the one-kernel form"
