"""The engine's host-side logic on a machine without a GPU: the kernels are
replaced by their plain stand-ins (tests/plain_ops.py), everything else is the
engine's own code: packing, cache, scheduler, engine loop."""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_ops
import tiny_configs
import vllm_from_scratch_b200 as engine


@pytest.fixture(autouse=True)
def plain_kernels(monkeypatch):
    plain_ops.patch(monkeypatch)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("cpu_models")
    return {"A": helpers.make_model_folder(base, tiny_configs.TINY_A, seed=31),
            "B": helpers.make_model_folder(base, tiny_configs.TINY_B, seed=32),
            "C": helpers.make_model_folder(base, tiny_configs.TINY_C, seed=33)}


@pytest.mark.parametrize("name,page", [("A", 16), ("B", 8), ("C", 16)])
def test_every_cut_gives_the_plain_logits(folders, name, page):
    raw = getattr(tiny_configs, f"TINY_{name}")
    lengths = {"a": 45, "b": 70, "c": 33, "d": 3, "e": 90}
    sequences = {rid: helpers.random_tokens(raw["vocab_size"], n, seed=n) for rid, n in lengths.items()}
    expected = {rid: helpers.plain_logits(folders[name], toks) for rid, toks in sequences.items()}
    cuts = {
        "whole": helpers.cut_whole(lengths), "tail": helpers.cut_tail_one_by_one(lengths, 32),
        "portions": helpers.cut_changing_portions(lengths), "mixed": helpers.cut_mixed(lengths, seed=2),
    }
    for label, steps in cuts.items():
        pages = sum(sorted((-(-n // page) for n in lengths.values()), reverse=True)[:4])
        runner = engine.ModelRunner.from_folder(folders[name], "float32", page, pages, 4, device="cpu")
        results = helpers.run_schedule(runner, sequences, steps)
        for rid in sequences:
            diff = float((results[rid] - expected[rid]).abs().max())
            assert diff < 2e-5, (name, label, rid, diff)


def greedy(folder, prompts, **options):
    llm = engine.LLM(folder, dtype="float32", device="cpu", enforce_eager=True, **options)
    outs = llm.generate(prompts, engine.SamplingParams(temperature=0.0, max_tokens=10))
    llm.engine.runner.manager.check_invariants()
    assert llm.engine.runner.manager.stats()["requests"] == 0
    return [o.token_ids for o in outs], llm


def test_generation_is_the_same_under_every_engine_setting(folders):
    raw = tiny_configs.TINY_B
    prompts = [helpers.random_tokens(raw["vocab_size"], n, seed=7 * n) for n in (1, 7, 40, 64, 3, 100)]
    prompts.append(prompts[3][:48] + [5, 6, 7])             # shares three pages with prompts[3]
    base, _ = greedy(folders["B"], prompts, max_model_len=128, block_size=8, max_num_seqs=4,
                     max_num_batched_tokens=32)
    for prompt, tokens in zip(prompts[:3], base[:3]):
        sequence = list(prompt)
        for token in tokens:
            logits = helpers.plain_logits(folders["B"], sequence)[-1]
            assert token == int(logits.argmax())
            sequence.append(token)
    shared, llm = greedy(folders["B"], prompts, max_model_len=128, block_size=8, max_num_seqs=4,
                         max_num_batched_tokens=32, enable_prefix_caching=True)
    assert shared == base
    assert llm.engine.runner.manager.pools[0].num_published > 0
    small, llm = greedy(folders["B"], prompts, max_model_len=128, block_size=8, max_num_seqs=4,
                        max_num_batched_tokens=64, num_gpu_blocks=20)
    assert small == base and llm.engine.scheduler.num_preemptions > 0
    one_by_one, _ = greedy(folders["B"], prompts, max_model_len=128, block_size=8, max_num_seqs=1,
                           max_num_batched_tokens=7)
    assert one_by_one == base


def test_first_step_inputs_are_recorded(folders):
    llm = engine.LLM(folders["A"], dtype="float32", device="cpu", enforce_eager=True, max_model_len=64,
                     block_size=16, max_num_seqs=2, max_num_batched_tokens=8)
    llm.generate([[1, 2, 3, 4, 5], [9, 8, 7, 6, 5, 4]], engine.SamplingParams(temperature=0.0, max_tokens=2))
    first = llm.engine.first_step_inputs
    assert first["num_scheduled_tokens"] == {"gen-0": 5, "gen-1": 3}
    assert first["positions"] == [0, 1, 2, 3, 4, 0, 1, 2]
    assert first["query_start"] == [0, 5, 8] and first["seq_lens"] == [5, 3]
    table = first["block_table"][0]
    assert first["slot_mapping"][0] == [table[0][0] * 16 + i for i in range(5)] + [table[1][0] * 16 + i for i in range(3)]


def test_stop_token_and_min_tokens(folders):
    raw = tiny_configs.TINY_A
    prompt = helpers.random_tokens(raw["vocab_size"], 9, seed=3)
    llm = engine.LLM(folders["A"], dtype="float32", device="cpu", enforce_eager=True, max_model_len=64)
    free = llm.generate([prompt], engine.SamplingParams(temperature=0.0, max_tokens=6))[0].token_ids
    stopper = free[2]
    stopped = llm.generate([prompt], engine.SamplingParams(temperature=0.0, max_tokens=6,
                                                           stop_token_ids=[stopper]))[0]
    assert stopped.token_ids == free[:free.index(stopper) + 1] and stopped.finish_reason.name == "STOP"
    assert stopped.stop_reason == stopper
    held = llm.generate([prompt], engine.SamplingParams(temperature=0.0, max_tokens=6, min_tokens=6,
                                                        stop_token_ids=[stopper]))[0]
    assert stopper not in held.token_ids[:5] and len(held.token_ids) == 6
    # outputs carry text where the engine has a tokenizer
    class Spelled:
        def decode(self, ids, skip_special_tokens=True):
            return " ".join(f"<{i}>" for i in ids)
    worded = engine.LLM(folders["A"], dtype="float32", device="cpu", enforce_eager=True, max_model_len=64,
                        tokenizer=Spelled())
    out = worded.generate([prompt], engine.SamplingParams(temperature=0.0, max_tokens=3))[0]
    assert out.token_ids == free[:3] and out.text == " ".join(f"<{i}>" for i in free[:3]) and held.text is None
    # the counts the entry point reports, and an abort between steps
    core = llm.engine
    core.add_request("x", prompt, engine.SamplingParams(temperature=0.0, max_tokens=5))
    core.add_request("y", prompt, engine.SamplingParams(temperature=0.0, max_tokens=5))
    assert core.get_num_unfinished_requests() == 2 and core.has_unfinished_requests()
    core.step()
    core.abort_request(["x"])
    assert core.get_num_unfinished_requests() == 1
    while core.has_unfinished_requests():
        core.step()
    assert core.get_num_unfinished_requests() == 0 and core.runner.manager.stats()["requests"] == 0


def test_a_kernel_error_flag_stops_the_engine(folders, monkeypatch):
    """A kernel that gave up a bounded wait leaves a flag; the engine reads the flags when
    its requests are done (and now and then) and refuses to hand such results on."""
    import vllm_from_scratch_b200.kernels as kernels
    llm = engine.LLM(folders["A"], dtype="float32", device="cpu", enforce_eager=True, max_model_len=64)
    runner = llm.engine.runner
    runner.check_device()                                   # nothing wrong
    monkeypatch.setattr(kernels, "device_error", lambda: "attention kernel gave up waiting (code 25)")
    with pytest.raises(RuntimeError, match="gave up waiting"):
        runner.check_device()
    with pytest.raises(RuntimeError, match="results since the last check are void"):
        llm.generate([[1, 2, 3]], engine.SamplingParams(temperature=0.0, max_tokens=2))
    with pytest.raises(engine.EngineDeadError):
        llm.engine.step()


def test_error_words_come_with_every_sampling_step(folders, monkeypatch):
    """The kernels' error words travel with the sampled ids of every step: a step in which a
    kernel gave up is refused before its tokens are committed or handed out, not steps later."""
    import vllm_from_scratch_b200.kernels as kernels
    llm = engine.LLM(folders["A"], dtype="float32", device="cpu", enforce_eager=True, max_model_len=64)
    core = llm.engine
    core._carry_status = True
    words = [0, 0, 0]
    monkeypatch.setattr(kernels, "collect_status",
                        lambda flag, out: out.copy_(torch.tensor(words, dtype=torch.int32)))
    core.add_request("r", [1, 2, 3], engine.SamplingParams(temperature=0.0, max_tokens=8))
    first = core.step()
    assert len(first) == 1 and len(first[0].token_ids) == 1
    words[1] = 25                                            # from now on: an attention kernel gave up
    with pytest.raises(RuntimeError, match=r"the step is void: attention kernel gave up waiting \(code 25\)"):
        core.step()
    assert len(core.scheduler.requests["r"].output_token_ids) == 1, "nothing of the void step was committed"
    with pytest.raises(engine.EngineDeadError):
        core.step()
    assert kernels.status_problem([4, 0, 41], 256) == (
        "token id outside the vocabulary [0, 256) at batch row 3; matrix-product kernel gave up waiting (code 41)")
    assert kernels.status_problem([0, 0, 0]) is None


def test_max_model_len_beyond_the_trained_positions_is_refused(folders):
    """minivllm/worker/worker.py:140: max_position_embeddings < max_model_len is an error."""
    with pytest.raises(ValueError, match="max_position_embeddings=128"):
        engine.LLM(folders["A"], dtype="float32", device="cpu", enforce_eager=True, max_model_len=129)
    engine.LLM(folders["A"], dtype="float32", device="cpu", enforce_eager=True, max_model_len=128)


def test_packing_with_empty_requests_and_repeated_wanted_rows(folders):
    """Shapes fixed in advance: requests without tokens after the real ones, wanted rows
    filled up with row 0; nothing about the real requests changes.  The request that brings
    one token is put ahead of the one that brings a portion; the wanted rows follow it."""
    runner = engine.ModelRunner.from_folder(folders["A"], "float32", 16, 8, 4, device="cpu")
    for rid, n in (("a", 5), ("b", 1)):
        runner.manager.admit(rid)
        assert runner.manager.allocate(rid, 20 + n)
    entries = [engine.StepEntry("a", [1, 2, 3, 4, 5], 20, [4]), engine.StepEntry("b", [9], 20, [])]
    step = runner.step_function
    plain, plain_meta = step.pack_host(entries, table_width=4)
    host, meta = step.pack_host(entries, pad_requests=4, table_width=4, pad_tokens=0, pad_wanted=4)
    assert meta["num_tokens"] == plain_meta["num_tokens"] == 6 and meta["num_requests"] == 4
    assert meta["query_start"] == [0, 1, 6, 6, 6] and meta["seq_lens"] == [21, 25, 0, 0]
    assert meta["num_wanted"] == 4 and meta["max_query_len"] == 5
    assert meta["num_decode"] == plain_meta["num_decode"] == 1
    ctx, ids, want = step.context_from(host, meta)
    plain_ctx, plain_ids, plain_want = step.context_from(plain, plain_meta)
    assert ids.tolist() == plain_ids.tolist() == [9, 1, 2, 3, 4, 5]
    assert want.tolist() == [5, 0, 0, 0] and plain_want.tolist() == [5]
    assert ctx.num_decode == 1
    assert ctx.groups[0].block_table[:2].tolist() == plain_ctx.groups[0].block_table.tolist()
    assert ctx.groups[0].block_table[2:].eq(-1).all()
    assert ctx.groups[0].slot_mapping.tolist() == plain_ctx.groups[0].slot_mapping.tolist()
    # the old form: padding requests of one token each
    host, meta = step.pack_host([entries[1]], pad_requests=2, table_width=4)
    assert meta["num_tokens"] == 2 and meta["query_start"] == [0, 1, 2] and meta["seq_lens"] == [21, 0]
    assert meta["num_decode"] == 0                      # one kind only
