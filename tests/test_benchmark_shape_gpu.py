"""The engine at the benchmark's widths against the plain implementation.

The tiny configurations never reach what the benchmark runs: a width of 2048 with 16
query heads on 8 key/value heads of 128, a feed-forward of 6144, a vocabulary of 151936
(the output product over it, the resident-rows products at K = 6144, the library's
products from 17 rows on, the tcgen05 attention inside a graph planned for a longer
context, decode graphs of 16 and 64 requests).  Here the model has these widths and 2 of
the 28 layers (fewer layers, not smaller ones; the two wider shapes the benchmark also
measures run one layer of their 36 and 64), random weights drawn on the GPU, and
every comparison is with ``plain_qwen3`` run on the GPU in float32 with the reduced-
precision matrix modes off: full against portions against token by token against the
oracle, as the reference's own check does (benchmarks/check_step57_model_logits.py:
300-326).
"""

from __future__ import annotations

import pytest
import torch

import helpers
import plain_qwen3

pytestmark = pytest.mark.gpu

def _shape(layers, hidden, heads, inter, tied):
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": 8, "head_dim": 128,
        "intermediate_size": inter, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
        "tie_word_embeddings": tied, "max_position_embeddings": 40960, "hidden_act": "silu",
        "attention_bias": False, "initializer_range": 0.02,
    }


# name -> (configuration with the layers run here, layers of the full model)
SHAPES = {
    "1.7b": (_shape(2, 2048, 16, 6144, True), 28),
    "8b": (_shape(1, 4096, 32, 12288, False), 36),
    "32b": (_shape(1, 5120, 64, 25600, False), 64),
}
SHAPE = SHAPES["1.7b"][0]
PAGE = 16
LENGTHS = {"a": 600, "b": 330, "c": 131, "d": 70, "e": 520}
# Bounds as fractions of the largest logit of the sequence, twice the worst seen over all shapes and
# cuts.  float32 (sums taken in another order over K of 2048 to 25600): worst 5.4e-6.  bfloat16
# (activations carry 8 bits): worst 1.19e-2.
F32_REL = 1.2e-5
BF16_REL = 0.024


def build_world(name):
    """Weights, sequences and the plain logits in both precisions, all on the GPU."""
    import vllm_from_scratch_b200 as engine
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    shape, layers_full = SHAPES[name]
    entry, config = engine.load_model_config(shape)
    weights = entry.random_weights(config, seed=21, dtype=torch.float32, device="cuda")
    rounded = {k: (v.to(torch.bfloat16).float() if v.dim() > 1 else v) for k, v in weights.items()}
    sequences = {rid: helpers.random_tokens(shape["vocab_size"], n, seed=500 + n) for rid, n in LENGTHS.items()}
    plain = {
        "float32": {rid: plain_qwen3.qwen3_logits(shape, weights, toks) for rid, toks in sequences.items()},
        "bfloat16": {rid: plain_qwen3.qwen3_logits(shape, rounded, toks) for rid, toks in sequences.items()},
    }
    return {"entry": entry, "config": config, "weights": weights, "rounded": rounded, "shape": shape,
            "sequences": sequences, "plain": plain,
            "layers": f"{shape['num_hidden_layers']} of {layers_full} layers"}


@pytest.fixture(scope="module")
def world():
    return build_world("1.7b")


@pytest.fixture(scope="module", params=["8b", "32b"])
def wider_world(request):
    world = build_world(request.param)
    yield request.param, world
    world.clear()
    torch.cuda.empty_cache()


def make_runner(world, dtype, pages, max_requests=4):
    import vllm_from_scratch_b200 as engine
    return engine.ModelRunner(world["entry"].build_spec(world["config"]), world["weights"], dtype, PAGE, pages,
                              max_requests, device="cuda", model_config=world["config"])


def compare(results, expected, dtype, what, layers=""):
    rel = F32_REL if dtype == "float32" else BF16_REL
    worst = 0.0
    for rid, logits in results.items():
        reference = expected[rid]
        assert logits.shape == reference.shape, (what, rid, logits.shape, reference.shape)
        scale = float(reference.abs().max())
        diff = (logits - reference).abs().max(dim=1).values
        if float(diff.max()) > rel * scale:
            position = int(diff.gt(rel * scale).nonzero()[0])
            raise AssertionError(
                f"{what}: request {rid!r} first differs at position {position} "
                f"(max |diff| there {float(diff[position]):.3e}, bound {rel * scale:.3e}, "
                f"largest anywhere {float(diff.max()):.3e})")
        worst = max(worst, float(diff.max()) / scale)
    print(f"{what} ({layers}): max |diff| / max |logit| = {worst:.3e}")


CUTS = {
    "whole": lambda: helpers.cut_whole(LENGTHS),
    "tail": lambda: helpers.cut_tail_one_by_one(LENGTHS, 32),
    "portions": lambda: helpers.cut_changing_portions(LENGTHS, seed=3),
    "mixed": lambda: helpers.cut_mixed(LENGTHS, seed=4, live=4, sizes=helpers.LARGE_PORTIONS),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
def test_every_cut_at_the_benchmark_widths(world, cut, dtype):
    # The mixed cut runs with the four longest requests' pages only, so that pages come back and go out again.
    pages = sum(sorted((-(-n // PAGE) for n in LENGTHS.values()), reverse=True)[:4])
    runner = make_runner(world, dtype, pages)
    results = helpers.run_schedule(runner, world["sequences"], CUTS[cut](), on_device=True)
    compare(results, world["plain"][dtype], dtype, f"1.7B widths/{cut}/{dtype}", world["layers"])
    assert runner.manager.stats()["requests"] == 0
    runner.check_device()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_wider_benchmark_shapes(wider_world, dtype):
    """The widths of the two larger shapes the benchmark measures (32 and 64 query heads on 8
    key/value heads, widths of 4096 and 5120, feed-forwards of 12288 and 25600, an output matrix
    of its own), one layer each: most of each request in one step and the rest token by token,
    then the mixed cut with long portions and pages used again."""
    name, world = wider_world
    pages = sum(sorted((-(-n // PAGE) for n in LENGTHS.values()), reverse=True)[:4])
    for cut in ("tail", "mixed"):
        runner = make_runner(world, dtype, pages)
        results = helpers.run_schedule(runner, world["sequences"], CUTS[cut](), on_device=True)
        compare(results, world["plain"][dtype], dtype, f"{name} widths/{cut}/{dtype}", world["layers"])
        assert runner.manager.stats()["requests"] == 0
        runner.check_device()
        del runner, results
        torch.cuda.empty_cache()


def plain_greedy(world, prompt, new_tokens):
    tokens, margins = list(prompt), []
    for _ in range(new_tokens):
        logits = plain_qwen3.qwen3_logits(SHAPE, world["rounded"], tokens)[-1]
        top = torch.topk(logits, 2).values
        margins.append(float(top[0] - top[1]))
        tokens.append(int(logits.argmax()))
    return tokens[len(prompt):], margins


@pytest.mark.parametrize("max_num_seqs", [16, 64])
def test_decode_graphs_of_many_requests_generate_the_plain_tokens(world, max_num_seqs):
    """bfloat16 through ``LLMEngine`` with graphs on: decode steps of 16 and 64 requests put the
    library's products and the merge of the key splits inside a capture planned for a context
    of 4096.  Greedy tokens must be the plain model's until a near-tie."""
    import vllm_from_scratch_b200 as engine
    max_model_len, new_tokens = 4096, 6
    lengths = [5 + (37 * i) % 90 for i in range(max_num_seqs)]
    prompts = [helpers.random_tokens(SHAPE["vocab_size"], n, seed=900 + i) for i, n in enumerate(lengths)]
    runner = make_runner(world, "bfloat16", max_num_seqs * 8, max_requests=max_num_seqs)
    llm = engine.LLMEngine(engine.EngineConfig(
        engine.ModelConfig("(random weights)", "bfloat16", max_model_len),
        engine.CacheConfig(PAGE, runner.storage.num_pages),
        engine.SchedulerConfig(max_num_seqs, 2048)), runner=runner)
    params = engine.SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
    for index, prompt in enumerate(prompts):
        llm.add_request(f"r{index}", prompt, params)
    latest = {}
    while llm.has_unfinished_requests():
        for output in llm.step():
            latest[output.request_id] = output
    assert llm.decode_graphs.replays >= new_tokens - 2, "decode steps must be graph replays"
    assert max(llm.decode_graphs._graphs) == max_num_seqs, "the widest bucket must have been captured"
    matched = 0
    for index, prompt in enumerate(prompts):
        got = latest[f"r{index}"].token_ids
        expected, margins = plain_greedy(world, prompt, new_tokens)
        scale = float(world["plain"]["bfloat16"]["a"].abs().max())
        for place, (a, b) in enumerate(zip(got, expected)):
            if a != b:
                # both sides may be off by the bfloat16 bound: a flip needs a margin inside twice that
                assert margins[place] < 2 * BF16_REL * scale, (
                    f"request {index}: token {place} is {a}, plain says {b} (margin {margins[place]:.3e})")
                break
        else:
            matched += 1
    print(f"{max_num_seqs} requests: {matched} of {len(prompts)} generate the plain tokens throughout")
    # (random weights give flat logits: a quarter to a third of the requests meet a near-tie within six
    # tokens, and which ones changes with any change of rounding; the bound above is the test, this count
    # only says that the comparison is not empty)
    assert matched >= len(prompts) // 2
    runner.check_device()


def test_prompt_steps_as_graph_replays_at_the_benchmark_widths(world):
    """Prompt steps through ``MixedGraphs``: a shape goes through the ordinary step function the
    first time, is captured the second time (for the longest context, which may choose a key
    split that the eager step did not have) and replayed from then on.  2,048-token prompts
    whole (the benchmark's prefill), then in portions of 512 tokens over a growing context.
    Last-row logits of every step against the plain model."""
    from vllm_from_scratch_b200 import StepEntry
    from vllm_from_scratch_b200.engine.decode_graph import MixedGraphs
    runner = make_runner(world, "bfloat16", 2 * 2048 // PAGE + 4, max_requests=2)
    graphs = MixedGraphs(runner, 4096)
    prompts = [helpers.random_tokens(SHAPE["vocab_size"], 2048, seed=700 + i) for i in range(3)]
    plain_last = {}

    def check(prompt_index, upto, logits, what):
        key = (prompt_index, upto)
        if key not in plain_last:
            plain_last[key] = plain_qwen3.qwen3_logits(SHAPE, world["rounded"], prompts[prompt_index][:upto])[-1]
        reference = plain_last[key]
        diff = float((logits[0] - reference).abs().max())
        bound = BF16_REL * float(reference.abs().max())
        assert diff <= bound, f"{what}: max |diff| {diff:.3e} > {bound:.3e}"
        return diff / float(reference.abs().max())

    worst = 0.0
    for portion in (2048, 512):
        for index, prompt in enumerate(prompts):
            rid = f"p{portion}-{index}"
            runner.manager.admit(rid)
            for start in range(0, len(prompt), portion):
                assert runner.manager.allocate(rid, start + portion)
                logits = graphs.run([StepEntry(rid, prompt[start:start + portion], start, [portion - 1])])
                worst = max(worst, check(index, start + portion, logits.clone(), f"{rid} at {start}"))
                runner.manager.commit(rid, start + portion)
            runner.manager.release(rid)
    assert graphs.replays >= 2 + 8, "the second and third prompt of each kind must be replays"
    print(f"prompt steps as replays: max |diff| / max |logit| = {worst:.3e}")
    runner.check_device()


@pytest.mark.parametrize("requests", [1, 8, 16])
def test_steps_of_few_tokens_split_their_norms(world, requests, monkeypatch):
    """Decode steps of up to 16 requests run no norm kernel between the first layer's and the final
    one (the products around a norm carry its halves), the same steps with the split switched off
    run two a layer, and both give the plain model's logits."""
    import vllm_from_scratch_b200.kernels as kernels
    from vllm_from_scratch_b200 import StepEntry
    from vllm_from_scratch_b200.kernels import gemm_bf16
    length = 40
    prompts = {f"r{i}": helpers.random_tokens(SHAPE["vocab_size"], length, seed=1200 + i) for i in range(requests)}
    plain = {rid: plain_qwen3.qwen3_logits(SHAPE, world["rounded"], toks)[-1:] for rid, toks in prompts.items()}
    calls = []
    real = kernels.add_rmsnorm
    monkeypatch.setattr(kernels, "add_rmsnorm", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    layers = SHAPE["num_hidden_layers"]
    for split, norm_kernels in ((True, 2), (False, 2 * layers + 1)):
        monkeypatch.setattr(gemm_bf16, "USE_SPLIT_NORM", split)
        runner = make_runner(world, "bfloat16", requests * 4, max_requests=requests)
        for rid, toks in prompts.items():
            runner.manager.admit(rid)
            assert runner.manager.allocate(rid, length)
            runner.step([StepEntry(rid, toks[:-1], 0, [])])
            runner.manager.commit(rid, length - 1)
        calls.clear()
        logits = runner.step([StepEntry(rid, toks[-1:], length - 1, [0]) for rid, toks in prompts.items()])
        assert len(calls) == norm_kernels, (split, len(calls))
        results = {rid: logits[i:i + 1].clone() for i, rid in enumerate(prompts)}
        compare(results, plain, "bfloat16", f"decode step of {requests}, norms split: {split}", world["layers"])
        runner.check_device()
