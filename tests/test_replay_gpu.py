"""The engine's step function against the plain implementation, under every way
of cutting requests into steps, in 32-bit and in bfloat16."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
import tiny_configs

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
CONFIGS = {"A": (tiny_configs.TINY_A, 16), "B": (tiny_configs.TINY_B, 8), "C": (tiny_configs.TINY_C, 16),
           "D": (tiny_configs.TINY_D, 16), "E": (tiny_configs.TINY_E, 16), "F": (tiny_configs.TINY_F, 16),
           "G": (tiny_configs.TINY_G, 32), "H": (tiny_configs.TINY_H, 8)}
LENGTHS = {
    "A": {"a": 70, "b": 45, "c": 100, "d": 37, "e": 64, "f": 3, "g": 128},
    "B": {"a": 70, "b": 145, "c": 100, "d": 37, "e": 64, "f": 2, "g": 200},
    "C": {"a": 70, "b": 145, "c": 100, "d": 37, "e": 64, "f": 5, "g": 300},
    "D": {"a": 70, "b": 145, "c": 100, "d": 37, "e": 64, "f": 2, "g": 410},
    "E": {"a": 70, "b": 145, "c": 100, "d": 37, "e": 64, "f": 2, "g": 330},
    "F": {"a": 70, "b": 145, "c": 100, "d": 37, "e": 64, "f": 2, "g": 230},
    "G": {"a": 70, "b": 145, "c": 100, "d": 37, "e": 64, "f": 3, "g": 310},
    "H": {"a": 70, "b": 145, "c": 100, "d": 37, "e": 64, "f": 2, "g": 280},
}
# The bounds (tiny_configs.F32_ATOL, BF16_REL) are twice the worst difference seen.
def tolerance(dtype: str, reference: torch.Tensor, name: str) -> float:
    return tiny_configs.F32_ATOL if dtype == "float32" else tiny_configs.BF16_REL[name] * float(reference.abs().max())


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("models")
    return {name: helpers.make_model_folder(base, raw, seed=3 + i)
            for i, (name, (raw, _)) in enumerate(CONFIGS.items())}


@pytest.fixture(scope="module")
def references(folders):
    out = {}
    for name, folder in folders.items():
        raw = CONFIGS[name][0]
        sequences = {rid: helpers.random_tokens(raw["vocab_size"], n, seed=sum(map(ord, name + rid)))
                     for rid, n in LENGTHS[name].items()}
        plain32 = {rid: helpers.plain_logits(folder, toks) for rid, toks in sequences.items()}
        plain16 = {rid: helpers.plain_logits(folder, toks, round_weights_to=torch.bfloat16)
                   for rid, toks in sequences.items()}
        out[name] = (sequences, {"float32": plain32, "bfloat16": plain16})
    return out


def make_runner(folder, dtype, page_size, num_pages, max_requests=4):
    from vllm_from_scratch_b200 import ModelRunner
    return ModelRunner.from_folder(folder, dtype, page_size, num_pages, max_requests, device="cuda")


def compare(results, expected, dtype, what):
    worst = worst_rel = 0.0
    for rid, logits in results.items():
        reference = expected[rid]
        assert logits.shape == reference.shape, (what, rid, logits.shape, reference.shape)
        diff = (logits - reference).abs()
        bound = tolerance(dtype, reference, what[0])
        if float(diff.max()) > bound:
            position = int(diff.max(dim=1).values.gt(bound).nonzero()[0])
            raise AssertionError(
                f"{what}: request {rid!r} first differs at position {position} "
                f"(max |diff| there {float(diff[position].max()):.3e}, bound {bound:.3e}, "
                f"largest anywhere {float(diff.max()):.3e})")
        worst = max(worst, float(diff.max()))
        worst_rel = max(worst_rel, float(diff.max()) / float(reference.abs().max()))
    print(f"{what}: max |diff| {worst:.3e}, as a fraction of the largest logit {worst_rel:.3e}")


CUTS = {
    "whole": lambda lengths: helpers.cut_whole(lengths),
    "tail": lambda lengths: helpers.cut_tail_one_by_one(lengths, 32),
    "portions": lambda lengths: helpers.cut_changing_portions(lengths, seed=1),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(CONFIGS))
def test_each_request_alone(folders, references, name, cut, dtype):
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    longest = max(LENGTHS[name].values())
    runner = make_runner(folders[name], dtype, page_size, -(-longest // page_size) + 1)
    results = helpers.run_schedule(runner, sequences, CUTS[cut](LENGTHS[name]))
    compare(results, expected[dtype], dtype, f"{name}/{cut}/{dtype}")
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [0, 1])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_mixed_batches_with_few_pages(folders, references, name, seed, dtype):
    """Up to four live requests, portions beside single tokens, and a pool so
    small that pages of finished requests are handed out again at once."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    steps = helpers.cut_mixed(LENGTHS[name], seed=seed, live=4)
    # Smallest pool that never runs dry: the four longest requests, in pages.
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:4])
    runner = make_runner(folders[name], dtype, page_size, pages)
    results = helpers.run_schedule(runner, sequences, steps)
    compare(results, expected[dtype], dtype, f"{name}/mixed{seed}/{dtype}")
    assert runner.manager.stats()["requests"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [2, 3])
@pytest.mark.parametrize("name", ["D", "E"])
def test_mixed_batches_with_long_portions(folders, references, name, seed, dtype):
    """The mixed cut with portions of 64, 100, 130 and 300 tokens: in bfloat16 one step then holds
    single tokens (the decode kernel; for head size 128 the one that also rotates and stores),
    a long portion at a row offset (head size 128: the tcgen05 kernel) and pages used again."""
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    steps = helpers.cut_mixed(LENGTHS[name], seed=seed, live=4, sizes=helpers.LARGE_PORTIONS)
    assert any(n >= 64 for step in steps for _, n in step if len(step) > 1), "a long portion beside other requests"
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:4])
    runner = make_runner(folders[name], dtype, page_size, pages)
    results = helpers.run_schedule(runner, sequences, steps)
    compare(results, expected[dtype], dtype, f"{name}/mixed-long{seed}/{dtype}")
    assert runner.manager.stats()["requests"] == 0
    runner.check_device()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("D", 24), ("D", 48), ("E", 24), ("E", 48)])
def test_pages_whose_size_is_no_power_of_two(folders, references, name, page_size, dtype):
    """Pages of 24 and 48 positions (head sizes 64 and 128): the kernels fed by tensor copies
    refuse them, the ones with per-thread copies serve them."""
    sequences, expected = references[name]
    longest = max(LENGTHS[name].values())
    for cut, steps in (("tail", helpers.cut_tail_one_by_one(LENGTHS[name], 32)),
                       ("portions", helpers.cut_changing_portions(LENGTHS[name], seed=5))):
        runner = make_runner(folders[name], dtype, page_size, -(-longest // page_size) + 1)
        results = helpers.run_schedule(runner, sequences, steps)
        compare(results, expected[dtype], dtype, f"{name}/page{page_size}/{cut}/{dtype}")
    steps = helpers.cut_mixed(LENGTHS[name], seed=6, live=4, sizes=helpers.LARGE_PORTIONS)
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:4])
    runner = make_runner(folders[name], dtype, page_size, pages)
    results = helpers.run_schedule(runner, sequences, steps)
    compare(results, expected[dtype], dtype, f"{name}/page{page_size}/mixed/{dtype}")
    runner.check_device()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "E"])
def test_mixed_steps_as_graph_replays_match_plain(folders, references, name, dtype):
    """The mixed cut through ``MixedGraphs``, twice over (the second pass under other request
    ids): a shape met again is captured for the longest context and replayed.  Both passes
    against the plain model; for head size 128 in bfloat16 the replayed steps hold the decode
    kernel beside the tcgen05 kernel with a key split planned for a length they do not have."""
    from vllm_from_scratch_b200.engine.decode_graph import MixedGraphs
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    steps = helpers.cut_mixed(LENGTHS[name], seed=7, live=4, sizes=helpers.LARGE_PORTIONS)
    pages = sum(sorted((-(-n // page_size) for n in LENGTHS[name].values()), reverse=True)[:4])
    runner = make_runner(folders[name], dtype, page_size, pages)
    graphs = MixedGraphs(runner, raw["max_position_embeddings"], max_graphs=512)
    for suffix in ("", "-again"):
        renamed = {rid + suffix: tokens for rid, tokens in sequences.items()}
        plan = [[(rid + suffix, n) for rid, n in step] for step in steps]
        results = helpers.run_schedule(runner, renamed, plan, step=graphs.run)
        compare({rid[:len(rid) - len(suffix)] if suffix else rid: logits for rid, logits in results.items()},
                expected[dtype], dtype, f"{name}/mixed-graphs{suffix}/{dtype}")
    assert graphs.replays >= len(steps) // 2, "most steps of the second pass must have been replays"
    assert runner.manager.stats()["requests"] == 0
    runner.check_device()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, references, tmp_path, dtype):
    """bin/trace_run in a process of its own, a mixed schedule, a pool of 4 x 128 positions."""
    name = "B"
    raw, page_size = CONFIGS[name]
    sequences, expected = references[name]
    lengths = {rid: min(n, 128) for rid, n in LENGTHS[name].items()}
    sequences = {rid: toks[:lengths[rid]] for rid, toks in sequences.items()}
    steps = helpers.cut_mixed(lengths, seed=5, live=4)
    lines = helpers.schedule_to_trace(sequences, steps)
    out = tmp_path / "out"
    process = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folders[name]), "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(4 * 128)],
        input="\n".join(json.dumps(line) for line in lines) + "\n", capture_output=True, text=True,
        timeout=900, env={**os.environ, "PYTHONPATH": ""})
    assert process.returncode == 0, process.stderr[-3000:]
    assert [l for l in process.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(lines))]
    vocab = raw["vocab_size"]
    done = {rid: 0 for rid in sequences}
    for line in lines:
        data = np.fromfile(out / f"{line['step']}.f32", dtype="<f4").reshape(-1, vocab)
        at = 0
        for entry in line["entries"]:
            n = len(entry["tokens"])
            reference = expected[dtype][entry["id"]][done[entry["id"]]:done[entry["id"]] + n]
            diff = (torch.from_numpy(data[at:at + n].copy()) - reference).abs().max()
            assert float(diff) <= tolerance(dtype, reference, name), (line["step"], entry["id"], float(diff))
            at += n
            done[entry["id"]] += n
        assert at == data.shape[0]
