"""The plain implementation itself: against the reference's saved logits
(tests/golden/, made by make_golden.py from the reference's own model code) and
against simple properties of its parts."""

from __future__ import annotations

from pathlib import Path

import pytest
import torch

import plain_qwen3
import tiny_configs
import vllm_from_scratch_b200 as engine

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_matches_the_reference_models_logits(name):
    saved = torch.load(GOLDEN / f"qwen3_tiny_{name}.pt", weights_only=False)
    entry, config = engine.load_model_config(saved["config"])
    weights = entry.random_weights(config, saved["seed"], dtype=torch.float32, **saved["init"])
    plain = plain_qwen3.qwen3_logits(saved["config"], weights, saved["tokens"])
    assert float((plain - saved["logits"]).abs().max()) < 1e-5
    finer = plain_qwen3.qwen3_logits(saved["config"], weights, saved["tokens"], dtype=torch.float64)
    assert float((finer.float() - saved["logits"]).abs().max()) < 1e-5


def test_parts_behave():
    x = torch.randn(5, 12)
    w = torch.rand(12) + 0.5
    y = plain_qwen3.rms_norm(x, w, 1e-6)
    assert torch.allclose((y / w).pow(2).mean(-1), torch.ones(5), atol=1e-4)
    # rotation keeps lengths and makes scores depend on the distance only
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    def score(pq, pk):
        cq, sq = plain_qwen3.rope_cos_sin(torch.tensor([pq]), 16, 1e4, torch.float32)
        ck, sk = plain_qwen3.rope_cos_sin(torch.tensor([pk]), 16, 1e4, torch.float32)
        return float((plain_qwen3.apply_rope(q, cq, sq) * plain_qwen3.apply_rope(k, ck, sk)).sum())
    assert abs(score(7, 3) - score(104, 100)) < 1e-4
    assert abs(score(7, 3) - score(7, 4)) > 1e-6
    # causal: the first query sees only the first key; a window drops old keys
    qs, ks, vs = torch.randn(6, 2, 8), torch.randn(6, 1, 8), torch.randn(6, 1, 8)
    out = plain_qwen3.causal_attention(qs, ks, vs, 0.3)
    assert torch.allclose(out[0].view(2, 8), vs[0].expand(2, 8), atol=1e-6)
    windowed = plain_qwen3.causal_attention(qs, ks, vs, 0.3, window=1)
    assert torch.allclose(windowed.view(6, 2, 8), vs.expand(6, 2, 8), atol=1e-6)


def test_window_changes_logits_only_past_the_window():
    entry, config = engine.load_model_config(tiny_configs.TINY_C)
    weights = entry.random_weights(config, 5, dtype=torch.float32, **tiny_configs.INIT)
    tokens = list(range(3, 63))
    full = dict(tiny_configs.TINY_C, use_sliding_window=False)
    with_window = plain_qwen3.qwen3_logits(tiny_configs.TINY_C, weights, tokens)
    without = plain_qwen3.qwen3_logits(full, weights, tokens)
    assert torch.allclose(with_window[:24], without[:24], atol=1e-6)
    assert float((with_window[40:] - without[40:]).abs().max()) > 1e-3
