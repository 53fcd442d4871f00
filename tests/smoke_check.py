"""A few greedy tokens from a tiny random model on cuda:0, compared with the plain
implementation.  Used by ``__graft_entry__.smoke``."""

from __future__ import annotations

import tempfile
from pathlib import Path

import torch

import helpers
import tiny_configs


def run() -> None:
    import vllm_from_scratch_b200 as engine
    with tempfile.TemporaryDirectory() as scratch:
        folder = helpers.make_model_folder(Path(scratch), tiny_configs.TINY_A, seed=21)
        prompts = [helpers.random_tokens(256, n, seed=n) for n in (5, 17, 33)]
        for dtype in ("float32", "bfloat16"):
            llm = engine.LLM(folder, dtype=dtype, max_model_len=128, block_size=16, max_num_seqs=4,
                             max_num_batched_tokens=32)
            outputs = llm.generate(prompts, engine.SamplingParams(temperature=0.0, max_tokens=6))
            for prompt, output in zip(prompts, outputs):
                tokens = list(prompt)
                for index, token in enumerate(output.token_ids):
                    logits = helpers.plain_logits(
                        folder, tokens, round_weights_to=None if dtype == "float32" else torch.bfloat16)[-1]
                    best = torch.topk(logits, 2)
                    margin = float(best.values[0] - best.values[1])
                    tie = 1e-4 if dtype == "float32" else 0.1
                    if token != int(best.indices[0]):
                        if margin < tie:
                            break       # a near-tie may go either way; the sequences part here
                        raise AssertionError(
                            f"{dtype}: prompt of {len(prompt)}, token {index}: engine {token}, "
                            f"plain {int(best.indices[0])} (margin {margin:.3e})")
                    tokens.append(token)
            print(f"smoke {dtype}: {[o.token_ids for o in outputs]} agree with the plain implementation")
