"""Compare the plain implementation (tests/plain_qwen3.py) with the reference's
own Qwen3 on the CPU, once, and save the reference's logits.

    python tests/golden/make_golden.py /path/to/vllm-from-scratch

For the two tiny configurations A and B it draws this engine's seeded random
weights, loads them into the reference's ``Qwen3ForCausalLM``, runs one whole
sequence through the reference's own runner path on the CPU in float32 (the way
its ``benchmarks/check_step57_model_logits.py:76-116`` does), and writes
``tests/golden/qwen3_tiny_{A,B}.pt`` with the tokens, the seed and the reference's
logits at every position.  ``tests/test_plain.py`` then checks the plain
implementation against these files without needing the reference.
"""

from __future__ import annotations

import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
sys.path.insert(0, str(HERE.parent.parent))

import plain_qwen3  # noqa: E402
import tiny_configs  # noqa: E402


def reference_logits(raw_config: dict, weights: dict, tokens: list[int], block_size: int) -> torch.Tensor:
    from minivllm import (CacheConfig, DeviceConfig, ModelConfig, SamplingParams, SchedulerConfig,
                          VllmConfig)
    from minivllm.core.sched.output import CachedRequestData, NewRequestData, SchedulerOutput
    from minivllm.models.qwen3 import Qwen3ForCausalLM
    from minivllm.worker.gpu_model_runner import GPUModelRunner
    model = Qwen3ForCausalLM(dict(raw_config))
    model.load_weights(iter(sorted(weights.items())))
    model.eval()
    blocks = -(-len(tokens) // block_size)
    config = VllmConfig(
        model_config=ModelConfig(model="(in memory)", dtype="float32", max_model_len=len(tokens) + 8,
                                 hf_config=dict(raw_config)),
        cache_config=CacheConfig(block_size=block_size, num_gpu_blocks=blocks + 1),
        scheduler_config=SchedulerConfig(max_num_seqs=2, max_num_batched_tokens=len(tokens) + 8),
        device_config=DeviceConfig(device="cpu"))
    runner = GPUModelRunner(config, "cpu", model=model)
    runner.initialize_kv_cache(runner.build_kv_cache_config())
    packet = SchedulerOutput(
        scheduled_new_reqs=[NewRequestData(
            req_id="r", prompt_token_ids=list(tokens), sampling_params=SamplingParams(temperature=0.0),
            block_ids=(list(range(blocks)),), num_computed_tokens=0)],
        scheduled_cached_reqs=CachedRequestData.make_empty(),
        num_scheduled_tokens={"r": len(tokens)}, total_num_scheduled_tokens=len(tokens),
        scheduled_spec_decode_tokens={}, finished_req_ids=set())
    runner._update_states(packet)
    inputs = runner._prepare_inputs(packet)
    with torch.no_grad():
        hidden = runner._run_model(inputs)
        return runner.model.compute_logits(hidden).float()


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__)
        return 2
    sys.path.insert(0, sys.argv[1])
    import vllm_from_scratch_b200 as engine
    for name, raw, block_size, length in (("A", tiny_configs.TINY_A, 16, 40), ("B", tiny_configs.TINY_B, 8, 57)):
        entry, config = engine.load_model_config(raw)
        seed = 2024
        weights = entry.random_weights(config, seed, dtype=torch.float32, **tiny_configs.INIT)
        generator = torch.Generator().manual_seed(7)
        tokens = torch.randint(0, raw["vocab_size"], (length,), generator=generator).tolist()
        reference = reference_logits(raw, weights, tokens, block_size)
        plain = plain_qwen3.qwen3_logits(raw, weights, tokens)
        difference = float((reference - plain).abs().max())
        print(f"tiny {name}: reference vs plain max |diff| = {difference:.3e} over {tuple(reference.shape)}")
        assert difference < 1e-5
        torch.save({"config": raw, "seed": seed, "init": tiny_configs.INIT, "tokens": tokens,
                    "logits": reference.to(torch.float32)}, HERE / f"qwen3_tiny_{name}.pt")
    return 0


if __name__ == "__main__":
    sys.exit(main())
