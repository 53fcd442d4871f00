#!/usr/bin/env python3
"""Decode and prefill throughput of the Qwen3-1.7B shape with random weights on
one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of ``--batch`` requests whose contexts start at
``--prompt-len`` tokens.  ``value`` is decoded tokens per second over K steps
timed with CUDA events (inputs packed on the host and copied every step, the
captured decode graph replayed, a greedy token picked on the device); ``e2e`` is
the same through the Python entry point (``LLMEngine.step``: host token ids in,
sampled ids back to the host every step).  One JSON line is printed.
"""

from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Qwen3-1.7B shape.
SHAPE = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 28,
    "hidden_size": 2048, "num_attention_heads": 16, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 6144, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 40960, "hidden_act": "silu",
    "attention_bias": False, "initializer_range": 0.02,
}
FULL_LAYERS = 28
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([field.strip() for field in out.split("\n")[0].split(",")])
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self) -> dict:
        mhz = [int(s[0]) for s in self.samples if s and s[0].isdigit()]
        top = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({name for s in self.samples if len(s) >= 6
                          for name, flag in zip(names, s[2:6]) if flag.lower().startswith("active")})
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(top) if top else None,
                "reasons": reasons, "samples": len(mhz)}


def build_runner(layers: int, max_requests: int, context: int, page_size: int):
    import torch

    import vllm_from_scratch_b200 as engine
    raw = dict(SHAPE, num_hidden_layers=layers)
    entry, config = engine.load_model_config(raw)
    weights = entry.random_weights(config, seed=0, dtype=torch.bfloat16, device="cuda")
    pages = max_requests * (-(-context // page_size)) + 8
    runner = engine.ModelRunner(entry.build_spec(config), weights, "bfloat16", page_size, pages,
                                max_requests, device="cuda", model_config=config)
    del weights
    torch.cuda.empty_cache()
    return runner, config


def random_prompt(vocab: int, length: int, seed: int) -> list[int]:
    import torch
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


def prefill_all(runner, ids: list[str], prompts: list[list[int]], chunk: int):
    """Every prompt into the cache, ``chunk`` tokens a step.  Returns the CUDA-event
    time in ms of the last full-size step (a 2,048-token prefill when chunk = 2048).
    Steps go the way the engine sends them: through the step function the first time a
    shape is seen, as a graph replay of the same step from the second time on."""
    import torch
    from vllm_from_scratch_b200 import StepEntry
    from vllm_from_scratch_b200.engine.decode_graph import MixedGraphs
    steps = MixedGraphs(runner, max(len(p) for p in prompts))
    last_ms = None
    for request_id, prompt in zip(ids, prompts):
        runner.manager.admit(request_id)
        done = 0
        while done < len(prompt):
            count = min(chunk, len(prompt) - done)
            assert runner.manager.allocate(request_id, done + count)
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            begin.record()
            steps.run([StepEntry(request_id, prompt[done:done + count], done, [count - 1])])
            end.record()
            torch.cuda.synchronize()
            if count == chunk:
                last_ms = begin.elapsed_time(end)
            done += count
            runner.manager.commit(request_id, done)
    return last_ms


def decode_loop(runner, graphs, ids: list[str], start: int, steps: int, warmup: int, vocab: int):
    """Teacher-forced decode steps timed on the device.  Returns (ms per step, launches)."""
    import torch

    import vllm_from_scratch_b200.kernels as kernels
    from vllm_from_scratch_b200 import StepEntry
    batch = len(ids)
    generator = torch.Generator().manual_seed(1234)
    feed = torch.randint(0, vocab, (warmup + steps, batch), generator=generator).tolist()
    temperature = torch.zeros(batch, device="cuda")
    zeros_i = torch.zeros(batch, dtype=torch.int32, device="cuda")
    ones_f = torch.ones(batch, device="cuda")
    zeros_f = torch.zeros(batch, device="cuda")
    keys = torch.zeros(batch, dtype=torch.int64, device="cuda")
    picked = torch.empty(batch, dtype=torch.int32, device="cuda")
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    position = start
    launches_before = 0
    for index in range(warmup + steps):
        if index == warmup:
            torch.cuda.synchronize()
            launches_before = kernels.launch_count
            begin.record()
        entries = []
        for row, request_id in enumerate(ids):
            assert runner.manager.allocate(request_id, position + 1)
            entries.append(StepEntry(request_id, [feed[index][row]], position, [0]))
        logits = graphs.run(entries)
        kernels.sample(logits, temperature, zeros_i, ones_f, zeros_f, keys, keys, picked, 1e-5)
        position += 1
    end.record()
    torch.cuda.synchronize()
    eager_launches = kernels.launch_count - launches_before          # the sampling kernel, once a step
    return begin.elapsed_time(end) / steps, eager_launches, position


def measure_point(runner, config, batch: int, prompt_len: int, steps: int, warmup: int, context: int,
                  want_prefill: bool):
    import torch

    import vllm_from_scratch_b200.kernels as kernels
    from vllm_from_scratch_b200.engine.decode_graph import DecodeGraphs
    ids = [f"bench-{batch}-{i}" for i in range(batch)]
    prompts = [random_prompt(config.vocab_size, prompt_len, seed=100 + i) for i in range(batch)]
    prefill_ms = prefill_all(runner, ids, prompts, prompt_len)
    graphs = DecodeGraphs(runner, batch, context)
    before = kernels.launch_count
    # The first run captures the graph: its launch count is the kernels in one replay.
    ms, eager_launches, position = decode_loop(runner, graphs, ids, prompt_len, 1, 1, config.vocab_size)
    per_replay = kernels.launch_count - before - 2          # minus the two sampling launches
    # capture ran the body twice (warm-up and capture), replay once more without Python launches
    per_replay //= 2
    ms, eager_launches, position = decode_loop(runner, graphs, ids, position, steps, warmup, config.vocab_size)
    mean_context = position - steps / 2
    for request_id in ids:
        runner.manager.release(request_id)
    del graphs
    torch.cuda.empty_cache()
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "launches": per_replay * steps + eager_launches,
            "mean_context": mean_context, "prefill_ms": prefill_ms if want_prefill else None}


def measure_e2e(runner, config, batch: int, prompt_len: int, steps: int, warmup: int, context: int):
    """The same decode steps through LLMEngine.step: host ids in, sampled ids out."""
    import torch

    import vllm_from_scratch_b200 as engine
    llm = engine.LLMEngine(engine.EngineConfig(
        engine.ModelConfig("(random weights)", "bfloat16", context),
        engine.CacheConfig(runner.storage.page_size, runner.storage.num_pages),
        engine.SchedulerConfig(batch, prompt_len, async_scheduling=True)), runner=runner)
    params = engine.SamplingParams(temperature=0.0, max_tokens=warmup + steps + batch + 8, ignore_eos=True)
    for i in range(batch):
        llm.add_request(f"e2e-{i}", random_prompt(config.vocab_size, prompt_len, seed=300 + i), params)
    while llm.scheduler.waiting:            # prompts, one per step under the token budget
        llm.step()
    for _ in range(warmup):
        llm.step()
    torch.cuda.synchronize()
    started = time.perf_counter()
    tokens = 0
    for _ in range(steps):
        tokens += len(llm.step())
    torch.cuda.synchronize()
    seconds = time.perf_counter() - started
    llm.abort_request([f"e2e-{i}" for i in range(batch)])
    # per step: the packed int32 inputs go up, one int32 token per request comes back
    h2d = llm.decode_graphs.last_h2d_bytes + batch * (4 * 4 + 8 * 2)
    return {"value": tokens / seconds, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * batch, "ms_per_step": 1000 * seconds / steps,
            "async_scheduling": True, "steps_ahead": llm.num_steps_ahead}


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--layers", type=int, default=FULL_LAYERS)
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    args = parser.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference has no setup.py or pyproject.toml: pip reports "
                          "'Directory is not installable', so baseline/_ref cannot be made"}))
        return 0
    if args.gpus != 1:
        print("bench.py measures one GPU only: this engine is built for a single B200 (--gpus 1)")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    if not torch.cuda.is_available():
        print("bench.py needs a CUDA device")
        return 1
    measured, peak_kind = peaks()
    largest = 64 if not args.no_points else args.batch
    runner, config = build_runner(args.layers, max(largest, args.batch), args.context, args.block_size)

    with ClockSampler() as clocks:
        main_point = measure_point(runner, config, args.batch, args.prompt_len, args.steps, args.warmup,
                                   args.context, want_prefill=True)
        e2e = measure_e2e(runner, config, args.batch, args.prompt_len, args.steps, args.warmup, args.context)
    points = {}
    if not args.no_points:
        for batch in (1, 64):
            point = measure_point(runner, config, batch, args.prompt_len, max(8, args.steps // 4), 3,
                                  args.context, want_prefill=False)
            points[f"decode_b{batch}"] = round(point["tok_s"], 1)

    weight_bytes = runner.model.num_weight_bytes()
    kv_bytes = args.batch * main_point["mean_context"] * runner.storage.bytes_per_token()
    achieved = (weight_bytes + kv_bytes) / (main_point["ms"] * 1e-3) / 1e9
    # prefill flops: 2 * tokens * matrix parameters (the output product runs on one row only)
    # + causal attention 2 * 2 * T^2 / 2 * heads * head_dim per layer
    tokens = args.prompt_len
    matrix_params = config.num_hidden_layers * (
        config.hidden_size * (config.q_width + 2 * config.kv_width) + config.q_width * config.hidden_size
        + 3 * config.hidden_size * config.intermediate_size)
    flops = 2 * tokens * matrix_params + config.num_hidden_layers * 2 * tokens * tokens * config.q_width \
        + 2 * config.vocab_size * config.hidden_size
    prefill_ms = main_point["prefill_ms"]
    prefill = {"value": round(tokens * 1000.0 / prefill_ms, 1), "tokens": tokens, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (measured["bf16_tflops"] * 1e12), 4)}

    record = {
        "metric": "decode tokens/s (Qwen3-1.7B shape, bf16, random weights)",
        "value": round(main_point["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_point["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": "Qwen3-1.7B shape", "global_batch": args.batch, "seq_len": args.context,
            "prompt_len": args.prompt_len, "parallelism": "single", "layers": args.layers,
            "layers_full": FULL_LAYERS, "hidden": config.hidden_size, "heads": config.num_attention_heads,
            "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim,
            "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "block_size": args.block_size, "tied": config.tie_word_embeddings,
            "l2": "inputs larger than L2 (weights read every step)", "peaks": peak_kind,
        },
        "e2e": {k: (round(v, 2) if isinstance(v, float) else v) for k, v in e2e.items()},
        "gpu_launches": int(main_point["launches"]),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": measured["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / measured["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.summary(),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
