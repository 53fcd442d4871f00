#!/usr/bin/env python3
"""Decode and prefill throughput of dense Qwen3 shapes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]
                    [--shape 1.7b|8b|32b] [--batch B] [--no-points]

``--shape 1.7b`` (the default): a step is one decode step of ``--batch`` requests whose
contexts start at ``--prompt-len`` tokens.  ``value`` is decoded tokens per second timed with
CUDA events (inputs packed on the host and copied every step, the captured decode graph
replayed, a greedy token picked on the device); ``e2e`` is the same through the Python entry
point (``LLMEngine.step``: host token ids in, sampled ids back to the host every step), with
the engine's defaults and with the queueing of steps ahead switched off.  ``prefill`` is one 2,048-token prompt,
``points`` hold decoding at batch 1 and 64 and, from runs of this program in processes of their
own, the two larger shapes.

``--shape 8b``: a step is a mixed batch, 64 requests that decode beside a 2,048-token portion of
a prompt, at contexts up to 8192.  ``--shape 32b``: decode steps at batch 1, 8 and 64 with the
cache pool sized from the memory that is free once the weights are loaded.

Every figure is the median of at least three timed regions of at least 200 ms each (``--steps``
is the least number of steps in a region); one JSON line is printed.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))


def _qwen3(layers, hidden, heads, inter, tied):
    return {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": layers,
        "hidden_size": hidden, "num_attention_heads": heads, "num_key_value_heads": 8, "head_dim": 128,
        "intermediate_size": inter, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
        "tie_word_embeddings": tied, "max_position_embeddings": 40960, "hidden_act": "silu",
        "attention_bias": False, "initializer_range": 0.02,
    }


# name -> (label, config.json, context length of the measurement)
SHAPES = {
    "1.7b": ("Qwen3-1.7B shape", _qwen3(28, 2048, 16, 6144, True), 4096),
    "8b": ("Qwen3-8B shape", _qwen3(36, 4096, 32, 12288, False), 8192),
    "32b": ("Qwen3-32B shape", _qwen3(64, 5120, 64, 25600, False), 4096),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
MIN_REGION_MS = 200.0
MIN_REPEATS = 3


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        return json.loads(path.read_text()), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while a timed region runs."""

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
            self._stop.wait(0.1)

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


def spread(values: list[float]) -> float:
    middle = statistics.median(values)
    return round((max(values) - min(values)) / middle, 4) if middle else 0.0


# ----------------------------------------------------------------------------- our engine
def build_runner(raw: dict, max_requests: int, tokens_in_pool: int | None, page_size: int):
    """Random weights drawn on the device; the pool holds ``tokens_in_pool`` positions, or, when
    that is None, what the free memory holds once the weights are loaded."""
    import torch

    import vllm_from_scratch_b200 as engine
    entry, config = engine.load_model_config(raw)
    weights = entry.random_weights(config, seed=0, dtype=torch.bfloat16, device="cuda")
    spec = entry.build_spec(config)
    pages = 1 if tokens_in_pool is None else -(-tokens_in_pool // page_size) + 8
    runner = engine.ModelRunner(spec, weights, "bfloat16", page_size, pages, max_requests, device="cuda",
                                model_config=config)
    # The parts keep their own (packed) copies of the matrices: let go of the drawn ones.
    weights.clear()
    del weights
    if tokens_in_pool is None:
        runner.rebuild_cache(page_size, runner.pages_that_fit(page_size, 0.9, 6 << 30))
    torch.cuda.empty_cache()
    return runner, config


def random_prompt(vocab: int, length: int, seed: int) -> list[int]:
    import torch
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


def fill_cache_randomly(runner) -> None:
    """Keys and values of the whole pool drawn at random (scaled like normalised keys): what a
    decode step reads is then as real as what a prefill would have left, without running one."""
    for group in runner.storage.groups:
        for layer in range(group.slab.shape[0]):
            group.slab[layer].normal_(0.0, 1.0)


def hold_context(runner, request_id: str, tokens: int) -> None:
    """A request that owns ``tokens`` positions of (randomly filled) cache."""
    runner.manager.admit(request_id)
    assert runner.manager.allocate(request_id, tokens), "the pool is too small for the benchmark's requests"
    runner.manager.commit(request_id, tokens)


def prefill_all(runner, ids: list[str], prompts: list[list[int]]) -> None:
    """Every prompt into the cache, one prompt a step, the way the engine sends such steps: through
    the step function the first time a shape is seen, as a graph replay from the second time on."""
    from vllm_from_scratch_b200 import StepEntry
    from vllm_from_scratch_b200.engine.decode_graph import MixedGraphs
    steps = MixedGraphs(runner, max(len(p) for p in prompts))
    for request_id, prompt in zip(ids, prompts):
        runner.manager.admit(request_id)
        assert runner.manager.allocate(request_id, len(prompt))
        steps.run([StepEntry(request_id, prompt, 0, [len(prompt) - 1])])
        runner.manager.commit(request_id, len(prompt))


def measure_prefill(runner, config, tokens: int) -> dict:
    """One prompt of ``tokens`` tokens in one step (one row of logits), as a graph replay: steps of
    different requests queued one behind the other the way the engine queues steps that sample
    nothing (the host packs the next while the device runs the last), timed by CUDA events around
    regions of them: the median per step over at least three regions of at least 200 ms."""
    import torch
    from vllm_from_scratch_b200 import StepEntry
    from vllm_from_scratch_b200.engine.decode_graph import MixedGraphs
    steps = MixedGraphs(runner, tokens)
    counter = [0]

    def one_step() -> None:
        request_id = f"prefill-{counter[0]}"
        prompt = random_prompt(config.vocab_size, tokens, seed=5000 + counter[0] % 7)
        counter[0] += 1
        runner.manager.admit(request_id)
        assert runner.manager.allocate(request_id, tokens)
        steps.run([StepEntry(request_id, prompt, 0, [tokens - 1])])
        runner.manager.release(request_id)

    def region(count: int) -> float:
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(count):
            one_step()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / count

    for _ in range(3):                      # the first goes the ordinary way, the second is the capture
        one_step()
    torch.cuda.synchronize()
    with ClockSampler() as clocks:
        estimate = region(3)
        count = max(3, math.ceil(MIN_REGION_MS / estimate))
        times = [region(count) for _ in range(MIN_REPEATS)]
    return {"ms": statistics.median(times), "repeats": len(times), "steps_timed": count, "spread": spread(times),
            "clocks": clocks.summary()}


class DecodeLoop:
    """Teacher-forced decode steps of a fixed set of requests, timed on the device."""

    def __init__(self, runner, ids: list[str], start: int, context: int, vocab: int) -> None:
        import torch
        from vllm_from_scratch_b200.engine.decode_graph import DecodeGraphs
        self.runner, self.ids, self.position, self.vocab = runner, ids, start, vocab
        self.graphs = DecodeGraphs(runner, len(ids), context)
        batch = len(ids)
        self.generator = torch.Generator().manual_seed(1234)
        self.temperature = torch.zeros(batch, device="cuda")
        self.zeros_i = torch.zeros(batch, dtype=torch.int32, device="cuda")
        self.ones_f = torch.ones(batch, device="cuda")
        self.zeros_f = torch.zeros(batch, device="cuda")
        self.keys = torch.zeros(batch, dtype=torch.int64, device="cuda")
        self.picked = torch.empty(batch, dtype=torch.int32, device="cuda")

    def run(self, steps: int) -> float:
        """``steps`` decode steps; returns the CUDA-event time of all of them in ms."""
        import torch

        import vllm_from_scratch_b200.kernels as kernels
        from vllm_from_scratch_b200 import StepEntry
        feed = torch.randint(0, self.vocab, (steps, len(self.ids)), generator=self.generator).tolist()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        begin.record()
        for index in range(steps):
            entries = []
            for row, request_id in enumerate(self.ids):
                assert self.runner.manager.allocate(request_id, self.position + 1)
                entries.append(StepEntry(request_id, [feed[index][row]], self.position, [0]))
            logits = self.graphs.run(entries)
            kernels.sample(logits, self.temperature, self.zeros_i, self.ones_f, self.zeros_f, self.keys, self.keys,
                           self.picked, 1e-5, 1)        # every row is greedy: the kernel for rows without a filter alone
            self.position += 1
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end)


def measure_decode(runner, config, batch: int, start: int, steps: int, warmup: int, context: int,
                   prompts: list[list[int]] | None):
    """Decode steps at ``batch``: median over at least three regions of at least 200 ms.  With
    ``prompts`` they are prefilled first (and the prefill step is timed), else the requests take
    over ``start`` positions of the randomly filled cache."""
    import vllm_from_scratch_b200.kernels as kernels
    ids = [f"bench-{batch}-{i}" for i in range(batch)]
    if prompts is not None:
        prefill_all(runner, ids, prompts)
    else:
        for request_id in ids:
            hold_context(runner, request_id, start)
    loop = DecodeLoop(runner, ids, start, context, config.vocab_size)
    before = kernels.launch_count
    loop.run(1)                                             # captures the graph: warm-up run, capture, replay
    per_replay = (kernels.launch_count - before - 1) // 2   # the body ran twice under Python; minus one sampling launch
    with ClockSampler() as clocks:
        estimate = loop.run(max(warmup, 3)) / max(warmup, 3)
        room = context - loop.position - 2
        region = max(steps, math.ceil(MIN_REGION_MS / estimate))
        region = max(1, min(region, room // MIN_REPEATS))
        first_position = loop.position
        regions = [loop.run(region) / region for _ in range(MIN_REPEATS)]
    ms = statistics.median(regions)
    mean_context = (first_position + loop.position) / 2
    for request_id in ids:
        runner.manager.release(request_id)
    del loop
    import torch
    torch.cuda.empty_cache()
    return {"ms": ms, "tok_s": batch * 1000.0 / ms, "steps_timed": region, "repeats": MIN_REPEATS,
            "spread": spread(regions), "launches": (per_replay + 1) * region, "mean_context": mean_context,
            "clocks": clocks.summary()}


def measure_e2e(runner, config, batch: int, prompt_len: int, steps: int, warmup: int, context: int,
                ahead: bool):
    """The same decode steps through LLMEngine.step: host ids in, sampled ids out."""
    import torch

    import vllm_from_scratch_b200 as engine
    llm = engine.LLMEngine(engine.EngineConfig(
        engine.ModelConfig("(random weights)", "bfloat16", context),
        engine.CacheConfig(runner.storage.page_size, runner.storage.num_pages),
        engine.SchedulerConfig(batch, prompt_len, async_scheduling=ahead)), runner=runner)
    params = engine.SamplingParams(temperature=0.0, max_tokens=context - prompt_len - 1, ignore_eos=True)
    ids = [f"e2e-{int(ahead)}-{i}" for i in range(batch)]
    for i, request_id in enumerate(ids):
        llm.add_request(request_id, random_prompt(config.vocab_size, prompt_len, seed=300 + i), params)
    while llm.scheduler.waiting:            # prompts, one per step under the token budget
        llm.step()
    for _ in range(max(warmup, 3)):
        llm.step()

    def region(count: int) -> tuple[float, int]:
        torch.cuda.synchronize()
        started = time.perf_counter()
        tokens = 0
        for _ in range(count):
            tokens += len(llm.step())
        torch.cuda.synchronize()
        return time.perf_counter() - started, tokens

    seconds, _ = region(4)
    count = max(steps, math.ceil(MIN_REGION_MS / (1000.0 * seconds / 4)))
    rates, per_step = [], []
    for _ in range(MIN_REPEATS):
        seconds, tokens = region(count)
        rates.append(tokens / seconds)
        per_step.append(1000.0 * seconds / count)
    llm.abort_request(ids)
    llm.step()                              # the plan that carries the finished notices
    # per step: the packed int32 inputs go up; one int32 token per request and the status words come back
    h2d = llm.decode_graphs.last_h2d_bytes + batch * (4 * 4 + 8 * 2)
    from vllm_from_scratch_b200.kernels import STATUS_WORDS
    return {"value": round(statistics.median(rates), 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": 4 * (batch + STATUS_WORDS), "ms_per_step": round(statistics.median(per_step), 4),
            "async_scheduling": ahead, "steps_ahead": llm.num_steps_ahead, "steps_timed": count,
            "repeats": MIN_REPEATS, "spread": spread(rates)}


def flat_config(label, raw, args, context, peak_kind, extra=None) -> dict:
    config = {
        "model": label, "global_batch": args.batch, "seq_len": context, "prompt_len": args.prompt_len,
        "parallelism": "single", "layers": args.layers or raw["num_hidden_layers"],
        "layers_full": raw["num_hidden_layers"], "hidden": raw["hidden_size"],
        "heads": raw["num_attention_heads"], "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
        "intermediate": raw["intermediate_size"], "vocab": raw["vocab_size"], "block_size": args.block_size,
        "tied": raw["tie_word_embeddings"], "l2": "inputs larger than L2 (weights read every step)",
        "peaks": peak_kind,
    }
    config.update(extra or {})
    assert len(config) <= 20
    return config


def sub_shape(name: str, args) -> dict | None:
    """The line of another shape, measured by this program in a process of its own."""
    command = [sys.executable, str(ROOT / "bench.py"), "--shape", name, "--steps", str(args.steps),
               "--warmup", str(args.warmup), "--no-points"]
    try:
        done = subprocess.run(command, capture_output=True, text=True, timeout=900)
        for line in reversed(done.stdout.strip().split("\n")):
            if line.startswith("{"):
                return json.loads(line)
        print(f"bench.py --shape {name} printed no line (exit {done.returncode}): {done.stderr[-400:]}",
              file=sys.stderr)
    except Exception as error:              # the main line must not be lost to a side measurement
        print(f"bench.py --shape {name} failed: {error!r}", file=sys.stderr)
    return None


def run_small(args, measured, peak_kind) -> dict:
    """The Qwen3-1.7B shape: decode at ``--batch`` (the line's value), e2e, prefill, batch 1 and 64."""
    label, raw, context = SHAPES["1.7b"]
    raw = dict(raw, num_hidden_layers=args.layers or raw["num_hidden_layers"])
    context = args.context or context
    largest = args.batch if args.no_points else max(64, args.batch)
    runner, config = build_runner(raw, largest, largest * context, args.block_size)
    prompts = [random_prompt(config.vocab_size, args.prompt_len, seed=100 + i) for i in range(args.batch)]
    main_point = measure_decode(runner, config, args.batch, args.prompt_len, args.steps, args.warmup, context, prompts)
    with ClockSampler() as e2e_clocks:
        e2e_plain = measure_e2e(runner, config, args.batch, args.prompt_len, args.steps, args.warmup, context, False)
        e2e_default = measure_e2e(runner, config, args.batch, args.prompt_len, args.steps, args.warmup, context, True)
    prefill_point = measure_prefill(runner, config, args.prompt_len)
    points, point_notes = {}, {}
    if not args.no_points:
        for batch in (1, 64):
            more = [random_prompt(config.vocab_size, args.prompt_len, seed=700 + i) for i in range(batch)]
            point = measure_decode(runner, config, batch, args.prompt_len, args.steps, args.warmup, context, more)
            points[f"decode_b{batch}"] = round(point["tok_s"], 1)
            point_notes[f"decode_b{batch}"] = {"ms": round(point["ms"], 4), "spread": point["spread"],
                                               "steps_timed": point["steps_timed"], "clocks": point["clocks"]}
    weight_bytes = runner.model.num_weight_bytes()
    kv_bytes = args.batch * main_point["mean_context"] * runner.storage.bytes_per_token()
    achieved = (weight_bytes + kv_bytes) / (main_point["ms"] * 1e-3) / 1e9
    del runner
    import torch
    torch.cuda.empty_cache()
    if not args.no_points:
        mixed = sub_shape("8b", args)
        if mixed is not None:
            points["mixed_8b_tok_s"] = mixed["value"]
            points["mixed_8b_ms"] = mixed["ms_per_step"]
            points["mixed_8b_frac"] = mixed["roofline"]["frac"]
        large = sub_shape("32b", args)
        if large is not None:
            points["decode_32b_b8"] = large["value"]
            points["decode_32b_b8_frac"] = large["roofline"]["frac"]
            points.update({f"decode_32b_{key.split('_')[1]}": value for key, value in large["points"].items()})
    # prefill flops: 2 * tokens * matrix parameters (the output product runs on one row only)
    # + causal attention 2 * 2 * T^2 / 2 * heads * head_dim per layer
    tokens = args.prompt_len
    matrix_params = config.num_hidden_layers * (
        config.hidden_size * (config.q_width + 2 * config.kv_width) + config.q_width * config.hidden_size
        + 3 * config.hidden_size * config.intermediate_size)
    flops = 2 * tokens * matrix_params + config.num_hidden_layers * 2 * tokens * tokens * config.q_width \
        + 2 * config.vocab_size * config.hidden_size
    prefill_ms = prefill_point["ms"]
    prefill = {"value": round(tokens * 1000.0 / prefill_ms, 1), "tokens": tokens, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (measured["bf16_tflops"] * 1e12), 4),
               "repeats": prefill_point["repeats"], "steps_timed": prefill_point["steps_timed"],
               "spread": prefill_point["spread"], "clocks": prefill_point["clocks"]}
    return {
        "metric": "decode tokens/s (Qwen3-1.7B shape, bf16, random weights)",
        "value": round(main_point["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_point["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": flat_config(label, raw, args, context, peak_kind),
        "repeats": main_point["repeats"], "steps_timed": main_point["steps_timed"], "spread": main_point["spread"],
        # the engine's defaults (decode steps queued ahead); beside it the same with that switched off
        "e2e": {**e2e_default, "without_steps_queued_ahead": e2e_plain, "clocks": e2e_clocks.summary()},
        "gpu_launches": int(main_point["launches"]),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": measured["hbm_gbs"],
                     "unit": "GB/s", "frac": round(achieved / measured["hbm_gbs"], 4)},
        "points": points, "point_notes": point_notes,
        "clocks": main_point["clocks"],
    }


def run_mixed(args, measured, peak_kind) -> dict:
    """The Qwen3-8B shape: 64 requests decode beside a 2,048-token portion of a prompt; the prompt
    has 8192 tokens, so its four portions meet 0, 2048, 4096 and 6144 cached positions."""
    import torch
    from vllm_from_scratch_b200 import StepEntry
    from vllm_from_scratch_b200.engine.decode_graph import MixedGraphs
    import vllm_from_scratch_b200.kernels as kernels
    label, raw, context = SHAPES["8b"]
    raw = dict(raw, num_hidden_layers=args.layers or raw["num_hidden_layers"])
    decoders, portion, decode_context = 64, 2048, 4096
    runner, config = build_runner(raw, decoders + 1, decoders * (decode_context + 256) + context, args.block_size)
    fill_cache_randomly(runner)
    ids = [f"dec-{i}" for i in range(decoders)]
    for request_id in ids:
        hold_context(runner, request_id, decode_context)
    graphs = MixedGraphs(runner, context)
    generator = torch.Generator().manual_seed(7)
    position = decode_context
    launches = [0]

    def one_prompt(number: int) -> list[float]:
        """An 8192-token prompt in four portions, each beside the 64 decoding requests."""
        nonlocal position
        rid = f"prompt-{number}"
        runner.manager.admit(rid)
        prompt = torch.randint(0, config.vocab_size, (context,), generator=generator).tolist()
        feed = torch.randint(0, config.vocab_size, (context // portion, decoders), generator=generator).tolist()
        times = []
        for index, start in enumerate(range(0, context, portion)):
            entries = []
            for row, request_id in enumerate(ids):
                assert runner.manager.allocate(request_id, position + 1)
                entries.append(StepEntry(request_id, [feed[index][row]], position, [0]))
            assert runner.manager.allocate(rid, start + portion)
            entries.append(StepEntry(rid, prompt[start:start + portion], start, [portion - 1]))
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before = kernels.launch_count
            torch.cuda.synchronize()
            begin.record()
            graphs.run(entries)
            end.record()
            torch.cuda.synchronize()
            launches[0] = max(launches[0], kernels.launch_count - before)
            times.append(begin.elapsed_time(end))
            runner.manager.commit(rid, start + portion)
            position += 1
        runner.manager.release(rid)
        return times

    for number in range(2):                 # the ordinary path, then the capture
        one_prompt(number)
    per_replay = launches[0] // 2           # the capture ran the body twice under Python
    with ClockSampler() as clocks:
        rounds = [one_prompt(2 + number) for number in range(max(MIN_REPEATS, args.steps // 4, 1))]
        while sum(map(sum, rounds)) < MIN_REPEATS * MIN_REGION_MS:
            rounds.append(one_prompt(2 + len(rounds)))
    per_round = [statistics.mean(times) for times in rounds]
    ms = statistics.median(per_round)
    tokens = decoders + portion
    by_portion = [round(statistics.median(times[i] for times in rounds), 3) for i in range(context // portion)]
    # Floors: every matrix product over 2112 rows (the output product over 65), attention of the
    # portion over what it sees and of the decoders over their contexts; bytes: the weights once,
    # the decoders' cache, the cache the portion reads and writes.
    layers = config.num_hidden_layers
    matrix_params = layers * (
        config.hidden_size * (config.q_width + 2 * config.kv_width) + config.q_width * config.hidden_size
        + 3 * config.hidden_size * config.intermediate_size)
    mean_seen = sum(start + portion / 2 for start in range(0, context, portion)) / (context // portion)
    flops = (2 * tokens * matrix_params + 2 * (decoders + 1) * config.vocab_size * config.hidden_size
             + layers * 4 * portion * mean_seen * config.q_width
             + layers * 4 * decoders * (position - 2) * config.q_width)
    per_token = runner.storage.bytes_per_token()
    bytes_read = runner.model.num_weight_bytes() + decoders * position * per_token + (mean_seen + portion / 2) * per_token
    flop_ms = flops / (measured["bf16_tflops"] * 1e12) * 1e3
    hbm_ms = bytes_read / (measured["hbm_gbs"] * 1e9) * 1e3
    floor = max(flop_ms, hbm_ms)
    return {
        "metric": "tokens/s of a mixed step: 64 decoding requests beside a 2,048-token prompt portion "
                  "(Qwen3-8B shape, bf16, random weights)",
        "value": round(tokens * 1000.0 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": flat_config(label, raw, dict_args(args, batch=decoders + 1, prompt_len=portion), context, peak_kind,
                              {"decoders": decoders, "decode_context": decode_context}),
        "repeats": len(rounds), "steps_timed": 4 * len(rounds), "spread": spread(per_round),
        "ms_by_portion_start": dict(zip(map(str, range(0, context, portion)), by_portion)),
        "gpu_launches": int(per_replay * 4 * len(rounds)),
        "roofline": {"bound": "flops" if flop_ms >= hbm_ms else "hbm", "flop_floor_ms": round(flop_ms, 3),
                     "hbm_floor_ms": round(hbm_ms, 3), "achieved": round(flops / (ms * 1e-3) / 1e12, 1),
                     "peak": measured["bf16_tflops"], "unit": "TFLOP/s", "frac": round(floor / ms, 4)},
        "points": {}, "clocks": clocks.summary(),
    }


def dict_args(args, **changes):
    copy = argparse.Namespace(**vars(args))
    for key, value in changes.items():
        setattr(copy, key, value)
    return copy


def run_large(args, measured, peak_kind) -> dict:
    """The Qwen3-32B shape: decode at batch 1, 8 and 64 with the pool sized from what is free."""
    label, raw, context = SHAPES["32b"]
    raw = dict(raw, num_hidden_layers=args.layers or raw["num_hidden_layers"])
    context = args.context or context
    runner, config = build_runner(raw, 64, None, args.block_size)
    pool_tokens = runner.storage.num_pages * args.block_size
    if pool_tokens < 64 * context:
        print(f"the pool holds {pool_tokens} positions, fewer than 64 x {context}", file=sys.stderr)
    fill_cache_randomly(runner)
    results = {}
    for batch in (8, 1, 64):
        results[batch] = measure_decode(runner, config, batch, args.prompt_len, args.steps, args.warmup, context, None)
    main_point = results[8]
    weight_bytes = runner.model.num_weight_bytes()
    per_token = runner.storage.bytes_per_token()

    def fraction(batch):
        moved = weight_bytes + batch * results[batch]["mean_context"] * per_token
        return moved / (results[batch]["ms"] * 1e-3) / 1e9

    return {
        "metric": "decode tokens/s (Qwen3-32B shape, bf16, random weights)",
        "value": round(main_point["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(main_point["ms"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": flat_config(label, raw, dict_args(args, batch=8), context, peak_kind,
                              {"pool_pages": runner.storage.num_pages, "pool": "sized from free memory"}),
        "repeats": main_point["repeats"], "steps_timed": main_point["steps_timed"], "spread": main_point["spread"],
        "gpu_launches": int(main_point["launches"]),
        "roofline": {"bound": "hbm", "achieved": round(fraction(8), 1), "peak": measured["hbm_gbs"],
                     "unit": "GB/s", "frac": round(fraction(8) / measured["hbm_gbs"], 4)},
        "points": {f"decode_b{batch}": round(results[batch]["tok_s"], 1) for batch in (1, 64)},
        "point_notes": {f"decode_b{batch}": {"ms": round(results[batch]["ms"], 4),
                                             "frac": round(fraction(batch) / measured["hbm_gbs"], 4),
                                             "spread": results[batch]["spread"], "clocks": results[batch]["clocks"]}
                        for batch in (1, 64)},
        "clocks": main_point["clocks"],
    }


# -------------------------------------------------------------------------- the reference
REFERENCE_ROOT = ROOT / "baseline" / "_ref"


def write_reference_model(raw: dict, folder: Path) -> None:
    """config.json and model.safetensors with random weights under the checkpoint's names, drawn
    with torch alone (nothing of this repository's engine is on the reference arm's path)."""
    import torch
    from safetensors.torch import save_file
    generator = torch.Generator(device="cuda").manual_seed(0)
    hidden, inter, d = raw["hidden_size"], raw["intermediate_size"], raw["head_dim"]
    q_width, kv_width = raw["num_attention_heads"] * d, raw["num_key_value_heads"] * d

    def matrix(rows, columns):
        return torch.empty(rows, columns, device="cuda").normal_(0.0, raw["initializer_range"], generator=generator
                                                                 ).to(torch.bfloat16).cpu()

    def norm(size):
        return (1.0 + torch.empty(size, device="cuda").normal_(0.0, 0.1, generator=generator)).to(torch.bfloat16).cpu()

    tensors = {"model.embed_tokens.weight": matrix(raw["vocab_size"], hidden), "model.norm.weight": norm(hidden)}
    for index in range(raw["num_hidden_layers"]):
        prefix = f"model.layers.{index}."
        tensors[prefix + "input_layernorm.weight"] = norm(hidden)
        tensors[prefix + "post_attention_layernorm.weight"] = norm(hidden)
        tensors[prefix + "self_attn.q_proj.weight"] = matrix(q_width, hidden)
        tensors[prefix + "self_attn.k_proj.weight"] = matrix(kv_width, hidden)
        tensors[prefix + "self_attn.v_proj.weight"] = matrix(kv_width, hidden)
        tensors[prefix + "self_attn.o_proj.weight"] = matrix(hidden, q_width)
        tensors[prefix + "self_attn.q_norm.weight"] = norm(d)
        tensors[prefix + "self_attn.k_norm.weight"] = norm(d)
        tensors[prefix + "mlp.gate_proj.weight"] = matrix(inter, hidden)
        tensors[prefix + "mlp.up_proj.weight"] = matrix(inter, hidden)
        tensors[prefix + "mlp.down_proj.weight"] = matrix(hidden, inter)
    if not raw["tie_word_embeddings"]:
        tensors["lm_head.weight"] = matrix(raw["vocab_size"], hidden)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(raw, indent=2))
    save_file(tensors, str(folder / "model.safetensors"))


def ensure_reference_copy() -> bool:
    """``baseline/_ref/minivllm``, a plain copy of the reference's source tree (it needs no
    installation): made, if it is missing, from ``$REFERENCE_SOURCE`` or from a folder ``reference``
    beside this repository.  False if there is neither."""
    if (REFERENCE_ROOT / "minivllm" / "__init__.py").is_file():
        return True
    source = Path(os.environ.get("REFERENCE_SOURCE", str(ROOT.parent / "reference"))) / "minivllm"
    if not source.is_dir():
        return False
    REFERENCE_ROOT.mkdir(parents=True, exist_ok=True)
    shutil.copytree(source, REFERENCE_ROOT / "minivllm")
    return True


def run_reference(args) -> dict:
    """The unmodified reference (``baseline/_ref/minivllm``, a copy of its source tree) through its
    own entry point: stock ``LLMEngine`` + ``UniProcExecutor`` + ``Worker`` on CUDA in bfloat16, the
    same shape, batch, prompt length, steps and warm-up."""
    if not ensure_reference_copy():
        return {"impl": "reference", "unavailable": "baseline/_ref/minivllm is missing and there is no "
                                                    "reference source tree to copy it from"}
    import torch
    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device"}
    label, raw, context = SHAPES[args.shape]
    if args.shape != "1.7b":
        return {"impl": "reference", "unavailable": "the reference arm measures the headline shape (1.7b) only"}
    raw = dict(raw, num_hidden_layers=args.layers or raw["num_hidden_layers"])
    context = args.context or context
    scratch = tempfile.mkdtemp(prefix="reference_model_")
    try:
        write_reference_model(raw, Path(scratch))
        sys.path.insert(0, str(REFERENCE_ROOT))
        try:
            from minivllm import (CacheConfig, DeviceConfig, LLMEngine, ModelConfig, SamplingParams,
                                  SchedulerConfig, UniProcExecutor, VllmConfig, Worker)
            pages = args.batch * (-(-context // args.block_size)) + 8
            config = VllmConfig(
                model_config=ModelConfig(model=scratch, dtype="bfloat16", max_model_len=context, hf_config=raw),
                cache_config=CacheConfig(block_size=args.block_size, num_gpu_blocks=pages),
                scheduler_config=SchedulerConfig(max_num_seqs=args.batch, max_num_batched_tokens=args.prompt_len),
                device_config=DeviceConfig(device="cuda"))
            engine = LLMEngine(config, UniProcExecutor(config, Worker(config)))
            warmup = max(args.warmup, 3)
            params = SamplingParams(max_tokens=warmup + args.steps + args.batch + 8, temperature=0.0,
                                    ignore_eos=True)
            for i in range(args.batch):
                engine.add_request(f"ref-{i}", random_prompt(raw["vocab_size"], args.prompt_len, seed=300 + i), params)
            decoding = 0
            prefill_started = time.perf_counter()
            while decoding < args.batch:            # prompts, one per step under the token budget
                decoding = max(decoding, len(engine.step()))
            torch.cuda.synchronize()
            prefill_seconds = time.perf_counter() - prefill_started
            for _ in range(warmup):
                engine.step()
            with ClockSampler() as clocks:
                torch.cuda.synchronize()
                started = time.perf_counter()
                tokens = 0
                for _ in range(args.steps):
                    tokens += len(engine.step())
                torch.cuda.synchronize()
                seconds = time.perf_counter() - started
            engine.shutdown()
        except Exception as error:
            text = " ".join(f"{type(error).__name__}: {error}".split())
            return {"impl": "reference", "unavailable": f"the reference failed on this device: {text[:300]}"}
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    value = tokens / seconds
    return {
        "metric": "decode tokens/s (Qwen3-1.7B shape, bf16, random weights)", "impl": "reference",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(1000.0 * seconds / args.steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": flat_config(label, raw, args, context, "n/a"),
        "e2e": {"value": round(value, 1), "unit": "tokens/s",
                "note": "the reference's entry point is its only path: host ids in, sampled ids out every step"},
        "prefill_all_prompts_s": round(prefill_seconds, 3),
        "clocks": clocks.summary(),
    }


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=("ours", "reference"))
    parser.add_argument("--shape", default="1.7b", choices=tuple(SHAPES))
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--prompt-len", type=int, default=2048)
    parser.add_argument("--context", type=int, default=None, help="default: the shape's own")
    parser.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (named in config)")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--no-points", action="store_true", help="the main point only")
    args = parser.parse_args()

    if args.gpus != 1:
        print("bench.py measures one GPU only: this engine is built for a single B200 (--gpus 1)")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        print(json.dumps(run_reference(args)))
        return 0

    import torch
    if not torch.cuda.is_available():
        print("bench.py needs a CUDA device")
        return 1
    measured, peak_kind = peaks()
    record = {"1.7b": run_small, "8b": run_mixed, "32b": run_large}[args.shape](args, measured, peak_kind)
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
