"""Shared helpers of the tests: model folders made in a temporary folder, token
sequences, and ways of cutting requests into steps."""

from __future__ import annotations

import json
import random
from pathlib import Path

import torch

import plain_qwen3
import tiny_configs


def make_model_folder(tmp_path: Path, raw_config: dict, seed: int = 1, dtype=torch.float32,
                      special=None) -> Path:
    """Write a random model folder.  ``special(weights, raw_config)`` may edit the
    tensors before they are saved (to make one key stand out, for instance)."""
    import vllm_from_scratch_b200 as engine
    folder = tmp_path / f"model_{abs(hash(json.dumps(raw_config, sort_keys=True))) % 10**8}_{seed}"
    entry, typed = engine.load_model_config(raw_config)
    weights = entry.random_weights(typed, seed, dtype=dtype, **tiny_configs.INIT)
    if special is not None:
        special(weights, raw_config)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(typed.to_dict(), indent=2))
    from safetensors.torch import save_file
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    generator = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=generator).tolist()


def plain_logits(folder: Path, tokens: list[int], dtype=torch.float32, round_weights_to=None) -> torch.Tensor:
    raw, weights = plain_qwen3.load_folder(folder)
    if round_weights_to is not None:
        weights = {k: (v.to(round_weights_to) if v.dim() > 1 else v) for k, v in weights.items()}
    return plain_qwen3.qwen3_logits(raw, weights, tokens, dtype)


# ----------------------------------------------------------------------- cuts
# A schedule is a list of steps; a step is a list of (request id, number of
# tokens); "end" lists are derived: a request ends with its last token.

def cut_whole(lengths: dict[str, int]) -> list[list[tuple[str, int]]]:
    return [[(rid, n)] for rid, n in lengths.items()]


def cut_tail_one_by_one(lengths: dict[str, int], tail: int = 32) -> list[list[tuple[str, int]]]:
    steps = []
    for rid, n in lengths.items():
        head = max(1, n - tail)
        steps.append([(rid, head)])
        steps.extend([[(rid, 1)] for _ in range(n - head)])
    return steps


def cut_changing_portions(lengths: dict[str, int], seed: int = 0) -> list[list[tuple[str, int]]]:
    rng = random.Random(seed)
    steps = []
    for rid, n in lengths.items():
        left = n
        sizes = [2, 3, 17, 2, 9, 31, 5, 2, 64, 7]
        index = 0
        while left:
            size = min(left, sizes[index % len(sizes)] if index < 20 else rng.randint(2, 40))
            if left - size == 1:        # never leave a single token to a "portion"
                size = left
            steps.append([(rid, size)])
            left -= size
            index += 1
    return steps


SMALL_PORTIONS = (2, 3, 5, 8, 13, 16, 21, 33)
# With portions of 64 tokens and more a bfloat16 step at head size 128 reaches the tcgen05 kernel
# (at a row offset, behind the single tokens that went to the decode kernel), 300 and more its
# second row block.
LARGE_PORTIONS = (2, 3, 5, 8, 13, 16, 21, 33, 64, 100, 130, 300)


def cut_mixed(lengths: dict[str, int], seed: int = 0, live: int = 4, sizes=SMALL_PORTIONS
              ) -> list[list[tuple[str, int]]]:
    """Up to ``live`` requests at a time; each step takes a portion of some and a
    single token of others, leaves some out, and lets new requests in when one ends."""
    rng = random.Random(seed)
    waiting = list(lengths.items())
    running: dict[str, int] = {}
    steps = []
    while waiting or running:
        while waiting and len(running) < live:
            rid, n = waiting.pop(0)
            running[rid] = n
        step = []
        for rid in list(running):
            left = running[rid]
            choice = rng.random()
            if choice < 0.2 and len(running) > 1:
                continue                                  # left out of this step
            if choice < 0.6:
                size = 1
            else:
                size = rng.choice(sizes)
            size = min(size, left)
            step.append((rid, size))
            running[rid] = left - size
            if running[rid] == 0:
                del running[rid]
        if step:
            steps.append(step)
    return steps


def run_schedule(runner, sequences: dict[str, list[int]], steps, want_all: bool = True, on_device: bool = False,
                 step=None) -> dict[str, torch.Tensor]:
    """Drive a ``ModelRunner`` through ``steps``; returns the logits of every
    position of every request, [length, vocab] on the CPU (``on_device``: where they
    were computed).  ``step``: the function that runs a list of entries (default: the
    runner's step function; a graph cache's ``run`` takes the same list)."""
    step_fn = step or runner.step
    from vllm_from_scratch_b200 import StepEntry
    done = {rid: 0 for rid in sequences}
    rows: dict[str, list[torch.Tensor]] = {rid: [] for rid in sequences}
    for planned in steps:
        entries = []
        for rid, n in planned:
            if not runner.manager.is_admitted(rid):
                runner.manager.admit(rid)
            start = done[rid]
            assert runner.manager.allocate(rid, start + n), f"no pages for {rid} at {start + n}"
            entries.append(StepEntry(rid, sequences[rid][start:start + n], start,
                                     list(range(n)) if want_all else [n - 1]))
        logits = step_fn(entries)
        logits = logits.clone() if on_device else logits.cpu()
        at = 0
        for entry in entries:
            count = len(entry.want)
            rows[entry.request_id].append(logits[at:at + count])
            at += count
            done[entry.request_id] += len(entry.tokens)
            runner.manager.commit(entry.request_id, done[entry.request_id])
            if done[entry.request_id] == len(sequences[entry.request_id]):
                runner.manager.release(entry.request_id)
        runner.manager.check_invariants()
    runner.model.check_token_ids()
    return {rid: torch.cat(parts) for rid, parts in rows.items()}


def schedule_to_trace(sequences: dict[str, list[int]], steps) -> list[dict]:
    """The same schedule as lines for ``bin/trace_run`` (every place wanted)."""
    done = {rid: 0 for rid in sequences}
    lines = []
    for number, step in enumerate(steps):
        entries, ended = [], []
        for rid, n in step:
            entries.append({"id": rid, "tokens": sequences[rid][done[rid]:done[rid] + n],
                            "want": list(range(n))})
            done[rid] += n
            if done[rid] == len(sequences[rid]):
                ended.append(rid)
        lines.append({"step": number, "entries": entries, "end": ended})
    return lines
