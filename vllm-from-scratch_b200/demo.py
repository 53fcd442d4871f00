"""Command line: a model folder (or a random-weights shape) to generated tokens.

    python -m vllm_from_scratch_b200.demo --model-dir DIR "1 2 3 4" "9 8 7"

Option names, defaults and meanings follow the reference's demo
(minivllm/demo.py:95-158) where it has them: ``--model-dir``, ``--max-new-tokens``,
``--max-model-len``, ``--max-num-seqs``, ``--max-num-batched-tokens``,
``--enforce-eager``, ``--block-size``, ``--num-kv-blocks``, ``--no-prefix-caching``,
``--dtype``, ``--device``, ``--temperature``, ``--top-k``, ``--top-p``, ``--min-p``,
the three penalties, ``--min-tokens``, ``--seed``, ``--ignore-eos``, ``--trace``,
``--scheduler-trace``.  The reference tokenizes questions with the model's chat
template; here a prompt is a list of token ids ("1 2 3"), or text when the model
folder has a tokenizer and ``--text`` is given.  ``--random-weights CONFIG.json``
writes a random model folder first (the reference has that only among its test
helpers).  Options of features that are out of scope (logprobs, structured
output, speculative decoding) do not exist.
"""

from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time
from pathlib import Path

DEFAULT_PROMPTS = ["1 2 3 4 5 6 7 8", "11 12 13"]


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="Generate with the B200 Qwen3 engine")
    parser.add_argument("questions", nargs="*", default=None,
                        help="prompts: token ids separated by spaces or commas (text with --text)")
    parser.add_argument("--model-dir", default="models/Qwen3-1.7B",
                        help="folder with config.json and safetensors")
    parser.add_argument("--max-new-tokens", type=int, default=24)
    parser.add_argument("--max-model-len", type=int, default=512)
    parser.add_argument("--max-num-seqs", type=int, default=2)
    parser.add_argument("--max-num-batched-tokens", type=int, default=64)
    parser.add_argument("--enforce-eager", action="store_true", help="no CUDA-graph replay of decode steps")
    parser.add_argument("--no-async-scheduling", action="store_true",
                        help="wait for a step's tokens before the next step is queued (the reference's only "
                             "mode; by default the next decode step is queued ahead)")
    parser.add_argument("--block-size", type=int, default=16)
    parser.add_argument("--num-kv-blocks", type=int, default=64)
    parser.add_argument("--no-prefix-caching", action="store_true")
    parser.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    parser.add_argument("--device", choices=("auto", "cuda"), default="auto",
                        help="the engine runs on a CUDA device only")
    parser.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    parser.add_argument("--top-k", type=int, default=-1)
    parser.add_argument("--top-p", type=float, default=1.0)
    parser.add_argument("--min-p", type=float, default=0.0)
    parser.add_argument("--repetition-penalty", type=float, default=1.0)
    parser.add_argument("--presence-penalty", type=float, default=0.0)
    parser.add_argument("--frequency-penalty", type=float, default=0.0)
    parser.add_argument("--min-tokens", type=int, default=0)
    parser.add_argument("--logprobs", type=int, default=None,
                        help="report every generated token's log-probability and this many most likely tokens")
    parser.add_argument("--seed", type=int, default=None)
    parser.add_argument("--ignore-eos", action="store_true")
    parser.add_argument("--trace", action="store_true", help="print what the first step fed to the model")
    parser.add_argument("--scheduler-trace", action="store_true", help="print the scheduler's decisions")
    parser.add_argument("--text", action="store_true", help="prompts are text for the folder's tokenizer")
    parser.add_argument("--random-weights", metavar="CONFIG_JSON", default=None,
                        help="write a random model for this config.json into a temporary folder and use it")
    parser.add_argument("--random-seed", type=int, default=0)
    return parser


def parse_prompt(text: str) -> list[int]:
    try:
        return [int(piece) for piece in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"prompt {text!r} is not a list of token ids (use --text for text)") from None


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    import vllm_from_scratch_b200 as engine

    scratch = None
    model_dir = Path(args.model_dir)
    if args.random_weights:
        scratch = tempfile.TemporaryDirectory()
        raw = json.loads(Path(args.random_weights).read_text())
        model_dir = engine.write_random_model(
            raw, args.random_seed, Path(scratch.name) / "model",
            dtype=torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    if not model_dir.is_dir():
        raise SystemExit(f"model folder {model_dir} does not exist (nothing is downloaded)")
    raw_config = json.loads((model_dir / "config.json").read_text())

    tokenizer = None
    questions = args.questions or DEFAULT_PROMPTS
    if args.text:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(model_dir, local_files_only=True)
        prompts = [tokenizer.encode(question) for question in questions]
    else:
        prompts = [parse_prompt(question) for question in questions]

    started = time.perf_counter()
    llm = engine.LLMEngine(engine.EngineConfig(
        engine.ModelConfig(str(model_dir), args.dtype, args.max_model_len, args.enforce_eager),
        engine.CacheConfig(args.block_size, args.num_kv_blocks, not args.no_prefix_caching),
        engine.SchedulerConfig(args.max_num_seqs, args.max_num_batched_tokens,
                               async_scheduling=not args.no_async_scheduling), "cuda"))
    load_seconds = time.perf_counter() - started
    runner = llm.runner
    config = runner.model_config
    print(f"model: {model_dir} ({config.architecture})")
    print(f"  {config.num_hidden_layers} layers, hidden={config.hidden_size}, "
          f"q/kv heads={config.num_attention_heads}/{config.num_key_value_heads}, head_dim={config.head_dim}")
    print(f"  run dtype {args.dtype}, {config.num_parameters() / 1e9:.3f} G parameters, "
          f"tied embedding={config.tie_word_embeddings}")
    print(f"  cache: {len(runner.storage.groups)} group(s) x {args.num_kv_blocks} pages x {args.block_size} "
          f"positions = {runner.storage.num_bytes() / 1e6:.1f} MB; loaded in {load_seconds:.2f} s")
    print(f"  prefix caching: {'on' if runner.manager.prefix_caching else 'off'}")

    for index, prompt in enumerate(prompts):
        llm.add_request(f"q{index}", prompt, engine.SamplingParams(
            max_tokens=args.max_new_tokens, temperature=args.temperature, top_k=args.top_k,
            top_p=args.top_p, min_p=args.min_p, seed=args.seed, min_tokens=args.min_tokens,
            ignore_eos=args.ignore_eos, repetition_penalty=args.repetition_penalty,
            presence_penalty=args.presence_penalty, frequency_penalty=args.frequency_penalty,
            logprobs=args.logprobs,
            eos_token_id=raw_config.get("eos_token_id") if not isinstance(raw_config.get("eos_token_id"), list)
            else raw_config["eos_token_id"][0]))
        print(f"\nprompt q{index}: {len(prompt)} tokens")

    start = time.perf_counter()
    steps = 0
    latest = {}
    while llm.has_unfinished_requests():
        for output in llm.step():
            latest[output.request_id] = output
        steps += 1
    torch.cuda.synchronize()
    seconds = time.perf_counter() - start

    if args.trace and llm.first_step_inputs:
        first = llm.first_step_inputs
        print(f"\nfirst step (num_scheduled_tokens={first['num_scheduled_tokens']}):")
        print(f"  positions       = {first['positions']}")
        print(f"  query_start     = {first['query_start']}   seq_lens={first['seq_lens']}")
        for group in first["slot_mapping"]:
            print(f"  group {group}: slot_mapping = {first['slot_mapping'][group]}")
            print(f"  group {group}: block_table  = {first['block_table'][group]}")

    generated = 0
    for index in range(len(prompts)):
        output = latest.get(f"q{index}")
        if output is None:
            continue
        generated += len(output.token_ids)
        shown = tokenizer.decode(output.token_ids, skip_special_tokens=True) if tokenizer else output.token_ids
        print(f"\nanswer[q{index}]: {shown}")
        print(f"   finish reason {output.finish_reason.name if output.finish_reason else None}")
        if output.logprobs is not None:
            print(f"   cumulative logprob {output.cumulative_logprob:.4f}")
            for token, entry in zip(output.token_ids, output.logprobs):
                others = ", ".join(f"{t}: {v.logprob:.3f}" for t, v in sorted(entry.items(), key=lambda kv: kv[1].rank)
                                   if t != token)
                print(f"   {token}: {entry[token].logprob:.3f} (rank {entry[token].rank})" + (f"   [{others}]" if others else ""))
    stats = runner.manager.stats()
    print(f"\n{steps} steps, {generated} tokens, {seconds:.2f} s ({generated / max(seconds, 1e-9):.1f} tok/s)")
    print(f"cache at the end: {stats}; preemptions {llm.scheduler.num_preemptions}")
    if args.scheduler_trace:
        print()
        print(llm.scheduler.format_trace())
    llm.shutdown()
    if scratch is not None:
        scratch.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
