"""Time one kernel on synthetic inputs of a given shape.

    python -m vllm_from_scratch_b200.kernels.microbench decode_attention --batch 64 --context 2048
    python -m vllm_from_scratch_b200.kernels.microbench decode_attention --batch 64 --context 2048 --fused
    python -m vllm_from_scratch_b200.kernels.microbench prefill_attention --tokens 2048
    python -m vllm_from_scratch_b200.kernels.microbench gemm --m 8 --n 12288 --k 2048
    python -m vllm_from_scratch_b200.kernels.microbench norm | silu_mul | rope --tokens 2048
    python -m vllm_from_scratch_b200.kernels.microbench layer_products --m 8 [--no-split-norm]
    python -m vllm_from_scratch_b200.kernels.microbench sample --batch 8 --top-k 50 --top-p 0.9 --repeat 10
    python -m vllm_from_scratch_b200.kernels.microbench step --layers 4 --tokens 2048          (a prompt step)
    python -m vllm_from_scratch_b200.kernels.microbench step --layers 4 --batch 8 --context 2048 --tokens 1

CUDA events around ``--iters`` launches after ``--warmup``; between launches a
buffer larger than L2 is written unless ``--keep-l2`` is given.  Prints one JSON
line with the time per launch and the achieved bytes/s or flop/s for the
algorithmic minimum of traffic or work.

``layer_products`` times what lies between two attention kernels of a decode step (output product,
sum and norm, gate and up with the activation, down product, sum and norm, the next layer's q/k/v
product) for ``--m`` token rows at the widths ``--hidden``, ``--heads`` x ``--head-dim``, ``--inter``,
with the norms split over the products around them or (``--no-split-norm``) as kernels of their own;
the time printed is per layer, over several layers' worth of weights, so that every launch reads
cold weights.

``step`` runs whole steps of a model of the Qwen3-1.7B widths (``--hidden``, ``--heads``, ...)
with ``--layers`` layers and random weights through the step function, without graphs: one
prompt of ``--tokens`` tokens, or with ``--tokens 1`` a decode step of ``--batch`` requests at
``--context`` positions.  The last of its steps runs between ``cudaProfilerStart`` and
``cudaProfilerStop``, so that ``ncu --profile-from-start off`` lists that step's launches.
"""

from __future__ import annotations

import argparse
import itertools
import json

import torch

from .. import kernels


def _time(fn, warmup: int, iters: int, flush: bool) -> float:
    """Median milliseconds of ``fn``.  ``fn`` is captured into a CUDA graph first, so
    that the time is the GPU's and not that of the Python calls that launch it."""
    scrub = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device="cuda") if flush else None
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    fn = graph.replay
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        if scrub is not None:
            scrub.fill_(1)
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end))
    times.sort()
    return times[len(times) // 2]


def _paged_case(batch, q_len, context, nq, nkv, d, page, dtype):
    pages_per = -(-context // page)
    total = batch * pages_per
    g = torch.Generator(device="cuda").manual_seed(0)
    table = torch.randperm(total, device="cuda", generator=g).to(torch.int32).view(batch, pages_per)
    kp = torch.randn(total, nkv, page, d, device="cuda", generator=g).to(dtype)
    vp = torch.randn(total, nkv, page, d, device="cuda", generator=g).to(dtype)
    q = torch.randn(batch * q_len, nq * d, device="cuda", generator=g).to(dtype)
    start = torch.tensor([0] + list(itertools.accumulate([q_len] * batch)), dtype=torch.int32, device="cuda")
    seq = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    return q, kp, vp, start, seq, table


def _step(args) -> int:
    """Whole steps of a small-in-depth model through the step function (see the module's text)."""
    import time

    from ..config.registry import load_model_config
    from ..engine.runner import ModelRunner
    from ..engine.step import StepEntry
    raw = {
        "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": args.layers,
        "hidden_size": args.hidden, "num_attention_heads": args.heads, "num_key_value_heads": args.kv_heads,
        "head_dim": args.head_dim, "intermediate_size": args.inter, "vocab_size": args.vocab,
        "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
        "max_position_embeddings": 40960, "hidden_act": "silu", "attention_bias": False, "initializer_range": 0.02,
    }
    entry, config = load_model_config(raw)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    weights = entry.random_weights(config, seed=0, dtype=dtype, device="cuda")
    decode = args.tokens == 1
    requests = args.batch if decode else 1
    positions = (args.context + 8) if decode else args.tokens
    runner = ModelRunner(entry.build_spec(config), weights, args.dtype, args.page,
                         requests * (-(-positions // args.page)) + 4, requests, device="cuda", model_config=config)
    del weights
    generator = torch.Generator().manual_seed(0)
    ids = [f"r{i}" for i in range(requests)]
    for request_id in ids:
        runner.manager.admit(request_id)
    steps = 3
    milliseconds = 0.0
    for number in range(steps):
        entries = []
        for request_id in ids:
            if decode:
                start = args.context + number
                tokens = torch.randint(0, args.vocab, (1,), generator=generator).tolist()
            else:
                start = 0
                tokens = torch.randint(0, args.vocab, (args.tokens,), generator=generator).tolist()
            assert runner.manager.allocate(request_id, start + len(tokens))
            entries.append(StepEntry(request_id, tokens, start, [len(tokens) - 1]))
        last = number == steps - 1
        torch.cuda.synchronize()
        if last:
            torch.cuda.profiler.start()
        started = time.perf_counter()
        runner.step(entries)
        torch.cuda.synchronize()
        milliseconds = 1000 * (time.perf_counter() - started)
        if last:
            torch.cuda.profiler.stop()
    print(json.dumps({"op": "step", "dtype": args.dtype, "layers": args.layers, "requests": requests,
                      "tokens_per_request": 1 if decode else args.tokens,
                      "context": args.context if decode else args.tokens,
                      "host_ms_of_the_last_step_without_graphs": round(milliseconds, 3)}))
    return 0


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("op", choices=("decode_attention", "prefill_attention", "gemm", "norm", "silu_mul", "rope",
                                       "layer_products", "sample", "step"))
    parser.add_argument("--temperature", type=float, default=0.8, help="sample: 0 for greedy rows")
    parser.add_argument("--top-k", type=int, default=0, help="sample")
    parser.add_argument("--top-p", type=float, default=1.0, help="sample")
    parser.add_argument("--min-p", type=float, default=0.0, help="sample")
    parser.add_argument("--spread", type=float, default=1.0, help="sample: standard deviation of the random logits")
    parser.add_argument("--logprobs", type=int, default=None,
                        help="sample: time the kernel for log-probabilities instead, with lists of this many tokens")
    parser.add_argument("--no-split-norm", action="store_true",
                        help="layer_products: the two norms as kernels of their own")
    parser.add_argument("--layers", type=int, default=4, help="step: layers of the model")
    parser.add_argument("--vocab", type=int, default=151936, help="step: rows of the embedding")
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--page", type=int, default=16)
    parser.add_argument("--hidden", type=int, default=2048)
    parser.add_argument("--inter", type=int, default=6144)
    parser.add_argument("--m", type=int, default=8)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=2048)
    parser.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    parser.add_argument("--planned-context", type=int, default=None,
                        help="context length the decode launch is planned for (default: --context)")
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--iters", type=int, default=10)
    parser.add_argument("--keep-l2", action="store_true")
    parser.add_argument("--repeat", type=int, default=1,
                        help="attention: launches per timed graph replay (the time printed is per launch); "
                             "short kernels need several, CUDA events resolve no better than some microseconds")
    parser.add_argument("--gated", action="store_true", help="gemm: fused silu(gate) * up, N = 2 * inter")
    parser.add_argument("--fused", action="store_true",
                        help="decode_attention: the kernel that takes the packed projection and also normalises "
                             "and rotates the heads and stores the new key and value")
    parser.add_argument("--past", type=int, default=0,
                        help="prefill_attention: positions the request has in the cache ahead of its --tokens")
    parser.add_argument("--no-key-split", action="store_true",
                        help="prefill_attention: never divide a row block's keys over several blocks")
    parser.add_argument("--no-tensor-memory", action="store_true",
                        help="prefill_attention: the mma.sync kernel instead of the tcgen05 one")
    parser.add_argument("--no-tma-decode", action="store_true",
                        help="decode_attention: the kernel with per-thread copies instead of tensor copies")
    parser.add_argument("--kernel", default="default", choices=("default", "library"),
                        help="gemm: the engine's choice or the vendor library")
    args = parser.parse_args(argv)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    size = 2 if dtype == torch.bfloat16 else 4
    nq, nkv, d = args.heads, args.kv_heads, args.head_dim
    record: dict = {"op": args.op, "dtype": args.dtype}

    if args.op == "step":
        return _step(args)
    if args.op in ("decode_attention", "prefill_attention"):
        from . import attention_bf16
        attention_bf16.USE_TC_KEY_SPLIT = not args.no_key_split
        attention_bf16.USE_TC_ATTENTION = not args.no_tensor_memory
        attention_bf16.USE_TMA_DECODE = not args.no_tma_decode
        decode = args.op == "decode_attention"
        batch = args.batch if decode else 1
        q_len = 1 if decode else args.tokens
        context = args.context if decode else args.tokens + args.past
        q, kp, vp, start, seq, table = _paged_case(batch, q_len, context, nq, nkv, d, args.page, dtype)
        out = torch.empty_like(q)
        planned = args.planned_context or context
        one = lambda: kernels.paged_attention(q, kp, vp, out, start, seq, table, nq, nkv, d, args.page,
                                              d ** -0.5, None, q_len, planned)
        if decode and args.fused:
            qkv = torch.randn(batch, (nq + 2 * nkv) * d, device="cuda").to(dtype)
            positions = (seq - 1).to(torch.int32)
            last_page = table[torch.arange(batch, device="cuda"), ((seq - 1) // args.page).long()]
            slots = (last_page * args.page + (seq - 1) % args.page).to(torch.int32)
            weight = torch.ones(d, device="cuda")
            inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()

            def one():
                if not kernels.fused_decode_attention(qkv, positions, slots, weight, weight, inv_freq, d, 1e-6, kp, vp,
                                                      out, seq, table, nq, nkv, d, args.page, d ** -0.5, None, planned):
                    raise SystemExit("no fused kernel for this shape")
            record["fused"] = True

        def fn():
            for _ in range(args.repeat):
                one()
        ms = _time(fn, args.warmup, args.iters, not args.keep_l2) / args.repeat
        record.update(batch=batch, context=context, heads=nq, kv_heads=nkv, head_dim=d, page=args.page)
        if decode:
            moved = batch * context * nkv * d * 2 * size
            record.update(bytes=moved, gb_s=round(moved / ms / 1e6, 1))
        else:
            flops = 2 * 2 * nq * d * q_len * (args.past + q_len / 2)
            record.update(flops=flops, tflop_s=round(flops / ms / 1e9, 1))
    elif args.op == "gemm":
        x = torch.randn(args.m, args.k, device="cuda").to(dtype)
        # Enough copies of the weight to exceed L2 several times over: launched back to
        # back, each launch reads cold weights and the launch gaps are amortised.
        copies = max(1, min(64, (512 * 1024 * 1024) // (args.n * args.k * size)))
        ws = [torch.randn(args.n, args.k, device="cuda").to(dtype) for _ in range(copies)]
        out = torch.empty(args.m, args.n // 2 if args.gated else args.n, device="cuda", dtype=dtype)
        if args.kernel == "library":
            one = lambda w: torch.mm(x, w.t(), out=out)
        elif args.gated:
            one = lambda w: kernels.gated_silu_gemm(x, w, out)
        else:
            one = lambda w: kernels.gemm(x, w, out)

        def sweep():
            for w in ws:
                one(w)
        ms = _time(sweep, args.warmup, args.iters, False) / copies
        moved = (args.n * args.k + args.m * args.k + args.m * args.n) * size
        flops = 2 * args.m * args.n * args.k
        record.update(m=args.m, n=args.n, k=args.k, gb_s=round(moved / ms / 1e6, 1),
                      tflop_s=round(flops / ms / 1e9, 2))
    elif args.op == "layer_products":
        m, hidden, inter = args.m, args.hidden, args.inter
        attended, qkv_width = nq * d, (nq + 2 * nkv) * d
        layer_bytes = (hidden * attended + 3 * inter * hidden + qkv_width * hidden) * 2
        copies = max(2, min(16, (768 * 1024 * 1024) // layer_bytes))
        rand = lambda *shape: (torch.randn(*shape, device="cuda") * shape[-1] ** -0.5).bfloat16()
        layers = [(rand(hidden, attended), rand(2 * inter, hidden), rand(hidden, inter), rand(qkv_width, hidden))
                  for _ in range(copies)]
        gain = torch.ones(hidden, device="cuda")
        x = torch.randn(m, attended, device="cuda").bfloat16()
        res = torch.randn(m, hidden, device="cuda")
        bf = lambda width: torch.empty(m, width, device="cuda", dtype=torch.bfloat16)
        out, normed, act, down, qkv = bf(hidden), bf(hidden), bf(inter), bf(hidden), bf(qkv_width)
        squares = [torch.empty(m, hidden // 8, device="cuda") for _ in range(2)]

        def sweep():
            for w_out, w_gate_up, w_down, w_qkv in layers:
                if args.no_split_norm:
                    kernels.gemm(x, w_out, out)
                    kernels.add_rmsnorm(out, res, gain, 1e-6, normed)
                    kernels.gated_silu_gemm(normed, w_gate_up, act)
                    kernels.gemm(act, w_down, down)
                    kernels.add_rmsnorm(down, res, gain, 1e-6, normed)
                    kernels.gemm(normed, w_qkv, qkv)
                    continue
                # a norm is split only where the engine would split it: both products around it its own kernels'
                first = kernels.split_norm_ok(m, w_out, True) and kernels.split_norm_ok(m, w_gate_up, False, True)
                second = kernels.split_norm_ok(m, w_down, True) and kernels.split_norm_ok(m, w_qkv, False)
                if first:
                    kernels.gemm(x, w_out, out, fold=(res, gain, squares[0]))
                    kernels.gated_silu_gemm(out, w_gate_up, act, scale=(squares[0], 1e-6))
                else:
                    kernels.gemm(x, w_out, out)
                    kernels.add_rmsnorm(out, res, gain, 1e-6, normed)
                    kernels.gated_silu_gemm(normed, w_gate_up, act)
                if second:
                    kernels.gemm(act, w_down, down, fold=(res, gain, squares[1]))
                    kernels.gemm(down, w_qkv, qkv, scale=(squares[1], 1e-6))
                else:
                    kernels.gemm(act, w_down, down)
                    kernels.add_rmsnorm(down, res, gain, 1e-6, normed)
                    kernels.gemm(normed, w_qkv, qkv)
        ms = _time(sweep, args.warmup, args.iters, False) / copies
        record.update(m=m, hidden=hidden, inter=inter, attended=attended, qkv=qkv_width,
                      split_norm=not args.no_split_norm, gb_s=round(layer_bytes / ms / 1e6, 1))
    elif args.op == "sample":
        rows = args.batch
        logits = torch.randn(rows, args.vocab, device="cuda") * args.spread
        full = lambda value, kind: torch.full((rows,), value, dtype=kind, device="cuda")
        temperature, top_k = full(args.temperature, torch.float32), full(args.top_k, torch.int32)
        top_p, min_p = full(args.top_p, torch.float32), full(args.min_p, torch.float32)
        seeds, draws = torch.arange(rows, dtype=torch.int64, device="cuda"), full(3, torch.int64)
        picked = torch.empty(rows, dtype=torch.int32, device="cuda")
        filtered = args.temperature >= 1e-5 and (args.top_k > 0 or args.top_p < 1.0 or args.min_p > 0.0)

        def launches():
            for _ in range(args.repeat):
                kernels.sample(logits, temperature, top_k, top_p, min_p, seeds, draws, picked, 1e-5, 2 if filtered else 1)
        if args.logprobs is not None:
            launches()
            width = args.logprobs + 1
            ids = torch.empty(rows, width, dtype=torch.int32, device="cuda")
            values = torch.empty(rows, width, device="cuda")
            places = torch.empty(rows, dtype=torch.int32, device="cuda")
            wanted = full(args.logprobs, torch.int32)

            def launches():
                for _ in range(args.repeat):
                    kernels.logprobs(logits, picked, wanted, ids, values, places)
            record.update(logprobs=args.logprobs)
        ms = _time(launches, args.warmup, args.iters, not args.keep_l2) / args.repeat
        record.update(rows=rows, vocab=args.vocab, temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
                      min_p=args.min_p, repeat=args.repeat, gb_s=round(rows * args.vocab * 4 / ms / 1e6, 1))
    elif args.op == "norm":
        x = torch.randn(args.tokens, args.hidden, device="cuda").to(dtype)
        residual = torch.randn(args.tokens, args.hidden, device="cuda")
        weight = torch.ones(args.hidden, device="cuda")
        out = torch.empty_like(x)
        ms = _time(lambda: kernels.add_rmsnorm(x, residual, weight, 1e-6, out), args.warmup, args.iters,
                   not args.keep_l2)
        moved = args.tokens * args.hidden * (2 * size + 8)
        record.update(tokens=args.tokens, hidden=args.hidden, gb_s=round(moved / ms / 1e6, 1))
    elif args.op == "silu_mul":
        gate_up = torch.randn(args.tokens, 2 * args.inter, device="cuda").to(dtype)
        out = torch.empty(args.tokens, args.inter, device="cuda", dtype=dtype)
        ms = _time(lambda: kernels.silu_mul(gate_up, out), args.warmup, args.iters, not args.keep_l2)
        moved = args.tokens * args.inter * 3 * size
        record.update(tokens=args.tokens, inter=args.inter, gb_s=round(moved / ms / 1e6, 1))
    else:
        tokens = args.tokens
        qkv = torch.randn(tokens, (nq + 2 * nkv) * d, device="cuda").to(dtype)
        positions = torch.arange(tokens, dtype=torch.int32, device="cuda")
        slots = torch.arange(tokens, dtype=torch.int32, device="cuda")
        pages = -(-tokens // args.page)
        kp = torch.zeros(pages, nkv, args.page, d, device="cuda", dtype=dtype)
        vp = torch.zeros_like(kp)
        q_out = torch.empty(tokens, nq * d, device="cuda", dtype=dtype)
        weight = torch.ones(d, device="cuda")
        inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
        ms = _time(lambda: kernels.head_norm_rope_cache(qkv, positions, slots, weight, weight, inv_freq, d,
                                                        1e-6, q_out, kp, vp, nq, nkv, d, args.page),
                   args.warmup, args.iters, not args.keep_l2)
        moved = tokens * (nq + 2 * nkv) * d * 2 * size
        record.update(tokens=tokens, gb_s=round(moved / ms / 1e6, 1))
    record["us"] = round(ms * 1000, 2)
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
