"""Python face of the hand-written sm_100a kernels.

Each function checks its tensors (device, dtype, contiguity, shapes), then calls
one ``extern "C"`` launcher on torch's current CUDA stream.  Nothing here has a
CPU or library alternative: a tensor that is not on a CUDA device, or a kernel
library that cannot be built, raises.  (The bfloat16 matrix product may go to
the vendor's library, as the reference's does through ``F.linear``,
minivllm/layers/quantization/methods.py:36-37.)
"""

from __future__ import annotations

import ctypes
import os
from typing import Sequence

import torch

from ..csrc.build import is_loaded, load_library

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels are built for float32 and bfloat16, not {dtype}") from None


# Full validation of every operand costs a few microseconds per launch.  The engine's
# own step function switches it off (``validation(False)``) once a batch shape has run
# with it on; everything else (tests, parts written by users, direct calls) keeps it.
# The environment variable B200_VALIDATE=1 keeps it on everywhere.
_validate = True


class validation:
    """Context manager: ``with validation(False): ...`` skips operand checks inside."""

    def __init__(self, enabled: bool) -> None:
        self.enabled = enabled or os.environ.get("B200_VALIDATE") == "1"

    def __enter__(self):
        global _validate
        self.previous, _validate = _validate, self.enabled
        return self

    def __exit__(self, *exc):
        global _validate
        _validate = self.previous


def _check(name: str, tensor: torch.Tensor | None, dtype: torch.dtype | Sequence[torch.dtype] | None = None,
           shape: Sequence[int | None] | None = None, optional: bool = False) -> int:
    """Validate one operand and return its device address (0 for an absent optional)."""
    if tensor is None:
        if optional:
            return 0
        raise KernelError(f"{name}: tensor is required")
    if not _validate:
        return tensor.data_ptr()
    if not tensor.is_cuda:
        raise KernelError(
            f"{name}: tensor lives on {tensor.device}; the engine's kernels run on a CUDA device only")
    if not tensor.is_contiguous():
        raise KernelError(f"{name}: tensor must be contiguous, strides {tensor.stride()}")
    if dtype is not None:
        allowed = (dtype,) if isinstance(dtype, torch.dtype) else tuple(dtype)
        if tensor.dtype not in allowed:
            raise KernelError(f"{name}: dtype {tensor.dtype}, expected {allowed}")
    if shape is not None:
        if tensor.dim() != len(shape) or any(s is not None and s != t for s, t in zip(shape, tensor.shape)):
            raise KernelError(f"{name}: shape {tuple(tensor.shape)}, expected {tuple(shape)}")
    return tensor.data_ptr()


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


launch_count = 0        # kernel launchers called so far (the benchmark reports the difference)


def count_launch(count: int = 1) -> None:
    global launch_count
    launch_count += count


def _run(library: str, symbol: str, *args) -> None:
    count_launch()
    lib = load_library(library)
    status = getattr(lib, symbol)(*args)
    if status != 0:
        raise KernelError(lib.b200_last_error().decode())


def device_error() -> str | None:
    """What a kernel whose bounded wait ran out has left behind, or ``None``.  Such a
    kernel stops issuing work and returns, so its results are wrong: callers check this
    between steps.  Reads a few bytes from the device (synchronises); the flags are
    cleared by reading."""
    found = []
    if is_loaded("attention_bf16"):
        code = int(load_library("attention_bf16").b200_attention_error())
        if code:
            found.append(f"attention kernel gave up waiting (code {code})")
    if is_loaded("gemm_bf16"):
        code = int(load_library("gemm_bf16").b200_stream_gemm_error())
        if code:
            found.append(f"matrix-product kernel gave up waiting (code {code})")
    return "; ".join(found) or None


STATUS_WORDS = 3        # token-id flag, attention kernels' error word, matrix-product kernels' error word
_status_addresses: dict[int, tuple[int, int]] = {}


def collect_status(token_flag: torch.Tensor | None, out: torch.Tensor) -> None:
    """Write the step's error words into ``out`` (int32 ``[STATUS_WORDS]`` on the device) without
    waiting for anything: ``token_flag`` (the embedding kernel's word for a token id outside the
    vocabulary) and the words that kernels with bounded waits set when they give up.  A caller
    copies ``out`` to the host with results it waits for anyway and hands the values to
    :func:`status_problem`.  Words of libraries that are not loaded read as 0."""
    device = out.device.index if out.device.index is not None else torch.cuda.current_device()
    attention = is_loaded("attention_bf16")
    product = is_loaded("gemm_bf16")
    cached = _status_addresses.get(device)
    if cached is None or (attention and not cached[0]) or (product and not cached[1]):
        a = b = 0
        if attention:
            fn = load_library("attention_bf16").b200_attention_error_address
            fn.restype = ctypes.c_void_p
            a = fn() or 0
        if product:
            fn = load_library("gemm_bf16").b200_stream_gemm_error_address
            fn.restype = ctypes.c_void_p
            b = fn() or 0
        cached = _status_addresses[device] = (a, b)
    _run("sampling", "b200_collect_status",
         ctypes.c_void_p(token_flag.data_ptr() if token_flag is not None else 0), ctypes.c_void_p(cached[0]),
         ctypes.c_void_p(cached[1]), ctypes.c_void_p(_check("status words", out, torch.int32, (STATUS_WORDS,))),
         _stream())


def status_problem(words: Sequence[int], vocab_size: int | None = None) -> str | None:
    """What the words written by :func:`collect_status` say, or None if all is well."""
    found = []
    if words[0]:
        found.append(f"token id outside the vocabulary{'' if vocab_size is None else f' [0, {vocab_size})'} "
                     f"at batch row {words[0] - 1}")
    if words[1]:
        found.append(f"attention kernel gave up waiting (code {words[1]})")
    if words[2]:
        found.append(f"matrix-product kernel gave up waiting (code {words[2]})")
    return "; ".join(found) or None


_P = ctypes.c_void_p
_I = ctypes.c_int
_F = ctypes.c_float


# ------------------------------------------------------------------ elementwise
def embedding(table: torch.Tensor, ids: torch.Tensor, residual: torch.Tensor,
              error_flag: torch.Tensor) -> None:
    """``residual[t] = float32(table[ids[t]])``; an id outside the table sets
    ``error_flag`` to 1 + the token's row and writes zeros."""
    vocab, hidden = table.shape
    tokens = ids.shape[0]
    _run("norm", "b200_embedding",
         _P(_check("embedding table", table, (torch.float32, torch.bfloat16))),
         _P(_check("token ids", ids, torch.int32, (tokens,))),
         _P(_check("residual", residual, torch.float32, (tokens, hidden))),
         _I(tokens), _I(hidden), _I(vocab),
         _P(_check("error flag", error_flag, torch.int32)), _I(_code(table.dtype)), _stream())


def add_rmsnorm(x: torch.Tensor | None, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None) -> None:
    """``residual += x`` in float32 (skipped when ``x`` is None), then
    ``out = residual * rsqrt(mean(residual^2) + eps) * weight`` in ``out``'s dtype.
    With ``rows`` only those rows are normalised, written compactly to ``out``,
    and ``residual`` is left as it was."""
    tokens, hidden = residual.shape
    out_rows = tokens if rows is None else rows.shape[0]
    _run("norm", "b200_add_rmsnorm",
         _P(_check("norm input", x, out.dtype, (tokens, hidden), optional=True)),
         _P(_check("residual", residual, torch.float32)),
         _P(_check("norm weight", weight, torch.float32, (hidden,))),
         _P(_check("norm output", out, (torch.float32, torch.bfloat16), (out_rows, hidden))),
         _P(_check("row index", rows, torch.int32, optional=True)),
         _I(out_rows), _I(hidden), _F(eps), _I(_code(out.dtype)), _stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]`` computed in float32."""
    tokens, inter = out.shape
    _run("norm", "b200_silu_mul",
         _P(_check("gate_up", gate_up, out.dtype, (tokens, 2 * inter))),
         _P(_check("activation output", out, (torch.float32, torch.bfloat16))),
         _I(tokens), _I(inter), _I(_code(out.dtype)), _stream())


# --------------------------------------------------------------- matrix product
def split_norm_ok(tokens: int, w: torch.Tensor, fold: bool, gated: bool = False) -> bool:
    """Whether the product of ``tokens`` rows with ``w`` can carry half of an RMSNorm: scale its
    result by the root of :class:`~..parts.base.HalfNormedRows`, or, with ``fold``, add its result
    into the residual and write such rows (``gemm`` with ``scale`` / ``fold``).  True for the few
    rows and the bfloat16 matrices that the resident-rows kernel takes."""
    if w.dtype != torch.bfloat16 or not w.is_cuda:
        return False
    from . import gemm_bf16
    return gemm_bf16.split_norm_ok(tokens, w, fold, gated)


def gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor,
         scale: tuple[torch.Tensor, float] | None = None,
         fold: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None) -> None:
    """``out[M, N] = x[M, K] @ w[N, K]^T``.  float32 operands: the engine's own
    fused-multiply-add kernel (no tensor-core mode).  bfloat16 operands: float32
    accumulation on the tensor cores; ``out`` may be bfloat16 or float32.

    The halves of a split RMSNorm, where :func:`split_norm_ok` says so: ``scale = (squares, eps)``
    multiplies row ``m`` of the result by ``rsqrt(squares[m].sum() / K + eps)``; ``fold = (residual,
    weight, squares_out)`` adds the rounded result into the float32 ``residual`` ``[M, N]`` in place,
    writes ``residual * weight`` to ``out`` instead, and the sums of the new residual's squares over
    blocks of eight columns to ``squares_out`` ``[M, N / 8]``."""
    m, k = x.shape
    n = w.shape[0]
    if scale is not None or fold is not None:
        _check("gemm input", x, torch.bfloat16)
        _check("gemm weight", w, torch.bfloat16, (n, k))
        _check("gemm output", out, torch.bfloat16, (m, n))
        from . import gemm_bf16
        gemm_bf16.split_norm_gemm(x, w, out, 0, scale, fold)
        return
    if x.dtype == torch.float32:
        _run("gemm_f32", "b200_gemm_f32",
             _P(_check("gemm input", x, torch.float32)), _P(_check("gemm weight", w, torch.float32, (n, k))),
             _P(_check("gemm output", out, torch.float32, (m, n))), _I(m), _I(n), _I(k), _stream())
        return
    _check("gemm input", x, torch.bfloat16)
    _check("gemm weight", w, torch.bfloat16, (n, k))
    _check("gemm output", out, (torch.bfloat16, torch.float32), (m, n))
    from . import gemm_bf16
    gemm_bf16.gemm_bf16(x, w, out)


def gated_silu_gemm(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor,
                    scale: tuple[torch.Tensor, float] | None = None) -> None:
    """``out[M, I] = silu(x @ w[:I]^T) * (x @ w[I:]^T)`` for ``w_gate_up`` of shape
    ``[2 I, K]`` (gate rows first).  One fused kernel where the shape allows it,
    otherwise the product followed by the activation kernel.  ``scale``: as for :func:`gemm`
    (both products are scaled before the activation)."""
    m, k = x.shape
    inter = out.shape[1]
    _check("gated input", x, (torch.float32, torch.bfloat16))
    _check("gate_up weight", w_gate_up, x.dtype, (2 * inter, k))
    _check("gated output", out, x.dtype, (m, inter))
    if scale is not None:
        from . import gemm_bf16
        gemm_bf16.split_norm_gemm(x, w_gate_up, out, inter, scale, None)
        return
    if x.dtype == torch.bfloat16:
        from . import gemm_bf16
        if gemm_bf16.gated_silu_gemm_bf16(x, w_gate_up, out):
            return
    gate_up = torch.empty((m, 2 * inter), dtype=x.dtype, device=x.device)
    gemm(x, w_gate_up, gate_up)
    silu_mul(gate_up, out)


# -------------------------------------------------------------------- attention
def head_norm_rope_cache(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                         q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                         inv_freq: torch.Tensor | None, rotary_dim: int, eps: float,
                         q_out: torch.Tensor, k_pages: torch.Tensor | None,
                         v_pages: torch.Tensor | None, num_q_heads: int, num_kv_heads: int,
                         head_dim: int, page_size: int) -> None:
    """From the packed projection ``[T, (nq + 2 nkv) d]``: per-head RMSNorm of
    queries and keys, rotate-half position encoding, queries to ``q_out``, keys
    and values to their pages at ``slots`` (negative slot: not stored; pages None:
    nothing stored)."""
    tokens = qkv.shape[0]
    dtype = qkv.dtype
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    page_shape = (None, num_kv_heads, page_size, head_dim)
    _run("rope_cache", "b200_head_norm_rope_cache",
         _P(_check("qkv", qkv, (torch.float32, torch.bfloat16), (tokens, width))),
         _P(_check("positions", positions, torch.int32, (tokens,))),
         _P(_check("slot mapping", slots, torch.int32, (tokens,))),
         _P(_check("q head-norm weight", q_weight, torch.float32, (head_dim,), optional=True)),
         _P(_check("k head-norm weight", k_weight, torch.float32, (head_dim,), optional=True)),
         _P(_check("inverse frequencies", inv_freq, torch.float32, (rotary_dim // 2,), optional=True)),
         _P(_check("q output", q_out, dtype, (tokens, num_q_heads * head_dim))),
         _P(_check("key pages", k_pages, dtype, page_shape, optional=True)),
         _P(_check("value pages", v_pages, dtype, page_shape, optional=True)),
         _I(tokens), _I(num_q_heads), _I(num_kv_heads), _I(head_dim), _I(rotary_dim), _I(page_size),
         _F(eps), _I(_code(dtype)), _stream())


def fused_decode_attention(qkv: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor,
                           q_weight: torch.Tensor | None, k_weight: torch.Tensor | None,
                           inv_freq: torch.Tensor | None, rotary_dim: int, eps: float, k_pages: torch.Tensor,
                           v_pages: torch.Tensor, out: torch.Tensor, seq_lens: torch.Tensor,
                           block_table: torch.Tensor, num_q_heads: int, num_kv_heads: int, head_dim: int,
                           page_size: int, scale: float, window: int | None, max_seq_len: int) -> bool:
    """``head_norm_rope_cache`` and ``paged_attention`` of a decode step (one new token per
    request, in the order of the requests) as one kernel, where there is one for the shape:
    returns False, having done nothing, where there is not."""
    tokens = qkv.shape[0]
    requests = seq_lens.shape[0]
    if (qkv.dtype != torch.bfloat16 or tokens != requests or inv_freq is None or k_pages is None
            or v_pages is None):
        return False
    width = (num_q_heads + 2 * num_kv_heads) * head_dim
    page_shape = (None, num_kv_heads, page_size, head_dim)
    _check("qkv", qkv, torch.bfloat16, (tokens, width))
    _check("positions", positions, torch.int32, (tokens,))
    _check("slot mapping", slots, torch.int32, (tokens,))
    _check("q head-norm weight", q_weight, torch.float32, (head_dim,), optional=True)
    _check("k head-norm weight", k_weight, torch.float32, (head_dim,), optional=True)
    _check("inverse frequencies", inv_freq, torch.float32, (rotary_dim // 2,))
    _check("key pages", k_pages, torch.bfloat16, page_shape)
    _check("value pages", v_pages, torch.bfloat16, page_shape)
    _check("attention output", out, torch.bfloat16, (tokens, num_q_heads * head_dim))
    _check("sequence lengths", seq_lens, torch.int32, (requests,))
    _check("block table", block_table, torch.int32, (requests, None))
    from . import attention_bf16
    return attention_bf16.fused_decode_attention_bf16(
        qkv, positions, slots, q_weight, k_weight, inv_freq, rotary_dim, eps, k_pages, v_pages, out, seq_lens,
        block_table, num_q_heads, num_kv_heads, head_dim, page_size, scale, window, max_seq_len)


def paged_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, out: torch.Tensor,
                    query_start: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
                    num_q_heads: int, num_kv_heads: int, head_dim: int, page_size: int, scale: float,
                    window: int | None, max_query_len: int, max_seq_len: int, num_decode: int = 0,
                    decode_done: bool = False) -> None:
    """Causal attention of every request's new queries over its pages.  ``num_decode``: in a
    step that mixes them, the first that many requests bring one token each (the bfloat16
    kernels then take the two kinds in a launch each); ``decode_done``: those requests have
    their output already, only the others are run."""
    tokens = q.shape[0]
    requests = seq_lens.shape[0]
    dtype = q.dtype
    page_shape = (None, num_kv_heads, page_size, head_dim)
    args_checked = (
        _check("queries", q, (torch.float32, torch.bfloat16), (tokens, num_q_heads * head_dim)),
        _check("key pages", k_pages, dtype, page_shape),
        _check("value pages", v_pages, dtype, page_shape),
        _check("attention output", out, dtype, (tokens, num_q_heads * head_dim)),
        _check("query_start", query_start, torch.int32, (requests + 1,)),
        _check("seq_lens", seq_lens, torch.int32, (requests,)),
        _check("block table", block_table, torch.int32, (requests, None)),
    )
    if dtype == torch.bfloat16:
        from . import attention_bf16
        if attention_bf16.paged_attention_bf16(
                q, k_pages, v_pages, out, query_start, seq_lens, block_table, num_q_heads,
                num_kv_heads, head_dim, page_size, scale, window, max_query_len, max_seq_len, num_decode,
                decode_done):
            return
    if decode_done:
        raise KernelError("paged_attention: decode_done is for the bfloat16 kernels only")
    _run("attention_generic", "b200_paged_attention_generic",
         *(_P(a) for a in args_checked),
         _I(requests), _I(tokens), _I(block_table.shape[1]), _I(num_q_heads), _I(num_kv_heads),
         _I(head_dim), _I(page_size), _F(scale), _I(window or 0), _I(_code(dtype)), _stream())


# --------------------------------------------------------------------- sampling
_U64 = ctypes.c_uint64


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           min_p: torch.Tensor, seeds: torch.Tensor, draw_index: torch.Tensor, tokens: torch.Tensor,
           greedy_eps: float, kinds: int = 3) -> None:
    """One token per row of float32 ``logits``: argmax where ``temperature`` is
    below ``greedy_eps``, otherwise temperature, min-p, top-k, top-p and a seeded
    draw keyed by ``(seeds[r], draw_index[r], token id)``.  Rows without a filter
    (greedy, or ``top_k <= 0``, ``top_p >= 1`` and ``min_p <= 0``) and rows with one
    have a kernel each; a caller that knows the values may say in ``kinds`` which
    are there (bit 0: rows without a filter, bit 1: rows with) and save a launch."""
    rows, vocab = logits.shape
    _run("sampling", "b200_sample",
         _P(_check("logits", logits, torch.float32)), _I(rows), _I(vocab),
         _P(_check("temperature", temperature, torch.float32, (rows,))),
         _P(_check("top_k", top_k, torch.int32, (rows,))),
         _P(_check("top_p", top_p, torch.float32, (rows,))),
         _P(_check("min_p", min_p, torch.float32, (rows,))),
         _P(_check("seeds", seeds, torch.int64, (rows,))),
         _P(_check("draw index", draw_index, torch.int64, (rows,))),
         _P(_check("sampled tokens", tokens, torch.int32, (rows,))), _F(greedy_eps), _I(kinds), _stream())


MAX_LOGPROBS = 32       # the longest list of largest tokens that `logprobs` returns beside the sampled one


def logprobs(logits: torch.Tensor, tokens: torch.Tensor, wanted: torch.Tensor, ids: torch.Tensor,
             values: torch.Tensor, place: torch.Tensor) -> None:
    """For every row r with ``wanted[r] >= 0``: ``values[r, 0]`` = log_softmax(logits[r]) at
    ``tokens[r]`` (``ids[r, 0]``), ``place[r]`` = how many logits of the row are at least as large,
    and columns ``1 .. wanted[r]`` the largest tokens in order with their log-probabilities."""
    rows, vocab = logits.shape
    width = ids.shape[1]
    _run("sampling", "b200_logprobs",
         _P(_check("logits", logits, torch.float32)), _I(rows), _I(vocab),
         _P(_check("sampled tokens", tokens, torch.int32, (rows,))),
         _P(_check("lengths of the lists", wanted, torch.int32, (rows,))), _I(width),
         _P(_check("token ids", ids, torch.int32, (rows, width))),
         _P(_check("log-probabilities", values, torch.float32, (rows, width))),
         _P(_check("places", place, torch.int32, (rows,))), _stream())


def apply_penalties(logits: torch.Tensor, offsets: torch.Tensor, seen_tokens: torch.Tensor,
                    output_counts: torch.Tensor, repetition: torch.Tensor, frequency: torch.Tensor,
                    presence: torch.Tensor, last_tokens: torch.Tensor | None = None,
                    last_rows: torch.Tensor | None = None) -> None:
    """In place: for row r and each distinct seen token ``seen_tokens[offsets[r]:
    offsets[r + 1]]`` apply the repetition, frequency and presence penalties.  With
    ``last_tokens`` and ``last_rows`` row r has one more generated token,
    ``last_tokens[last_rows[r]]`` (none where ``last_rows[r]`` is negative), which the lists do
    not hold because it has not reached the host yet."""
    rows, vocab = logits.shape
    last = (0, 0)
    if last_tokens is not None:
        last = (_check("last tokens", last_tokens, torch.int32), _check("rows of the last tokens", last_rows, torch.int32, (rows,)))
    _run("sampling", "b200_penalties",
         _P(_check("logits", logits, torch.float32)), _I(rows), _I(vocab),
         _P(_check("offsets", offsets, torch.int32, (rows + 1,))),
         _P(_check("seen tokens", seen_tokens, torch.int32)),
         _P(_check("output counts", output_counts, torch.int32, tuple(seen_tokens.shape))),
         _P(_check("repetition", repetition, torch.float32, (rows,))),
         _P(_check("frequency", frequency, torch.float32, (rows,))),
         _P(_check("presence", presence, torch.float32, (rows,))), _P(last[0]), _P(last[1]), _stream())


def mask_tokens(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor) -> None:
    """In place: ``logits[rows[i], tokens[i]] = -inf``."""
    count = rows.shape[0]
    _run("sampling", "b200_mask_tokens",
         _P(_check("logits", logits, torch.float32)), _I(logits.shape[1]),
         _P(_check("rows", rows, torch.int32, (count,))), _P(_check("tokens", tokens, torch.int32, (count,))),
         _I(count), _stream())
