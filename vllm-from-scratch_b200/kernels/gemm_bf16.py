"""bfloat16 matrix products with float32 accumulation.

Few rows (decode steps of small batches): the engine's own weight-streaming kernels,
optionally with the gated SiLU fused in.  Otherwise the vendor's library through
``torch.mm``, as the reference's ``F.linear`` does (minivllm/layers/quantization/
methods.py:36-37).
"""

from __future__ import annotations

import ctypes

import torch

from ..csrc.build import load_library

# Partial sums of a product split along K stay in float32: the library must not
# add them up in bfloat16.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False

# Where the engine's own few-rows kernel is the faster one (CUDA-graph timings on B200,
# cold weights): up to 8 rows and up to 8192 weight rows it takes 7.3 / 11.1 / 6.1 us on
# 4096 x 2048, 2048 x 6144 and 2048 x 2048 against the library's 7.3 / 15.0 / 6.6 us; on
# wider matrices (12288 x 2048: 15.5 us against 10.1 us) and from 9 rows on the library's
# kernels are ahead and are used.
SKINNY_MAX_ROWS = 8
# The kernel with weight rows resident in shared memory (slab_gemm.cuh) is ahead of the library up
# to 16 token rows: a decode step at batch 12 takes 1.89 against 2.08 ms, at batch 16 2.05 against 2.22.
RESIDENT_MAX_ROWS = 16
SKINNY_MAX_WEIGHT_ROWS = 8192
# The engine's own few-rows kernels win on the short products of a small model's layer, where
# the wait for the first bytes is most of the time and their copies start before the kernel ahead
# has finished.  A matrix of tens of megabytes streams long enough for that not to matter, and
# there the library's kernels are ahead; their time hardly grows with the token rows, the own
# kernels' does, and the library is at its worst on few weight rows of a long K (launches back to
# back over cold weights, microseconds own / library at 1, 8 and 16 token rows):
#   2048 x 6144 (25 MB)    6.5 / 16.9    7.8 / 14.7    9.6 / 10.2
#   2560 x 4096 (21 MB)    7.5 / 12.7    6.9 / 12.0    8.7 /  8.1
#   6144 x 2560 (31 MB)    8.7 /  8.4   10.1 /  7.8   13.7 /  8.4
#   4096 x 4096 (34 MB)    9.1 / 13.3   12.0 / 11.7   16.9 /  9.7
#   2560 x 9728 (50 MB)   17.8 / 23.3   22.5 / 23.5   29.1 / 15.0
#   6144 x 4096 (50 MB)   12.7 / 11.9   14.9 / 11.4   18.3 / 12.5
#   4096 x 12288 (101 MB) 31.2 / 31.4   37.9 / 30.3   50.1 / 21.6
#   gated 19456 x 2560 (100 MB) 23.0 / 20.4, 24.6 / 19.9, 34.1 / 20.1 (the library's with the activation kernel)
# and the output product over 151936 x 2048 takes the library 105.6 us, 0.90 of the copy bandwidth.
# The limits below follow these; whole decode steps with them against one limit of 40 MB for every
# number of rows (models of 10 to 12 layers): Qwen3-4B widths 1.000 against 1.052 ms at batch 1, 1.236
# against 1.254 at 16; Qwen3-8B widths 1.427 against 1.477 at 16; Qwen3-1.7B widths the same choices.
OWN_MAX_GATED_WEIGHT_BYTES = 64 << 20


def own_limit_bytes(m: int, weight_rows: int, gated: bool) -> int:
    """The largest weight matrix that the engine's own kernels take for ``m`` token rows."""
    if gated:
        return OWN_MAX_GATED_WEIGHT_BYTES
    few_rows = weight_rows <= 4096
    if m <= 4:
        return (56 if few_rows else 40) << 20
    if m <= 8:
        return (36 if few_rows else 28) << 20
    return 26 << 20


_P, _I = ctypes.c_void_p, ctypes.c_int


def _skinny_ok(m: int, n: int, k: int, *tensors: torch.Tensor) -> bool:
    return (1 <= m <= SKINNY_MAX_ROWS and n <= SKINNY_MAX_WEIGHT_ROWS and k >= 32 and k % 32 == 0
            and all(t.data_ptr() % 16 == 0 for t in tensors))


def _small_enough(m: int, w: torch.Tensor, gated: bool) -> bool:
    """Whether a product of ``m`` token rows with ``w`` is one for the engine's own kernels."""
    return w.numel() * w.element_size() <= own_limit_bytes(m, w.shape[0] // 2 if gated else w.shape[0], gated)




def _resident_ok(m: int, k: int, gated: bool, *tensors: torch.Tensor) -> bool:
    """Whether the kernel that keeps a block's weight rows in shared memory takes the
    shape (any number of weight rows): at most 16 tokens, K a multiple of 128, and 8 (gated:
    16) rows of K within 200 KB."""
    rows = 16 if gated else 8
    return (1 <= m <= RESIDENT_MAX_ROWS and k % 128 == 0 and rows * (2 * k + 16) + 192 <= 200 * 1024
            and all(t.data_ptr() % 16 == 0 for t in tensors))


def _skinny(x, w, out, gated_inter: int) -> None:
    from . import KernelError, _stream, count_launch
    lib = load_library("gemm_bf16")
    status = lib.b200_skinny_gemm_bf16(
        _P(x.data_ptr()), _P(w.data_ptr()), _P(out.data_ptr()), _I(x.shape[0]), _I(w.shape[0]), _I(x.shape[1]),
        _I(gated_inter), _I(1 if out.dtype == torch.bfloat16 else 0), _stream())
    if status != 0:
        raise KernelError(lib.b200_last_error().decode())
    count_launch()


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    if _small_enough(x.shape[0], w, False) and (
            _skinny_ok(x.shape[0], w.shape[0], x.shape[1], x, w, out)
            or (w.shape[0] <= SKINNY_MAX_WEIGHT_ROWS and _resident_ok(x.shape[0], x.shape[1], False, x, w, out))):
        _skinny(x, w, out, 0)
    elif out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        # float32 result straight from the float32 accumulator (no bfloat16 rounding).
        out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))


def gated_silu_gemm_bf16(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> bool:
    """``out = silu(x w[:I]^T) * (x w[I:]^T)`` in one kernel; False if the shape is
    not one the fused kernel takes (the caller then does it in two steps)."""
    if tc_gated_ok(x.shape[0], out.shape[1], x.shape[1], x, w_gate_up, out):
        tc_gated_gemm(x, w_gate_up, out)
        return True
    if not _small_enough(x.shape[0], w_gate_up, True) or not (
            _skinny_ok(x.shape[0], w_gate_up.shape[0], x.shape[1], x, w_gate_up, out)
            or _resident_ok(x.shape[0], x.shape[1], True, x, w_gate_up, out)):
        return False
    _skinny(x, w_gate_up, out, out.shape[1])
    return True


# Tests switch the split of the norms off to run the same steps with norm kernels of their own.
USE_SPLIT_NORM = True


def split_norm_ok(tokens: int, w: torch.Tensor, fold: bool, gated: bool = False) -> bool:
    """Whether ``split_norm_gemm`` takes the product: a shape for the resident-rows kernel, where the
    engine would use that kernel anyway, and whole blocks of eight result columns."""
    rows = w.shape[0] // 2 if gated else w.shape[0]
    return (USE_SPLIT_NORM and rows % 8 == 0 and _small_enough(tokens, w, gated)
            and (gated or w.shape[0] <= SKINNY_MAX_WEIGHT_ROWS) and _resident_ok(tokens, w.shape[1], gated, w))


def split_norm_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated_inter: int,
                    scale: tuple[torch.Tensor, float] | None,
                    fold: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None) -> None:
    """The resident-rows product with half of an RMSNorm on either side (see ``kernels.gemm``)."""
    from . import KernelError, _check, _stream, count_launch
    m, k = x.shape
    n = w.shape[0]
    squares_in = pieces = 0
    eps = 0.0
    if scale is not None:
        squares, eps = scale
        squares_in = _check("sums of squares", squares, torch.float32, (m, None))
        pieces = squares.shape[1]
    residual = weight = squares_out = 0
    if fold is not None:
        residual = _check("residual", fold[0], torch.float32, (m, n))
        weight = _check("norm weight", fold[1], torch.float32, (n,))
        squares_out = _check("sums of squares out", fold[2], torch.float32, (m, n // 8))
    lib = load_library("gemm_bf16")
    status = lib.b200_split_norm_gemm_bf16(
        _P(x.data_ptr()), _P(w.data_ptr()), _P(out.data_ptr()), _I(m), _I(n), _I(k), _I(gated_inter),
        _P(squares_in), _I(pieces), ctypes.c_float(eps), _P(residual), _P(weight), _P(squares_out), _stream())
    if status != 0:
        raise KernelError(lib.b200_last_error().decode())
    count_launch()


# The gated product on the 5th-generation tensor cores (csrc/tc_gemm.cuh) is ahead of the library's
# product followed by the activation kernel for whole blocks of 128 token rows from 2048 rows on
# (microseconds own / library + activation: 12288 x 2048 at 2048 rows 80.3 / 83.3, 4096 rows 159 /
# 166, 8192 rows 281 / 317; 24576 x 4096 at 2048 rows 301 / 326, 8192 rows 1287 / 1527; 51200 x 5120 at
# 2048 rows 723 / 857) and level or behind below that and where the last block of rows is partly
# empty (2112 rows: 92.9 / 86.8), so that is where it is used.
USE_TC_GATED = True
TC_GATED_MIN_ROWS = 2048


def tc_gated_ok(m: int, inter: int, k: int, *tensors: torch.Tensor) -> bool:
    if not (USE_TC_GATED and m >= TC_GATED_MIN_ROWS and m % 128 == 0 and all(t.data_ptr() % 16 == 0 for t in tensors)):
        return False
    return int(load_library("gemm_bf16").b200_tc_gated_gemm_tile(_I(m), _I(inter), _I(k))) != 0


def tc_gated_gemm(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """``out = silu(x w[:I]^T) * (x w[I:]^T)`` by the tensor-memory kernel (any number of token rows;
    K a multiple of 64, I a multiple of 96 or 128)."""
    from . import KernelError, _stream, count_launch
    lib = load_library("gemm_bf16")
    status = lib.b200_tc_gated_gemm_bf16(_P(x.data_ptr()), _P(w_gate_up.data_ptr()), _P(out.data_ptr()), _I(x.shape[0]),
                                         _I(out.shape[1]), _I(x.shape[1]), _stream())
    if status != 0:
        raise KernelError(lib.b200_last_error().decode())
    count_launch()


def device_error_code() -> int:
    """0, or the code left by a kernel whose bounded wait ran out (synchronises)."""
    lib = load_library("gemm_bf16")
    return int(lib.b200_stream_gemm_error())
