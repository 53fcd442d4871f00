"""bfloat16 matrix products with float32 accumulation.

Few rows and a matrix of moderate height (decode steps of small batches): the
engine's own weight-streaming kernel, optionally with the gated SiLU fused in.
Otherwise the vendor's library through ``torch.mm``, as the reference's ``F.linear``
does (minivllm/layers/quantization/methods.py:36-37).  A tcgen05 / tensor-memory
kernel for up to 256 rows (``tc_gemm_bf16``: K split over a thread-block cluster, the
partial tiles added through distributed shared memory) is built and tested; alone it is
ahead of the library for three of a layer's four products up to about 32 rows, in a
decode step of 24 or 64 requests it is level with it or behind, so it is chosen only
when ``B200_TC_GEMM_ROWS`` says up to how many rows.
"""

from __future__ import annotations

import ctypes
import os

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
# Up to this many token rows (above RESIDENT_MAX_ROWS) the tcgen05 weight-streaming kernel
# (tc_gemm.cuh) is chosen; the environment variable B200_TC_GEMM_ROWS overrides it.  Measured
# (CUDA graphs, cold weights, 4096 x 2048 / 2048 x 2048 / gated 12288 x 2048 / 2048 x 6144):
# 17 rows 6.8 / 5.2 / 12.7 / 8.9 us against the library's 5.9 / 5.6 / 13.9 (with the
# activation kernel) / 10.6; 64 rows 8.5 / 6.8 / 14.3 / 10.1 against 6.4 / 5.8 / 14.1 / 10.8.
# A decode step: 24 requests 2.46 against 2.41 ms, 64 requests 4.31 against 4.16 ms.
TC_MAX_ROWS = 0
_P, _I = ctypes.c_void_p, ctypes.c_int


def _skinny_ok(m: int, n: int, k: int, *tensors: torch.Tensor) -> bool:
    return (1 <= m <= SKINNY_MAX_ROWS and n <= SKINNY_MAX_WEIGHT_ROWS and k >= 32 and k % 32 == 0
            and all(t.data_ptr() % 16 == 0 for t in tensors))


def _resident_ok(m: int, k: int, gated: bool, *tensors: torch.Tensor) -> bool:
    """Whether the kernel that keeps a block's weight rows in shared memory takes the
    shape (any number of weight rows): at most 16 tokens, K a multiple of 128, and 8 (gated:
    16) rows of K within 200 KB."""
    if os.environ.get("B200_NO_SLAB_GEMM") is not None or (gated and os.environ.get("B200_NO_SLAB_GATED") is not None):
        return False
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


def _tc_ok(m: int, n: int, k: int, *tensors: torch.Tensor) -> bool:
    """Whether the tcgen05 weight-streaming kernel is the choice for the shape."""
    rows = int(os.environ.get("B200_TC_GEMM_ROWS", TC_MAX_ROWS))
    return (RESIDENT_MAX_ROWS < m <= rows and n <= SKINNY_MAX_WEIGHT_ROWS * 2 and tc_gemm_supported(m, n, k)
            and all(t.data_ptr() % 16 == 0 for t in tensors))


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    if _tc_ok(x.shape[0], w.shape[0], x.shape[1], x, w, out):
        tc_gemm_bf16(x, w, out)
    elif (_skinny_ok(x.shape[0], w.shape[0], x.shape[1], x, w, out)
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
    if _tc_ok(x.shape[0], w_gate_up.shape[0], x.shape[1], x, w_gate_up, out):
        tc_gemm_bf16(x, w_gate_up, out, gated=True)
        return True
    if not (_skinny_ok(x.shape[0], w_gate_up.shape[0], x.shape[1], x, w_gate_up, out)
            or _resident_ok(x.shape[0], x.shape[1], True, x, w_gate_up, out)):
        return False
    _skinny(x, w_gate_up, out, out.shape[1])
    return True


# ------------------------------------------------------------ tcgen05 product
def tc_gemm_supported(m: int, n: int, k: int) -> bool:
    return 1 <= m <= 256 and k >= 64 and k % 8 == 0 and n >= 1


def tc_gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, gated: bool = False) -> None:
    """The tensor-memory kernel (tc_gemm.cuh): ``out = x @ w^T``, or with ``gated``
    ``out = silu(x @ w[:I]^T) * (x @ w[I:]^T)``.  Allocates nothing."""
    from . import KernelError, _stream, count_launch
    lib = load_library("gemm_bf16")
    m, k = x.shape
    n = w.shape[0]
    status = lib.b200_tc_gemm_bf16(
        _P(x.data_ptr()), _P(w.data_ptr()), _P(out.data_ptr()), _I(m), _I(n), _I(k), _I(n // 2 if gated else 0),
        _I(1 if out.dtype == torch.bfloat16 else 0), _stream())
    if status != 0:
        raise KernelError(lib.b200_last_error().decode())
    count_launch()


def device_error_code() -> int:
    """0, or the code left by a kernel whose bounded wait ran out (synchronises)."""
    lib = load_library("gemm_bf16")
    return int(lib.b200_stream_gemm_error())
