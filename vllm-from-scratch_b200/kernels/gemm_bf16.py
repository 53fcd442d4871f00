"""bfloat16 matrix product with float32 accumulation.

The product goes to the vendor's library through ``torch.mm``, as the
reference's ``F.linear`` does (minivllm/layers/quantization/methods.py:36-37).
"""

from __future__ import annotations

import torch

# Partial sums of a product split along K stay in float32: the library must not
# add them up in bfloat16.
torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False


def gemm_bf16(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    if out.dtype == torch.bfloat16:
        torch.mm(x, w.t(), out=out)
    else:
        # float32 result straight from the float32 accumulator (no bfloat16 rounding).
        out.copy_(torch.mm(x, w.t(), out_dtype=torch.float32))
