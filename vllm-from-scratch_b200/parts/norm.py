"""RMSNorm with the residual sum fused in.

``y = x * rsqrt(mean(x^2) + eps) * weight`` with the statistics in float32
(minivllm/layers/ops/layernorm.py:196-227; class minivllm/layers/layernorm.py:26-52).
The residual stream it adds into is float32.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import NORMS, Norm, PartEnv, WeightInfo


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """params: ``eps`` (inside the root), ``size`` (defaults to the residual width)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.eps = float(params["eps"])
        self.size = int(params.get("size", env.hidden_size))
        self.weight: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        return {"weight": WeightInfo((self.size,), "vector")}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]

    def split(self) -> tuple[torch.Tensor, float] | None:
        return (self.weight, self.eps) if self.size == self.env.hidden_size else None

    def forward(self, x: torch.Tensor | None, residual: torch.Tensor, out: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            count = residual.shape[0] if rows is None else rows.shape[0]
            out = torch.empty((count, self.size), dtype=self.env.dtype, device=residual.device)
        kernels.add_rmsnorm(x, residual, self.weight, self.eps, out, rows)
        return out
