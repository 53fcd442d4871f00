"""Dense gated feed-forward: ``down(silu(gate(x)) * up(x))``, no biases
(minivllm/models/qwen3.py:44-65).  ``gate`` and ``up`` are held as one matrix
``[2 I, H]`` with the gate rows first (minivllm/layers/linear.py:261-359), so one
product serves both."""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import FEED_FORWARDS, FeedForward, HalfNormedRows, Norm, PartEnv, StepContext, WeightInfo


@FEED_FORWARDS.register("gated_silu")
class GatedSiluFeedForward(FeedForward):
    """params: ``intermediate_size``."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.intermediate_size = int(params["intermediate_size"])
        self.gate_up: torch.Tensor | None = None
        self.down: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        inter, hidden = self.intermediate_size, self.env.hidden_size
        return {
            "gate_proj.weight": WeightInfo((inter, hidden)),
            "up_proj.weight": WeightInfo((inter, hidden)),
            "down_proj.weight": WeightInfo((hidden, inter)),
        }

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.gate_up = torch.cat([tensors["gate_proj.weight"], tensors["up_proj.weight"]], dim=0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def splits_norms(self, tokens: int) -> bool:
        return (kernels.split_norm_ok(tokens, self.gate_up, fold=False, gated=True)
                and kernels.split_norm_ok(tokens, self.down, fold=True))

    def forward(self, x: torch.Tensor | HalfNormedRows, ctx: StepContext,
                fold: tuple[torch.Tensor, Norm] | None = None) -> torch.Tensor | HalfNormedRows:
        scale = (x.squares, x.eps) if isinstance(x, HalfNormedRows) else None
        x = x.rows if isinstance(x, HalfNormedRows) else x
        tokens = x.shape[0]
        hidden = torch.empty((tokens, self.intermediate_size), dtype=x.dtype, device=x.device)
        kernels.gated_silu_gemm(x, self.gate_up, hidden, scale=scale)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        if fold is None:
            kernels.gemm(hidden, self.down, out)
            return out
        residual, norm = fold
        weight, eps = norm.split()
        squares = torch.empty((tokens, self.env.hidden_size // 8), dtype=torch.float32, device=x.device)
        kernels.gemm(hidden, self.down, out, fold=(residual, weight, squares))
        return HalfNormedRows(out, squares, eps)
