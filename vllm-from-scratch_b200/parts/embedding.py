"""The two ends of the model: token ids into the residual stream, and normalised rows of
it into logits.

``token_embedding``: a row of the ``[vocab, hidden]`` table per token, widened to float32
(minivllm/models/qwen3.py:300-306).  ``linear_head``: logits = rows . W^T in float32, W
being the embedding's table when ``tied`` (minivllm/models/qwen3.py:372-376, 393-395).
Both are parts like any other: an architecture whose embedding is scaled, or whose logits
are capped, registers its own kinds and names them in its ``ModelSpec``.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import EMBEDDINGS, OUTPUT_HEADS, Embedding, OutputHead, PartEnv, StepContext, WeightInfo


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Embedding):
    """params: ``vocab_size``."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.vocab_size = int(params["vocab_size"])
        self.weight: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        return {"weight": WeightInfo((self.vocab_size, self.env.hidden_size))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, residual: torch.Tensor,
                error_flag: torch.Tensor) -> None:
        kernels.embedding(self.weight, token_ids, residual, error_flag)

    def table(self) -> torch.Tensor:
        return self.weight


@OUTPUT_HEADS.register("linear_head")
class LinearHead(OutputHead):
    """params: ``vocab_size``, ``tied`` (default False)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.vocab_size = int(params["vocab_size"])
        self.tied = bool(params.get("tied", False))
        self.weight: torch.Tensor | None = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        return {} if self.tied else {"weight": WeightInfo((self.vocab_size, self.env.hidden_size))}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def bind_embedding(self, embedding: Embedding) -> None:
        if self.tied:
            self.weight = embedding.table()         # the very tensor: read once a step, held once

    def forward(self, normed: torch.Tensor) -> torch.Tensor:
        out = torch.empty((normed.shape[0], self.vocab_size), dtype=torch.float32, device=normed.device)
        kernels.gemm(normed, self.weight, out)
        return out
