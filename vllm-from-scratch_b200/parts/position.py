"""Position encodings of the rotary family.

``rotary``: rotate-half ("neox") rotation of the first ``rotary_dim`` channels of
every query and key head by the angle ``position * theta^(-2j / rotary_dim)``
(minivllm/layers/rotary_embedding.py:143-185 builds the same frequencies;
minivllm/layers/ops/rotary_embedding.py:243-257 applies them).  The reference
tabulates cos/sin per position and casts the table to the run dtype; here the
angle is formed and its sine and cosine taken in float32 inside the kernel, so
only the frequencies are stored.

``none``: no rotation.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .base import POSITION_ENCODINGS, PartEnv, PositionEncoding


@POSITION_ENCODINGS.register("rotary")
class RotaryPositionEncoding(PositionEncoding):
    """params: ``theta`` (base), ``rotary_dim`` (channels rotated, even),
    ``scaling_factor`` (positions are divided by it; 1.0 = plain)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        super().__init__(params, env)
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        self.scaling_factor = float(params.get("scaling_factor", 1.0))
        if self.theta <= 0 or self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary position encoding: theta={self.theta}, rotary_dim={self.rotary_dim}")
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponents)
        if self.scaling_factor != 1.0:
            inv_freq = inv_freq / self.scaling_factor
        self._inv_freq = inv_freq.to(env.device)

    def inverse_frequencies(self) -> torch.Tensor:
        return self._inv_freq


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    rotary_dim = 0
    graph_safe = True
