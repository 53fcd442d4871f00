"""The decoder assembled from a :class:`~.spec.ModelSpec`.

Embedding -> the schedule's layer executions -> final norm on the wanted rows ->
output product on those rows only (the reference computes logits for selected
rows too, minivllm/models/qwen3.py:393-395 and minivllm/worker/
gpu_model_runner.py:1647-1653).  The model owns the parts and their weights; it
owns no cache and knows no request: the step function hands it a
:class:`~.base.StepContext` and one :class:`~.base.CacheView` per schedule entry.
"""

from __future__ import annotations

from typing import Mapping

import torch

from .. import kernels
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheView,
                   KVPagesNeed, PartEnv, StateNeed, StepContext, WeightInfo)
from .spec import LayerSpec, ModelSpec


def _join(prefix: str, name: str) -> str:
    return f"{prefix}.{name}" if prefix and name else prefix or name


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.layers: list[Block] = [self._build_layer(layer) for layer in spec.layers]
        self.final_norm = NORMS.get(spec.final_norm.kind)(
            spec.final_norm.params, self._env(spec.final_norm.name))
        self.tied_output = bool(spec.output_head.params.get("tied", False))
        self.embedding: torch.Tensor | None = None
        self.output_weight: torch.Tensor | None = None
        self._token_error = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ---------------------------------------------------------------- assembly
    def _env(self, prefix: str) -> PartEnv:
        return PartEnv(self.hidden_size, self.dtype, self.device, prefix)

    def _build_layer(self, layer: LayerSpec) -> Block:
        def env(part) -> PartEnv:
            return self._env(_join(layer.name, part.name))
        position = POSITION_ENCODINGS.get(layer.position.kind)(layer.position.params, env(layer.position))
        mixer = MIXERS.get(layer.mixer.kind)(layer.mixer.params, env(layer.mixer), position)
        mixer_norm = NORMS.get(layer.mixer_norm.kind)(layer.mixer_norm.params, env(layer.mixer_norm))
        feed_forward = FEED_FORWARDS.get(layer.feed_forward.kind)(
            layer.feed_forward.params, env(layer.feed_forward))
        feed_forward_norm = NORMS.get(layer.feed_forward_norm.kind)(
            layer.feed_forward_norm.params, env(layer.feed_forward_norm))
        return BLOCKS.get(layer.block.kind)(
            layer.block.params, env(layer.block), mixer=mixer, mixer_norm=mixer_norm,
            feed_forward=feed_forward, feed_forward_norm=feed_forward_norm)

    def _parts(self):
        for block in self.layers:
            yield from (block, block.mixer_norm, block.mixer, block.feed_forward_norm, block.feed_forward)
        yield self.final_norm

    # ----------------------------------------------------------------- weights
    def expected_weights(self) -> dict[str, WeightInfo]:
        names: dict[str, WeightInfo] = {
            _join(self.spec.embedding.name, "weight"): WeightInfo((self.vocab_size, self.hidden_size)),
        }
        if not self.tied_output:
            names[_join(self.spec.output_head.name, "weight")] = WeightInfo(
                (self.vocab_size, self.hidden_size))
        for part in self._parts():
            for name, info in part.expected_weights().items():
                names[_join(part.env.prefix, name)] = info
        return names

    def ignored_weights(self) -> set[str]:
        ignored = set(self.spec.ignored_weights)
        if self.tied_output:
            # A tied checkpoint may still carry the output matrix; it is not read
            # (minivllm/models/qwen3.py:427-430).
            ignored.add(_join(self.spec.output_head.name, "weight"))
        return ignored

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """``tensors``: full checkpoint name -> tensor on the device in the dtype
        its kind asks for (see ``weights.loader``)."""
        self.embedding = tensors[_join(self.spec.embedding.name, "weight")].contiguous()
        self.output_weight = (self.embedding if self.tied_output else
                              tensors[_join(self.spec.output_head.name, "weight")].contiguous())
        for part in self._parts():
            wanted = part.expected_weights()
            if wanted:
                part.load_weights({name: tensors[_join(part.env.prefix, name)] for name in wanted})

    def num_weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in self._parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                    seen.add(value.data_ptr())
                    total += value.numel() * value.element_size()
        for value in (self.embedding, self.output_weight):
            if value is not None and value.data_ptr() not in seen:
                seen.add(value.data_ptr())
                total += value.numel() * value.element_size()
        return total

    # ------------------------------------------------------------------- cache
    def cache_needs(self) -> list[KVPagesNeed | StateNeed | None]:
        """One entry per schedule entry: what its execution must own (None when
        it owns nothing, including when it reads another entry's cache)."""
        needs: list[KVPagesNeed | StateNeed | None] = []
        for entry in self.spec.schedule:
            need = self.layers[entry.layer].mixer.cache_need()
            needs.append(None if entry.cache_from is not None else need)
        return needs

    # ----------------------------------------------------------------- forward
    def forward(self, token_ids: torch.Tensor, ctx: StepContext, caches: list[CacheView]
                ) -> tuple[torch.Tensor | None, torch.Tensor]:
        """Run every schedule entry over the batch.  Returns the last layer's
        not-yet-added output and the float32 residual stream."""
        tokens = token_ids.shape[0]
        residual = torch.empty((tokens, self.hidden_size), dtype=torch.float32, device=token_ids.device)
        kernels.embedding(self.embedding, token_ids, residual, self._token_error)
        x: torch.Tensor | None = None
        for entry, cache in zip(self.spec.schedule, caches):
            x = self.layers[entry.layer].forward(x, residual, ctx, cache)
        return x, residual

    def logits(self, x: torch.Tensor | None, residual: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits ``[len(rows), vocab]`` at the given token rows."""
        normed = self.final_norm.forward(x, residual, rows=rows)
        out = torch.empty((rows.shape[0], self.vocab_size), dtype=torch.float32, device=residual.device)
        kernels.gemm(normed, self.output_weight, out)
        return out

    def check_token_ids(self) -> None:
        """Raise if a step since the last check met a token id outside the vocabulary."""
        flag = int(self._token_error.item())
        if flag:
            self._token_error.zero_()
            raise ValueError(f"token id outside [0, {self.vocab_size}) at batch row {flag - 1}")
