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
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, MIXERS, NORMS, OUTPUT_HEADS, POSITION_ENCODINGS, Block,
                   CacheView, KVPagesNeed, PartEnv, StateNeed, StepContext, WeightInfo)
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
        sizes = {"vocab_size": spec.vocab_size}
        self.embedding = EMBEDDINGS.get(spec.embedding.kind)(
            {**sizes, **spec.embedding.params}, self._env(spec.embedding.name))
        self.output_head = OUTPUT_HEADS.get(spec.output_head.kind)(
            {**sizes, **spec.output_head.params}, self._env(spec.output_head.name))
        self._token_error = torch.zeros(1, dtype=torch.int32, device=self.device)

    # ---------------------------------------------------------------- assembly
    def _env(self, prefix: str) -> PartEnv:
        return PartEnv(self.hidden_size, self.dtype, self.device, prefix)

    def _build_layer(self, layer: LayerSpec) -> Block:
        def env(part) -> PartEnv:
            return self._env(_join(layer.name, part.name))
        position = POSITION_ENCODINGS.get(layer.position.kind)(layer.position.params, env(layer.position))
        mixer = MIXERS.get(layer.mixer.kind)(layer.mixer.params, env(layer.mixer), position)
        norms = {role: NORMS.get(part.kind)(part.params, env(part)) for role, part in layer.norms.items()}
        feed_forward = None
        if layer.feed_forward is not None:
            feed_forward = FEED_FORWARDS.get(layer.feed_forward.kind)(
                layer.feed_forward.params, env(layer.feed_forward))
        return BLOCKS.get(layer.block.kind)(
            layer.block.params, env(layer.block), mixer=mixer, feed_forward=feed_forward, norms=norms)

    def _parts(self):
        yield self.embedding
        for block in self.layers:
            yield from (block, block.mixer, block.mixer.position, *block.norms.values())
            if block.feed_forward is not None:
                yield block.feed_forward
        yield from (self.final_norm, self.output_head)

    def graph_safe(self) -> bool:
        """Whether every part says that steps through it may be replayed as CUDA graphs."""
        return all(part.graph_safe for part in self._parts())

    # ----------------------------------------------------------------- weights
    def expected_weights(self) -> dict[str, WeightInfo]:
        names: dict[str, WeightInfo] = {}
        for part in self._parts():
            for name, info in part.expected_weights().items():
                names[_join(part.env.prefix, name)] = info
        return names

    def ignored_weights(self) -> set[str]:
        ignored = set(self.spec.ignored_weights)
        if getattr(self.output_head, "tied", False):
            # A tied checkpoint may still carry the output matrix; it is not read
            # (minivllm/models/qwen3.py:427-430).
            ignored.add(_join(self.spec.output_head.name, "weight"))
        return ignored

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """``tensors``: full checkpoint name -> tensor on the device in the dtype
        its kind asks for (see ``weights.loader``)."""
        for part in self._parts():
            wanted = part.expected_weights()
            if wanted:
                part.load_weights({name: tensors[_join(part.env.prefix, name)] for name in wanted})
        self.output_head.bind_embedding(self.embedding)

    def num_weight_bytes(self) -> int:
        """Bytes of all distinct weight tensors the parts hold (a tied matrix counts once)."""
        seen, total = set(), 0
        for part in self._parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
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
        self.embedding.forward(token_ids, ctx, residual, self._token_error)
        x = None
        blocks = [self.layers[entry.layer] for entry in self.spec.schedule]
        for number, (block, cache) in enumerate(zip(blocks, caches)):
            # Two blocks that both say so for this many tokens split the norm between them: the
            # first adds its output into the residual itself and hands on rows half-normalised
            # under the second's first norm.
            after = blocks[number + 1] if number + 1 < len(blocks) else None
            norm = after.first_norm() if after is not None and after.takes_half_normed(tokens) else None
            if norm is not None and block.folds_into(norm, tokens):
                x = block.forward(x, residual, ctx, cache, next_norm=norm)
            else:
                x = block.forward(x, residual, ctx, cache)
        return x, residual

    def logits(self, x: torch.Tensor | None, residual: torch.Tensor, rows: torch.Tensor) -> torch.Tensor:
        """float32 logits ``[len(rows), vocab]`` at the given token rows."""
        return self.output_head.forward(self.final_norm.forward(x, residual, rows=rows))

    def check_token_ids(self) -> None:
        """Raise if a step since the last check met a token id outside the vocabulary."""
        flag = int(self._token_error.item())
        if flag:
            self._token_error.zero_()
            raise ValueError(f"token id outside [0, {self.vocab_size}) at batch row {flag - 1}")
