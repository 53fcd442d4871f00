"""Causal attention over a paged cache, with grouped key/value heads, optional
per-head RMSNorm of queries and keys, and an optional window.

Computation (minivllm/models/qwen3.py:103-124): one product for queries, keys and
values (rows ``[Q; K; V]`` of one matrix, minivllm/layers/linear.py:209-214) ->
per-head norm over ``head_dim`` with one weight vector for all heads -> position
encoding on queries and keys -> keys and values stored at the new tokens' slots ->
softmax(q k^T * scale + causal mask) v over everything the request has cached
(minivllm/attention/backends/torch_sdpa.py:450-489) -> output product.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from .base import (MIXERS, CacheView, HalfNormedRows, KVPagesNeed, Mixer, Norm, PartEnv, PositionEncoding,
                   StepContext, WeightInfo)


@MIXERS.register("paged_attention")
class PagedAttention(Mixer):
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale`` (default
    ``head_dim ** -0.5``), ``window`` (None = all keys), ``qk_norm_eps`` (None =
    no per-head norm)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params.get("scale", self.head_dim ** -0.5))
        window = params.get("window")
        self.window = None if window is None else int(window)
        eps = params.get("qk_norm_eps")
        self.qk_norm_eps = None if eps is None else float(eps)
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"num_heads={self.num_heads} is not a multiple of num_kv_heads={self.num_kv_heads}")
        if self.head_dim % 2 or self.head_dim > 512:
            raise ValueError(f"head_dim={self.head_dim}: the attention kernels take even sizes up to 512")
        if position.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim={position.rotary_dim} exceeds head_dim={self.head_dim}")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive, got {self.window}")
        self.qkv: torch.Tensor | None = None
        self.out_proj: torch.Tensor | None = None
        self.q_norm: torch.Tensor | None = None
        self.k_norm: torch.Tensor | None = None

    # ------------------------------------------------------------------ weights
    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, d = self.env.hidden_size, self.head_dim
        names = {
            "q_proj.weight": WeightInfo((self.num_heads * d, hidden)),
            "k_proj.weight": WeightInfo((self.num_kv_heads * d, hidden)),
            "v_proj.weight": WeightInfo((self.num_kv_heads * d, hidden)),
            "o_proj.weight": WeightInfo((hidden, self.num_heads * d)),
        }
        if self.qk_norm_eps is not None:
            names["q_norm.weight"] = WeightInfo((d,), "vector")
            names["k_norm.weight"] = WeightInfo((d,), "vector")
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"],
                              tensors["v_proj.weight"]], dim=0).contiguous()
        self.out_proj = tensors["o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors["q_norm.weight"], tensors["k_norm.weight"]

    # -------------------------------------------------------------------- cache
    def cache_need(self) -> KVPagesNeed:
        return KVPagesNeed(self.num_kv_heads, self.head_dim, self.window)

    # ------------------------------------------------------------------ forward
    def splits_norms(self, tokens: int) -> bool:
        return (kernels.split_norm_ok(tokens, self.qkv, fold=False)
                and kernels.split_norm_ok(tokens, self.out_proj, fold=True))

    def forward(self, x: torch.Tensor | HalfNormedRows, ctx: StepContext, cache: CacheView,
                fold: tuple[torch.Tensor, Norm] | None = None) -> torch.Tensor | HalfNormedRows:
        if cache.kind != "pages":
            raise ValueError("paged attention needs a cache of pages")
        group = ctx.groups[cache.group]
        scale = (x.squares, x.eps) if isinstance(x, HalfNormedRows) else None
        x = x.rows if isinstance(x, HalfNormedRows) else x
        tokens = x.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        qkv = torch.empty((tokens, (nq + 2 * nkv) * d), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.qkv, qkv, scale=scale)
        store = cache.writable
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        rope = (self.q_norm, self.k_norm, self.position.inverse_frequencies(), self.position.rotary_dim, eps)
        attended = torch.empty((tokens, nq * d), dtype=x.dtype, device=x.device)
        # Requests that bring one token (all of a decode step, the first ctx.num_decode of a
        # mixed one): norms, rotation, the store of the new key and value and the attention
        # in one kernel, where there is one for the shape.
        single = tokens if ctx.max_query_len == 1 and tokens == ctx.num_requests else ctx.num_decode
        fused = 0
        if store and single > 0 and kernels.fused_decode_attention(
                qkv[:single], ctx.positions[:single], group.slot_mapping[:single], *rope, cache.keys, cache.values,
                attended[:single], ctx.seq_lens[:single], group.block_table[:single], nq, nkv, d, group.page_size,
                self.scale, self.window, ctx.max_seq_len):
            fused = single
        if fused < tokens:
            q = torch.empty((tokens, nq * d), dtype=x.dtype, device=x.device)
            kernels.head_norm_rope_cache(
                qkv[fused:], ctx.positions[fused:], group.slot_mapping[fused:], *rope, q[fused:],
                cache.keys if store else None, cache.values if store else None, nq, nkv, d, group.page_size)
            kernels.paged_attention(
                q, cache.keys, cache.values, attended, ctx.query_start, ctx.seq_lens, group.block_table,
                nq, nkv, d, group.page_size, self.scale, self.window, ctx.max_query_len, ctx.max_seq_len,
                ctx.num_decode, decode_done=fused > 0)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        if fold is None:
            kernels.gemm(attended, self.out_proj, out)
            return out
        residual, norm = fold
        weight, eps = norm.split()
        squares = torch.empty((tokens, self.env.hidden_size // 8), dtype=torch.float32, device=x.device)
        kernels.gemm(attended, self.out_proj, out, fold=(residual, weight, squares))
        return HalfNormedRows(out, squares, eps)
