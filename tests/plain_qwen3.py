"""A plain, slow Qwen3: whole sequences, no cache, one function for each part.

Written from the reference's formulas (file:line cited at each function, paths
inside tutu04538/vllm-from-scratch); it shares no code with the engine.  It was
compared once with the reference's own ``Qwen3ForCausalLM`` on the CPU for two
tiny random models; the script and its small outputs are in ``tests/golden/``.

Everything is computed in the dtype asked for (float32 or float64), never lower,
on the device the weights are on (the CPU for the tiny models; a CUDA device, with
its reduced-precision matrix modes switched off by the caller, for wide ones).
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def read_config(raw: dict) -> dict:
    """The keys the reference's model reads, with its defaults
    (minivllm/models/qwen3.py:47-52, 71-101, 256-270, 364-376)."""
    heads = raw["num_attention_heads"]
    rope = dict(raw.get("rope_parameters") or {})
    layers = raw["num_hidden_layers"]
    windows = [None] * layers
    if raw.get("use_sliding_window", False):
        # Not read by the reference (full attention everywhere); meaning taken from
        # the checkpoint format: layers named "sliding_attention" see the last
        # `sliding_window` positions only.
        kinds = raw.get("layer_types") or [
            "sliding_attention" if i >= raw.get("max_window_layers", layers) else "full_attention"
            for i in range(layers)]
        windows = [raw["sliding_window"] if kind == "sliding_attention" else None for kind in kinds]
    return {
        "vocab": raw["vocab_size"], "hidden": raw["hidden_size"], "inter": raw["intermediate_size"],
        "layers": layers, "heads": heads, "kv_heads": raw.get("num_key_value_heads", heads),
        "head_dim": raw.get("head_dim", raw["hidden_size"] // heads),
        "eps": raw.get("rms_norm_eps", 1e-6),
        "theta": rope.get("rope_theta", raw.get("rope_theta", 10000.0)),
        "tied": raw.get("tie_word_embeddings", False),
        "windows": windows,
    }


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """minivllm/layers/ops/layernorm.py:196-227: variance = mean(x^2) over the
    last axis, y = x * rsqrt(variance + eps) * weight."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def rope_cos_sin(positions: torch.Tensor, rotary_dim: int, theta: float, dtype: torch.dtype):
    """minivllm/layers/rotary_embedding.py:143-185: inv_freq_j = theta^(-2j/rotary_dim)
    built in float32, angle = position * inv_freq_j."""
    inv_freq = (1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))).to(positions.device)
    if dtype == torch.float64:   # a finer oracle: the same float32 frequencies, exact product
        angles = positions.to(torch.float64)[:, None] * inv_freq.to(torch.float64)[None, :]
    else:
        angles = torch.einsum("i,j->ij", positions.to(torch.float32), inv_freq)
    return angles.cos().to(dtype), angles.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """minivllm/layers/ops/rotary_embedding.py:243-257 (rotate-half): x is
    [S, heads, d]; x1 = first half, x2 = second half; o1 = x1 cos - x2 sin,
    o2 = x2 cos + x1 sin."""
    half = cos.shape[-1]
    x1, x2, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s, rest), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None) -> torch.Tensor:
    """minivllm/attention/backends/torch_sdpa.py:450-489: q [S, nq, d], k/v [S, nkv,
    d]; query head h reads key/value head h // (nq / nkv); scores = q k^T * scale;
    key j visible to query i iff j <= i (and, with a window, j > i - window);
    softmax over visible keys; output [S, nq * d]."""
    seq, nq, d = q.shape
    group = nq // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(seq, device=q.device)[:, None]
    j = torch.arange(seq, device=q.device)[None, :]
    visible = j <= i
    if window is not None:
        visible = visible & (j > i - window)
    scores = scores.masked_fill(~visible[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hij,jhd->ihd", probs, v).reshape(seq, nq * d)


def attention_block(x: torch.Tensor, positions: torch.Tensor, w: dict, prefix: str, cfg: dict,
                    window: int | None) -> torch.Tensor:
    """minivllm/models/qwen3.py:103-124: projections, per-head RMSNorm of q and k
    over head_dim (one weight vector for all heads) BEFORE the rotation, rotation
    of q and k, attention, output projection."""
    seq = x.shape[0]
    nq, nkv, d = cfg["heads"], cfg["kv_heads"], cfg["head_dim"]
    q = (x @ w[prefix + "q_proj.weight"].T).view(seq, nq, d)
    k = (x @ w[prefix + "k_proj.weight"].T).view(seq, nkv, d)
    v = (x @ w[prefix + "v_proj.weight"].T).view(seq, nkv, d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], cfg["eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], cfg["eps"])
    cos, sin = rope_cos_sin(positions, d, cfg["theta"], x.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = causal_attention(q, k, v, 1.0 / math.sqrt(d), window)
    return out @ w[prefix + "o_proj.weight"].T


def feed_forward(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """minivllm/models/qwen3.py:44-65: down(silu(gate(x)) * up(x)), silu(z) = z sigmoid(z)."""
    gate = x @ w[prefix + "gate_proj.weight"].T
    up = x @ w[prefix + "up_proj.weight"].T
    return (gate * torch.sigmoid(gate) * up) @ w[prefix + "down_proj.weight"].T


def qwen3_hidden(cfg: dict, w: dict, tokens: torch.Tensor) -> torch.Tensor:
    """minivllm/models/qwen3.py:308-338 in its net effect: h += attn(norm(h));
    h += mlp(norm(h)) per layer, then the final norm."""
    positions = torch.arange(tokens.shape[0], device=tokens.device)
    h = w["model.embed_tokens.weight"][tokens]
    for layer in range(cfg["layers"]):
        prefix = f"model.layers.{layer}."
        normed = rms_norm(h, w[prefix + "input_layernorm.weight"], cfg["eps"])
        h = h + attention_block(normed, positions, w, prefix + "self_attn.", cfg, cfg["windows"][layer])
        normed = rms_norm(h, w[prefix + "post_attention_layernorm.weight"], cfg["eps"])
        h = h + feed_forward(normed, w, prefix + "mlp.")
    return rms_norm(h, w["model.norm.weight"], cfg["eps"])


def qwen3_logits(raw_config: dict, weights: dict, tokens, dtype: torch.dtype = torch.float32
                 ) -> torch.Tensor:
    """Logits at every position of one whole sequence, [S, vocab]
    (minivllm/models/qwen3.py:393-395; tied head :372-376)."""
    cfg = read_config(raw_config)
    w = {name: tensor.to(dtype) for name, tensor in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long).to(w["model.embed_tokens.weight"].device)
    hidden = qwen3_hidden(cfg, w, tokens)
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return hidden @ head.T


def load_folder(folder: str | Path) -> tuple[dict, dict]:
    from safetensors.torch import load_file
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))
