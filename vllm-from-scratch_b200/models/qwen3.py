"""Qwen3 dense decoder as a description made of parts.

Structure and tensor names follow minivllm/models/qwen3.py: layers of
(input_layernorm, self_attn with q/k head norms and rotate-half position
encoding, post_attention_layernorm, gated-SiLU mlp) :127-233, a final ``norm``
and an ``lm_head`` that is the embedding itself when ``tie_word_embeddings``
:360-376.  Checkpoint names: minivllm/testing/tiny_models.py:832-850.
"""

from __future__ import annotations

import torch

from ..config.model_config import Qwen3Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def build_spec(config: Qwen3Config) -> ModelSpec:
    norm = {"eps": config.rms_norm_eps}
    layers = []
    for index in range(config.num_hidden_layers):
        layers.append(LayerSpec(
            name=f"model.layers.{index}",
            block=PartSpec("pre_norm"),
            mixer=PartSpec("paged_attention", {
                "num_heads": config.num_attention_heads,
                "num_kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "scale": config.head_dim ** -0.5,
                "window": config.layer_windows[index],
                "qk_norm_eps": config.rms_norm_eps,
            }, name="self_attn"),
            feed_forward=PartSpec("gated_silu", {"intermediate_size": config.intermediate_size}, name="mlp"),
            position=PartSpec("rotary", {"theta": config.rope_theta, "rotary_dim": config.head_dim}),
            norms={"mixer": PartSpec("rms_norm", norm, name="input_layernorm"),
                   "feed_forward": PartSpec("rms_norm", norm, name="post_attention_layernorm")},
        ))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=PartSpec("token_embedding", name="model.embed_tokens"),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=index) for index in range(config.num_hidden_layers)),
        final_norm=PartSpec("rms_norm", norm, name="model.norm"),
        output_head=PartSpec("linear_head", {"tied": config.tie_word_embeddings}, name="lm_head"),
    )


def random_weights(config: Qwen3Config, seed: int, *, std: float | None = None, norm_std: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu"
                   ) -> dict[str, torch.Tensor]:
    """Seeded random tensors under the checkpoint's names: matrices and the
    embedding ``N(0, std)`` (``std`` defaults to the configuration's
    ``initializer_range``), norm weights ``1 + N(0, norm_std)``.  The reference's
    generator draws the matrices the same way and sets norm weights to one
    (minivllm/testing/tiny_models.py:811-850); weights of exactly one would hide a
    misplaced norm weight, hence the spread.  ``device`` says where the tensors are
    drawn (a CUDA device draws a large model in seconds; the values then differ from
    the CPU's for the same seed)."""
    std = config.initializer_range if std is None else std
    generator = torch.Generator(device=device).manual_seed(seed)

    def matrix(*shape: int) -> torch.Tensor:
        return torch.empty(*shape, dtype=torch.float32, device=device).normal_(
            0.0, std, generator=generator).to(dtype)

    def norm(size: int) -> torch.Tensor:
        return (1.0 + torch.empty(size, dtype=torch.float32, device=device).normal_(
            0.0, norm_std, generator=generator)).to(dtype)

    hidden, inter, d = config.hidden_size, config.intermediate_size, config.head_dim
    weights = {"model.embed_tokens.weight": matrix(config.vocab_size, hidden)}
    for index in range(config.num_hidden_layers):
        prefix = f"model.layers.{index}."
        weights[prefix + "input_layernorm.weight"] = norm(hidden)
        weights[prefix + "self_attn.q_proj.weight"] = matrix(config.q_width, hidden)
        weights[prefix + "self_attn.k_proj.weight"] = matrix(config.kv_width, hidden)
        weights[prefix + "self_attn.v_proj.weight"] = matrix(config.kv_width, hidden)
        weights[prefix + "self_attn.o_proj.weight"] = matrix(hidden, config.q_width)
        weights[prefix + "self_attn.q_norm.weight"] = norm(d)
        weights[prefix + "self_attn.k_norm.weight"] = norm(d)
        weights[prefix + "post_attention_layernorm.weight"] = norm(hidden)
        weights[prefix + "mlp.gate_proj.weight"] = matrix(inter, hidden)
        weights[prefix + "mlp.up_proj.weight"] = matrix(inter, hidden)
        weights[prefix + "mlp.down_proj.weight"] = matrix(hidden, inter)
    weights["model.norm.weight"] = norm(hidden)
    if not config.tie_word_embeddings:
        weights["lm_head.weight"] = matrix(config.vocab_size, hidden)
    return weights


register_architecture("Qwen3ForCausalLM", Qwen3Config, build_spec, random_weights)
