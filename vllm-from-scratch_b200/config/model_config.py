"""Typed configuration of the dense Qwen3 decoder, read from config.json keys.

The reference passes the raw config.json dict to its model and reads it with
``config[...]`` / ``config.get(..., default)`` (minivllm/models/qwen3.py:47-52,
69-101, 256-270, 364-376).  The same keys and the same defaults are read here,
once, into a frozen dataclass; every size and constant the engine uses comes
from this object and from nowhere else.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value the engine refuses."""


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "max_position_embeddings",
)


def _positive_int(raw: Mapping[str, Any], key: str, value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {key!r} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    """Sizes and constants of one Qwen3 dense checkpoint.

    Keys and defaults follow minivllm/models/qwen3.py:71-101 (attention),
    :47-52 (feed-forward), :256-270 (stack) and :364-376 (output head).
    ``layer_windows`` is the one addition: the reference never reads
    ``use_sliding_window`` / ``sliding_window`` / ``max_window_layers`` /
    ``layer_types`` and so runs every layer with all keys; here the keys are
    honoured when ``use_sliding_window`` is true (it is false in every published
    Qwen3 checkpoint, which gives the reference's behaviour).
    """

    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    eos_token_id: int | None
    initializer_range: float
    # One entry per layer: None = every earlier key is visible, W = the last W keys.
    layer_windows: tuple[int | None, ...] = field(default=())

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "Qwen3Config":
        missing = [key for key in _REQUIRED if key not in raw]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {', '.join(missing)}")
        architectures = raw.get("architectures")
        if not isinstance(architectures, (list, tuple)) or len(architectures) != 1:
            # minivllm/model_loader/base_loader.py:40-49: exactly one entry.
            raise ConfigError(
                f"config.json: 'architectures' must list exactly one name, got {architectures!r}")
        values = {key: _positive_int(raw, key, raw[key]) for key in _REQUIRED}
        heads = values["num_attention_heads"]
        kv_heads = _positive_int(raw, "num_key_value_heads", raw.get("num_key_value_heads", heads))
        head_dim = _positive_int(raw, "head_dim", raw.get("head_dim", values["hidden_size"] // heads))
        if heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads ({heads}) must be a multiple of num_key_value_heads ({kv_heads})")
        if head_dim % 2:
            raise ConfigError(f"head_dim ({head_dim}) must be even for rotate-half position encoding")
        if raw.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"only hidden_act='silu' is built, got {raw.get('hidden_act')!r}")
        if raw.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not built: Qwen3 dense checkpoints carry no biases")

        rope = dict(raw.get("rope_parameters") or raw.get("rope_scaling") or {})
        rope_type = rope.get("rope_type", rope.get("type", "default"))
        if rope_type != "default":
            raise ConfigError(f"only rope_type='default' is built, got {rope_type!r}")
        if float(rope.get("partial_rotary_factor", raw.get("partial_rotary_factor", 1.0))) != 1.0:
            raise ConfigError("partial_rotary_factor other than 1.0 is not part of Qwen3 dense")
        theta = float(rope.get("rope_theta", raw.get("rope_theta", 10000.0)))
        if theta <= 0:
            raise ConfigError(f"rope_theta must be positive, got {theta}")
        eps = float(raw.get("rms_norm_eps", 1e-6))
        if eps <= 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {eps}")

        layers = values["num_hidden_layers"]
        windows: list[int | None] = [None] * layers
        if raw.get("use_sliding_window", False):
            window = raw.get("sliding_window")
            window = _positive_int(raw, "sliding_window", window)
            layer_types = raw.get("layer_types")
            if layer_types is None:
                first_windowed = int(raw.get("max_window_layers", layers))
                layer_types = ["sliding_attention" if i >= first_windowed else "full_attention"
                               for i in range(layers)]
            if len(layer_types) != layers:
                raise ConfigError(
                    f"layer_types has {len(layer_types)} entries for {layers} layers")
            for index, kind in enumerate(layer_types):
                if kind == "sliding_attention":
                    windows[index] = window
                elif kind != "full_attention":
                    raise ConfigError(f"layer_types[{index}]={kind!r} is not an attention kind of Qwen3")

        eos = raw.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else None
        return cls(
            architecture=str(architectures[0]),
            vocab_size=values["vocab_size"],
            hidden_size=values["hidden_size"],
            intermediate_size=values["intermediate_size"],
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            max_position_embeddings=values["max_position_embeddings"],
            rms_norm_eps=eps,
            rope_theta=theta,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            eos_token_id=None if eos is None else int(eos),
            initializer_range=float(raw.get("initializer_range", 0.02)),
            layer_windows=tuple(windows),
        )

    @classmethod
    def from_json(cls, path: str | Path) -> "Qwen3Config":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        """config.json content that reads back to an equal object."""
        out: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "initializer_range": self.initializer_range,
        }
        if self.eos_token_id is not None:
            out["eos_token_id"] = self.eos_token_id
        windows = {w for w in self.layer_windows if w is not None}
        if windows:
            if len(windows) != 1:
                raise ConfigError("config.json can name one sliding_window size only")
            out["use_sliding_window"] = True
            out["sliding_window"] = windows.pop()
            out["layer_types"] = ["full_attention" if w is None else "sliding_attention"
                                  for w in self.layer_windows]
        return out

    # ------------------------------------------------------------------ derived
    @property
    def q_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_parameters(self) -> int:
        per_layer = (
            self.hidden_size * (self.q_width + 2 * self.kv_width)
            + self.q_width * self.hidden_size
            + 3 * self.hidden_size * self.intermediate_size
            + 2 * self.hidden_size
            + 2 * self.head_dim
        )
        embed = self.vocab_size * self.hidden_size
        head = 0 if self.tie_word_embeddings else embed
        return self.num_hidden_layers * per_layer + embed + head + self.hidden_size
