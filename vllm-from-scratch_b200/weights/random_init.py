"""Random-weights mode: write a model folder (config.json, model.safetensors)
from a configuration and a seed.

The reference has such a generator only among its test helpers
(minivllm/testing/tiny_models.py:31-130, 811-850); here it is part of the engine
so that benchmarks and the command line can run shapes for which no checkpoint
is at hand.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

import torch
from safetensors.torch import save_file

from ..config.registry import load_model_config


def write_random_model(config: Mapping[str, Any] | Any, seed: int, folder: str | Path,
                       dtype: torch.dtype = torch.bfloat16, **init: Any) -> Path:
    """``config`` is config.json content (a mapping) or a typed configuration.
    Returns the folder, which then loads like any checkpoint."""
    if isinstance(config, Mapping):
        entry, typed = load_model_config(config)
    else:
        typed = config
        entry, _ = load_model_config(typed.to_dict())
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(typed.to_dict(), indent=2) + "\n")
    tensors = entry.random_weights(typed, seed, dtype=dtype, **init)
    save_file({name: tensor.contiguous() for name, tensor in tensors.items()},
              str(folder / "model.safetensors"))
    return folder
