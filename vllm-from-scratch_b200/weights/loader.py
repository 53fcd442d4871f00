"""Weights from safetensors, by tensor name.

A model folder holds ``config.json`` and either ``model.safetensors`` or
``model.safetensors.index.json`` with its shards (minivllm/model_loader/
weight_utils.py:65-100).  Before any tensor is read, the names and shapes in the
files are compared with what the model's parts expect; every difference (missing,
unexpected, wrong shape, duplicated across shards) is reported in ONE error.  The
reference raises separate errors for these (minivllm/model_loader/
auto_weights_loader.py:168-227, minivllm/layers/linear.py:80-85, 566-568).

dtype on the device: a matrix is held in the run dtype (bfloat16 when serving,
float32 in the 32-bit mode); a per-channel vector is held in float32, which keeps
a tensor stored in 32-bit as it is and widens a bfloat16 one exactly; an integer
table becomes int32.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Mapping

import torch
from safetensors import safe_open

from ..parts.base import WeightInfo

_INTEGER = (torch.int8, torch.int16, torch.int32, torch.int64, torch.uint8)


class WeightLoadError(ValueError):
    """The checkpoint does not match the model; the message lists every mismatch."""

    def __init__(self, folder: str, missing: list[str], unexpected: list[str],
                 wrong_shape: list[tuple[str, tuple, tuple]], other: list[str]) -> None:
        self.missing, self.unexpected, self.wrong_shape, self.other = missing, unexpected, wrong_shape, other
        lines = [f"weights in {folder} do not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shape ({len(wrong_shape)}): " + ", ".join(
                f"{name} is {list(found)}, expected {list(expected)}" for name, found, expected in wrong_shape))
        lines.extend(f"  {line}" for line in other)
        super().__init__("\n".join(lines))


def weight_files(folder: str | Path) -> list[Path]:
    folder = Path(folder)
    if not folder.is_dir():
        raise FileNotFoundError(f"model folder {folder} does not exist")
    index = folder / "model.safetensors.index.json"
    single = folder / "model.safetensors"
    if index.is_file():
        shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        missing = [name for name in shards if not (folder / name).is_file()]
        if missing:
            raise FileNotFoundError(f"{index} names shards that are not there: {', '.join(missing)}")
        return [folder / name for name in shards]
    if single.is_file():
        return [single]
    others = sorted(p.name for p in folder.iterdir() if p.suffix in (".bin", ".pt", ".pth", ".gguf"))
    if others:
        raise NotImplementedError(
            f"{folder} holds {', '.join(others)}; only safetensors checkpoints are read")
    raise FileNotFoundError(
        f"no model.safetensors or model.safetensors.index.json in {folder} "
        f"(found: {', '.join(sorted(p.name for p in folder.iterdir())) or 'nothing'})")


def _target_dtype(info: WeightInfo, stored: torch.dtype, run_dtype: torch.dtype) -> torch.dtype:
    if info.kind == "table" or stored in _INTEGER:
        return torch.int32
    if info.kind == "vector":
        return torch.float32
    return run_dtype


def check_names(folder: str | Path, expected: Mapping[str, WeightInfo], ignored: set[str]) -> dict[str, Path]:
    """Compare file contents with ``expected``; return name -> file for the wanted tensors."""
    where: dict[str, Path] = {}
    shapes: dict[str, tuple] = {}
    other: list[str] = []
    for path in weight_files(folder):
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name in handle.keys():
                if name in where:
                    other.append(f"{name} appears in both {where[name].name} and {path.name}")
                    continue
                where[name] = path
                shapes[name] = tuple(handle.get_slice(name).get_shape())
    missing = sorted(name for name in expected if name not in where)
    unexpected = sorted(name for name in where if name not in expected and name not in ignored)
    wrong = sorted((name, shapes[name], tuple(info.shape)) for name, info in expected.items()
                   if name in shapes and shapes[name] != tuple(info.shape))
    if missing or unexpected or wrong or other:
        raise WeightLoadError(str(folder), missing, unexpected, wrong, other)
    return {name: where[name] for name in expected}


def load_weights(model, folder: str | Path) -> None:
    """Read the checkpoint in ``folder`` into ``model`` (a ``parts.DecoderModel``
    or anything with ``expected_weights``, ``ignored_weights``, ``load_weights``,
    ``dtype`` and ``device``)."""
    expected = model.expected_weights()
    where = check_names(folder, expected, model.ignored_weights())
    tensors: dict[str, torch.Tensor] = {}
    by_file: dict[Path, list[str]] = {}
    for name, path in where.items():
        by_file.setdefault(path, []).append(name)
    for path, names in by_file.items():
        with safe_open(str(path), framework="pt", device="cpu") as handle:
            for name in sorted(names):
                stored = handle.get_tensor(name)
                target = _target_dtype(expected[name], stored.dtype, model.dtype)
                tensors[name] = stored.to(device=model.device, dtype=target)
    model.load_weights(tensors)


def load_weights_from_tensors(model, tensors: Mapping[str, torch.Tensor]) -> None:
    """The same checks and conversions for tensors that are already in memory
    (the random-weights mode without a trip through the disk)."""
    expected = model.expected_weights()
    ignored = model.ignored_weights()
    missing = sorted(name for name in expected if name not in tensors)
    unexpected = sorted(name for name in tensors if name not in expected and name not in ignored)
    wrong = sorted((name, tuple(tensors[name].shape), tuple(info.shape)) for name, info in expected.items()
                   if name in tensors and tuple(tensors[name].shape) != tuple(info.shape))
    if missing or unexpected or wrong:
        raise WeightLoadError("(in memory)", missing, unexpected, wrong, [])
    model.load_weights({
        name: tensors[name].to(device=model.device,
                               dtype=_target_dtype(info, tensors[name].dtype, model.dtype))
        for name, info in expected.items()})
