"""One registry from an architecture's name (config.json ``architectures[0]``)
to the pair that builds it: the typed configuration class and the function that
turns a configuration into a model description made of parts.

The reference keeps a module-level dict filled by a decorator and raises a
``ValueError`` that lists what is registered (minivllm/models/registry.py:8-22).
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable, Mapping


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_class: Any                       # has from_dict(mapping) and to_dict()
    build_spec: Callable[[Any], Any]        # configuration -> parts.ModelSpec
    random_weights: Callable[..., dict]     # (configuration, seed, ...) -> {name: tensor}


_ARCHITECTURES: dict[str, ArchitectureEntry] = {}


def register_architecture(name: str, config_class: Any, build_spec: Callable[[Any], Any],
                          random_weights: Callable[..., dict]) -> ArchitectureEntry:
    if name in _ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    entry = ArchitectureEntry(name, config_class, build_spec, random_weights)
    _ARCHITECTURES[name] = entry
    return entry


def registered_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> ArchitectureEntry:
    _load_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ValueError(
            f"architecture {name!r} is not registered; registered: "
            f"{', '.join(sorted(_ARCHITECTURES)) or '(none)'}") from None


def load_model_config(source: str | Path | Mapping[str, Any]):
    """Read config.json (a folder, a file or an already parsed mapping), pick the
    architecture it names and return ``(entry, typed configuration)``."""
    if isinstance(source, Mapping):
        raw = source
    else:
        path = Path(source)
        if path.is_dir():
            path = path / "config.json"
        if not path.is_file():
            raise FileNotFoundError(f"no config.json at {path}")
        raw = json.loads(path.read_text())
    architectures = raw.get("architectures")
    if not isinstance(architectures, (list, tuple)) or len(architectures) != 1:
        raise ValueError(
            f"config.json: 'architectures' must list exactly one name, got {architectures!r}")
    entry = get_architecture(architectures[0])
    return entry, entry.config_class.from_dict(raw)


def _load_builtin() -> None:
    # The built-in architecture registers itself on import; done lazily so that
    # importing the configuration package alone pulls in nothing else.
    from .. import models  # noqa: F401
