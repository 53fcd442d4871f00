"""A model as data: which parts each layer is made of, with their sizes and
constants, and in which order the layers run.

Nothing here knows Qwen3.  An architecture is a function from its typed
configuration to a :class:`ModelSpec`; the assembled model (``parts/model.py``)
reads only the spec.  The reference hard-wires the same structure in classes
(minivllm/models/qwen3.py:127-233 for one layer, :242-338 for the stack).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from types import MappingProxyType
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and the parameters that kind takes."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    # Where its tensors sit in the checkpoint: a layer's parts give the segment
    # under the layer's prefix ("self_attn"), model-level parts the full prefix.
    name: str = ""

    def __post_init__(self) -> None:
        object.__setattr__(self, "params", MappingProxyType(dict(self.params)))

    def __hash__(self) -> int:  # MappingProxyType is not hashable
        return hash((self.kind, self.name, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer's parts.  ``name`` is the prefix of its tensors in the checkpoint.

    ``norms`` maps the role a norm plays in the block's arrangement to its part: the
    pre-norm arrangement asks for ``"mixer"`` and ``"feed_forward"`` (the norms in front
    of each), an arrangement with norms behind them as well would ask for four names.
    Which roles there are is the block kind's business (``Block.norm_roles``); the model
    checks that the layer brings exactly those.  ``feed_forward`` may be None for an
    arrangement that has none.
    """

    name: str
    block: PartSpec                   # how norms, mixer and feed-forward are arranged
    mixer: PartSpec                   # token mixing (attention here)
    feed_forward: PartSpec | None     # dense or experts
    position: PartSpec                # position encoding handed to the mixer
    norms: Mapping[str, PartSpec] = field(default_factory=dict)

    def __post_init__(self) -> None:
        object.__setattr__(self, "norms", MappingProxyType(dict(self.norms)))

    def __hash__(self) -> int:
        return hash((self.name, self.block, self.mixer, self.feed_forward, self.position,
                     tuple(sorted(self.norms.items()))))


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes :attr:`ModelSpec.layers`; the same index may appear in
    several entries (the layer's weights are then used more than once, each
    execution with a cache of its own).  ``cache_from`` names an earlier entry
    of the schedule whose cache this execution reads instead of owning one; it
    then writes nothing into a cache.
    """

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[ScheduleEntry, ...]
    final_norm: PartSpec
    output_head: PartSpec
    # Tensor names that a checkpoint may carry and the model does not read.
    ignored_weights: tuple[str, ...] = ()

    def __post_init__(self) -> None:
        for index, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"schedule[{index}] names layer {entry.layer}, "
                                 f"the model has {len(self.layers)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < index:
                    raise ValueError(
                        f"schedule[{index}].cache_from={entry.cache_from} must name an earlier entry")
                if self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(
                        f"schedule[{index}].cache_from={entry.cache_from} names an entry that "
                        f"owns no cache itself")
