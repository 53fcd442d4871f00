"""Interfaces of the parts and the registries that map a kind to its class.

A part is built from ``(params, env)``: ``params`` are the sizes and constants
of its :class:`~.spec.PartSpec`, ``env`` says what it is embedded in (the width
of the residual stream, the run dtype, the device, the prefix of its tensors).
A part never learns which model it belongs to.

Every part names the tensors it wants (:meth:`Part.expected_weights`) and takes
them in :meth:`Part.load_weights`; the loader compares the union of these names
with the checkpoint before any tensor is read.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch


# --------------------------------------------------------------------- weights
@dataclass(frozen=True)
class WeightInfo:
    """What a part expects of one checkpoint tensor."""

    shape: tuple[int, ...]
    # "matrix": kept in the run dtype (bfloat16 when serving).
    # "vector": small per-channel tensor used in 32-bit arithmetic, kept in float32.
    # "table":  integer table, kept as int32.
    kind: str = "matrix"


@dataclass(frozen=True)
class PartEnv:
    hidden_size: int
    dtype: torch.dtype
    device: torch.device
    prefix: str


# ----------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class KVPagesNeed:
    """Keys and values in pages.  ``window=None``: every earlier key stays
    readable; ``window=W``: only the last W positions are ever read."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class StateNeed:
    """A tensor of fixed shape per request, addressed by the request's slot."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ---------------------------------------------------------------- step context
@dataclass
class GroupContext:
    """What the layers of one cache group need to address their pages."""

    page_size: int
    block_table: torch.Tensor       # int32 [R, max_pages]; -1 where a page was given back
    slot_mapping: torch.Tensor      # int32 [T]; page * page_size + offset of each new token
    max_pages: int


@dataclass
class StepContext:
    """One batch as the parts see it: T tokens of R requests, flattened request
    after request.  Built by the step function; parts only read it."""

    num_tokens: int
    num_requests: int
    positions: torch.Tensor         # int32 [T] position of each token in its request
    query_start: torch.Tensor       # int32 [R+1] first token row of each request
    seq_lens: torch.Tensor          # int32 [R] tokens of each request after this step
    state_slots: torch.Tensor       # int32 [R] resident slot of each request
    token_request: torch.Tensor     # int32 [T] request row of each token
    max_query_len: int
    max_seq_len: int
    groups: dict[int, GroupContext] = field(default_factory=dict)
    # Host copies for parts written in plain tensor code (tests' toy parts).
    host_query_start: list[int] = field(default_factory=list)
    host_seq_lens: list[int] = field(default_factory=list)
    host_state_slots: list[int] = field(default_factory=list)
    # In a step that mixes them, the first num_decode requests bring one token each and the
    # others portions of prompts; 0 in a step of one kind (and for code that does not care).
    num_decode: int = 0


@dataclass
class CacheView:
    """The cache one execution of a layer works on.

    ``kind`` is "pages" (``keys``/``values`` are ``[pages, kv_heads, page_size,
    head_dim]`` views of this entry's slab and ``group`` indexes
    ``StepContext.groups``), "state" (``state`` is ``[slots, *shape]``) or "none".
    ``writable`` is False when the cache belongs to another schedule entry.
    """

    kind: str = "none"
    group: int = -1
    keys: torch.Tensor | None = None
    values: torch.Tensor | None = None
    state: torch.Tensor | None = None
    writable: bool = True


@dataclass
class HalfNormedRows:
    """Rows half-way through an RMSNorm that is split over the two products around it.

    For float32 residual rows ``v`` and the norm's weights ``g``: ``rows = v * g`` in the run
    dtype and ``squares`` (float32 ``[T, pieces]``) the pieces of every row's sum of ``v**2``.
    ``rmsnorm(v) g W^T = rsqrt(sum / width + eps) * ((v g) W^T)``: the product that takes these
    rows multiplies its result by the root, and no kernel of its own reads and writes the rows
    to normalise them."""

    rows: torch.Tensor
    squares: torch.Tensor
    eps: float


# ----------------------------------------------------------------------- parts
class Part:
    # Whether a step that runs this part may be captured into a CUDA graph and replayed with
    # other batches: everything that differs from step to step must then reach the part as
    # device data (the tensors of the StepContext), never as host values (its ``host_*``
    # lists, ``.item()``, Python branches on the batch).  The engine replays graphs only for
    # models all of whose parts say True; a part that does not say runs without graphs.
    graph_safe: bool = False

    def __init__(self, params: Mapping[str, Any], env: PartEnv) -> None:
        self.params = params
        self.env = env

    def expected_weights(self) -> dict[str, WeightInfo]:
        """Checkpoint names (without the prefix) and what is expected of each."""
        return {}

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take the tensors named by :meth:`expected_weights`, already on the
        device and in the dtype their kind asks for."""


class Norm(Part):
    def forward(self, x: torch.Tensor | None, residual: torch.Tensor, out: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        """``residual += x`` (when ``x`` is given) in 32-bit, then return the
        normalised residual in the run dtype.  With ``rows`` (int32 row indices)
        only those rows are normalised and returned, and ``residual`` is left
        unchanged."""
        raise NotImplementedError

    def split(self) -> tuple[torch.Tensor, float] | None:
        """``(weight, eps)`` if the norm is ``v * rsqrt(mean(v**2) + eps) * weight`` over the whole
        residual width, so that it can be split over the products around it
        (:class:`HalfNormedRows`); None otherwise."""
        return None


class PositionEncoding(Part):
    """Rotary family: the mixer's fused kernel applies it to queries and keys."""

    rotary_dim: int = 0

    def inverse_frequencies(self) -> torch.Tensor | None:
        """float32 ``[rotary_dim // 2]`` on the device, or None for no rotation."""
        return None


class Mixer(Part):
    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env)
        self.position = position

    def cache_need(self) -> KVPagesNeed | StateNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        """``x`` is ``[T, hidden]`` in the run dtype; returns the same shape."""
        raise NotImplementedError

    def splits_norms(self, tokens: int) -> bool:
        """Whether, for a step of so many tokens, ``forward`` also takes
        :class:`HalfNormedRows` for ``x`` and a keyword ``fold=(residual, norm)``, with which
        it adds its result into the float32 ``residual`` itself and returns the
        :class:`HalfNormedRows` of the sum under ``norm``.  A block only asks a part that
        says True."""
        return False


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def splits_norms(self, tokens: int) -> bool:
        """As :meth:`Mixer.splits_norms`."""
        return False


class Embedding(Part):
    """From token ids to the first content of the float32 residual stream.  params always
    hold ``vocab_size``.  ``table()`` is the ``[vocab, hidden]`` matrix an output head that
    is tied to the embedding multiplies by."""

    def forward(self, token_ids: torch.Tensor, ctx: StepContext, residual: torch.Tensor,
                error_flag: torch.Tensor) -> None:
        """Fill ``residual`` (float32 ``[T, hidden]``) for the int32 ``token_ids``; an id outside
        the vocabulary sets ``error_flag[0]`` to 1 + its row and leaves zeros.  ``ctx`` is there
        for embeddings that depend on more than the id (positions, for instance)."""
        raise NotImplementedError

    def table(self) -> torch.Tensor:
        raise NotImplementedError


class OutputHead(Part):
    """From normalised rows of the residual stream to float32 logits.  params always hold
    ``vocab_size``; ``tied`` (default False) says that the head owns no matrix and multiplies
    by the embedding's, which the model hands over with ``bind_embedding``."""

    def bind_embedding(self, embedding: Embedding) -> None:
        """Called once after the weights are loaded."""

    def forward(self, normed: torch.Tensor) -> torch.Tensor:
        """``normed`` is ``[rows, hidden]`` in the run dtype; returns float32 ``[rows, vocab]``."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of norms, a mixer and (usually) a feed-forward around the residual.

    ``norm_roles`` names the norms the arrangement uses; the layer's spec must bring a norm
    for each of them and no other (``norms`` maps role -> built norm).  ``needs_feed_forward``
    says whether a layer without a feed-forward is acceptable."""

    norm_roles: tuple[str, ...] = ()
    needs_feed_forward: bool = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, *, mixer: Mixer,
                 feed_forward: FeedForward | None, norms: Mapping[str, Norm]) -> None:
        super().__init__(params, env)
        if set(norms) != set(self.norm_roles):
            raise ValueError(f"block at {env.prefix!r} arranges norms {sorted(self.norm_roles)}, "
                             f"the layer brings {sorted(norms)}")
        if feed_forward is None and self.needs_feed_forward:
            raise ValueError(f"block at {env.prefix!r} needs a feed-forward, the layer has none")
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, dict(norms)

    def forward(self, x: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                cache: CacheView) -> torch.Tensor:
        """Takes the previous layer's output ``x`` (None for the first layer,
        whose input already sits in ``residual``) and the float32 residual
        stream, updated in place; returns this layer's not-yet-added output."""
        raise NotImplementedError

    # A block may hand its output over already added into the residual and half-normalised
    # under the *next* block's first norm (:class:`HalfNormedRows`), if both sides say so for
    # the step's number of tokens; the model then calls ``forward(..., next_norm=norm)`` and
    # passes what comes back to the next block as its ``x``.  The default is neither.
    def first_norm(self) -> Norm | None:
        """The norm this block applies to what it is handed, if it starts with one."""
        return None

    def takes_half_normed(self, tokens: int) -> bool:
        """Whether ``x`` may be :class:`HalfNormedRows` under :meth:`first_norm`."""
        return False

    def folds_into(self, norm: Norm, tokens: int) -> bool:
        """Whether ``forward`` takes ``next_norm=norm`` and then returns :class:`HalfNormedRows`."""
        return False


# ------------------------------------------------------------------ registries
class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._classes: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        def decorator(cls: Callable[..., Any]) -> Callable[..., Any]:
            if kind in self._classes:
                raise ValueError(f"{self.what} kind {kind!r} is already registered")
            self._classes[kind] = cls
            return cls
        return decorator

    def unregister(self, kind: str) -> None:
        self._classes.pop(kind, None)

    def get(self, kind: str) -> Callable[..., Any]:
        try:
            return self._classes[kind]
        except KeyError:
            raise ValueError(f"{self.what} kind {kind!r} is not registered; registered: "
                             f"{', '.join(sorted(self._classes)) or '(none)'}") from None

    def kinds(self) -> list[str]:
        return sorted(self._classes)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
OUTPUT_HEADS = Registry("output head")
