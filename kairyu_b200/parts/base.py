"""Interfaces of the parts a model is put together from.

A model is data: a tuple of :class:`LayerSpec` (which mixer, feed-forward and
norms a layer has, each with its own sizes) and a tuple of :class:`LayerCall`
(the order in which layers run and which cache slot each call uses).  Parts are
looked up by ``PartSpec.kind`` in open registries, so a new mixer, feed-forward,
norm, position encoding or block arrangement is added by registering a class;
no part knows which model it sits in.

The reference switches these per layer in code (``DecoderLayer`` picking
``Attention`` or ``MlaAttention`` and ``build_mlp``, kairyu/models/llama.py:46-69);
here the switch is the spec.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping, Optional, Sequence

import torch


# --------------------------------------------------------------------------- specs


class PartSpec:
    """``kind`` names a registered part class; ``params`` are its constructor arguments."""

    __slots__ = ("kind", "params")

    def __init__(self, kind: str, **params: Any) -> None:
        self.kind = kind
        self.params = dict(params)

    def _key(self) -> tuple:
        return (self.kind, tuple(sorted((k, repr(v)) for k, v in self.params.items())))

    def __eq__(self, other: object) -> bool:
        return isinstance(other, PartSpec) and self._key() == other._key()

    def __hash__(self) -> int:
        return hash(self._key())

    def __repr__(self) -> str:
        args = ", ".join(f"{k}={v!r}" for k, v in self.params.items())
        return f"PartSpec({self.kind!r}, {args})"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (``block``) of two norms, a mixer and a feed-forward."""

    prefix: str  # tensor-name prefix, e.g. "model.layers.3"
    block: str
    mixer: PartSpec
    ffn: PartSpec
    mixer_norm: PartSpec
    ffn_norm: PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may be named by several
    calls).  ``cache_slot`` is the cache this call's mixer uses; a call with
    ``writes_cache=False`` reads a slot that an earlier call of the same step
    wrote (one layer reading another layer's keys and values).
    """

    layer: int
    cache_slot: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    # A position encoding that acts on the embedding (learned absolute positions and the like);
    # rotary kinds belong to the mixers that use them.
    embedding_position: Optional[PartSpec] = None


# --------------------------------------------------------------------------- weights


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part wants.

    ``role``: ``matrix`` tensors feed matrix products and are held in the
    compute dtype; ``vector`` tensors (norm weights, biases) keep 32-bit storage
    when the file stores them so; ``int_table`` tensors are held as int32.
    ``init``: how the random-weights mode fills it (``normal`` ~N(0, 0.02),
    ``norm`` = 1 + N(0, 0.1), ``zeros``).
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    alias_of: str | None = None  # use that tensor when this one is absent (tied head)


# --------------------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values in pages: ``window=None`` keeps every key, an integer
    keeps the last ``window`` positions (older pages go back to the pool).
    ``v_head_dim``: the width of a value row where it differs from a key row's
    (a mixer whose values are narrower than its keys; None: the same).  Slots
    whose specs are equal share a group: pages of one geometry, one block table."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None
    v_head_dim: int | None = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (one slot per live request)."""

    shape: tuple[int, ...]
    dtype: str = "float32"


@dataclass
class CacheView:
    """What one call's mixer sees of the cache."""

    k: torch.Tensor | None = None  # [num_pages, page_size, kv_heads, head_dim]
    v: torch.Tensor | None = None  # [num_pages, page_size, kv_heads, value_dim]
    page_size: int = 0
    group: int = -1  # which block table of the step belongs to this slot
    state: torch.Tensor | None = None  # [num_state_slots, *StateSpec.shape]
    writes: bool = True


# --------------------------------------------------------------------------- step context


@dataclass
class StepContext:
    """Device-side description of one step's batch, shared by every layer.

    Rows are requests; tokens are flat over rows.  ``tiles[n]`` describes the
    n-query tiles of rows that carry more than one token (prompt portions) as
    (count, row of each tile, offset of each tile within the row's tokens), for
    every n some mixer of the model asked for (``Mixer.query_tile_sizes``);
    ``decode_*`` list rows that carry exactly one token.
    """

    num_tokens: int
    num_rows: int
    dtype: torch.dtype
    token_ids: torch.Tensor  # [T] i32
    positions: torch.Tensor  # [T] i32
    row_ids: torch.Tensor  # [T] i32
    qo_indptr: torch.Tensor  # [B+1] i32
    seq_lens: torch.Tensor  # [B] i32, keys visible to the row's last token
    write_from: torch.Tensor  # [B] i32
    state_slots: torch.Tensor  # [B] i32
    block_tables: dict[int, torch.Tensor]  # group -> [B, max_pages] i32
    host_qo_indptr: tuple[int, ...]
    host_seq_lens: tuple[int, ...]
    # attention work lists
    tiles: dict[int, tuple[int, torch.Tensor, torch.Tensor]] = field(default_factory=dict)
    num_decode_rows: int = 0
    decode_rows: torch.Tensor | None = None  # [n] i32 row ids of 1-token rows
    decode_tokens: torch.Tensor | None = None  # [n] i32 flat token index of each
    max_seq_len: int = 0  # host upper bound over rows (sizes split-KV grids)
    max_portion_seq_len: int = 0  # the same over rows that carry several tokens (prompt portions)
    workspace: Any = None
    error_flag: torch.Tensor | None = None  # [1] i32, set by kernels on bad indices
    extras: dict[str, Any] = field(default_factory=dict)


# --------------------------------------------------------------------------- part interfaces


class Part:
    """Anything with weights.  ``prefix`` is the tensor-name prefix it binds under."""

    # Whether the part's work for a step of prompt portions can be captured in a CUDA graph: every
    # launch takes what changes from step to step (tokens, positions, rows, lengths, pages) from the
    # step's device-side description, nothing from the host.  A part that loops over rows on the host
    # or reads a tensor back leaves this False, and steps of its model are launched one by one.
    graph_safe: bool = False

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Take the tensors named by ``tensor_specs`` (already on the device, in the held dtype)."""

    def bytes_streamed(self) -> int:
        """Weight bytes one step reads (for the roofline)."""
        return 0


class Norm(Part):
    def apply(
        self,
        residual: torch.Tensor,
        delta: torch.Tensor | None,
        ctx: StepContext,
        *,
        rows: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """``residual += delta`` (when given), return ``norm(residual)`` in the
        activation dtype.  With ``rows`` only those token rows are normed and
        the residual is left untouched."""
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_tables(self) -> tuple[torch.Tensor, torch.Tensor] | None:
        """(cos, sin), each [max_positions, rotary_dim/2] fp32, or None."""
        return None

    def embed_hook(self, residual: torch.Tensor, ctx: StepContext) -> None:
        """For encodings that act on the embedding rather than on q and k: called once a step
        with the fp32 residual the embedding produced (``ModelSpec.embedding_position``); changes
        it in place from ``ctx.positions``."""


class Mixer(Part):
    def cache_specs(self) -> tuple[Any, ...]:
        """What this mixer keeps between steps: PagedKVSpec and/or StateSpec."""
        return ()

    def query_tile_sizes(self) -> tuple[int, ...]:
        """Query-tile sizes this mixer's kernels want listed in the step's description
        (``ctx.tiles[n]``): the step function packs a list for every size a mixer names."""
        return ()

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """An arrangement of norms, mixer and feed-forward around the residual."""

    mixer: Mixer

    def forward(
        self,
        residual: torch.Tensor,
        delta: torch.Tensor | None,
        ctx: StepContext,
        cache: CacheView,
    ) -> tuple[torch.Tensor, torch.Tensor | None]:
        """Returns the residual and a not-yet-added delta; the next norm adds
        it, so the residual sum and the following norm are one kernel."""
        raise NotImplementedError


# --------------------------------------------------------------------------- registries


class Registry:
    def __init__(self, what: str) -> None:
        self._what = what
        self._items: dict[str, Callable[..., Any]] = {}

    def register(self, kind: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
        def add(factory: Callable[..., Any]) -> Callable[..., Any]:
            self._items[kind] = factory
            return factory

        return add

    def unregister(self, kind: str) -> None:
        self._items.pop(kind, None)

    def build(self, spec: PartSpec, **context: Any) -> Any:
        if spec.kind not in self._items:
            raise KeyError(
                f"unknown {self._what} {spec.kind!r}; registered: {sorted(self._items)}"
            )
        return self._items[spec.kind](**spec.params, **context)

    def kinds(self) -> Sequence[str]:
        return sorted(self._items)


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("output head")
