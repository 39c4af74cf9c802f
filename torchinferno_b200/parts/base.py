"""Interfaces of the parts a layer is put together from, and their registry.

A model is data: a list of blocks, each naming a mixer, a feed-forward, its
norms and a position encoding by *kind* with their sizes and constants as
parameters (:class:`PartSpec`).  The kinds are looked up here.  A part never
learns which model it is in: it sees its parameters, its weights (by names
relative to its own prefix) and, at run time, a :class:`LayerContext`.

Adding a part: subclass the interface, then ``register_part("mixer", "my_kind",
MyMixer)``; a model description may name it at once.

Interfaces
----------
``Part``           ``weight_specs()``, ``bind(weights)``
``Norm``           ``forward(residual, out, rows)`` / ``add_forward(delta, residual, out, rows)``
``PositionEncoding`` ``encode_and_store(qkv, q_out, ctx, heads, kv_heads, head_dim)``
``Mixer``          ``cache_spec()``, ``state_spec()``, ``forward(x, ctx) -> y``
``FeedForward``    ``forward(x, ctx) -> y``
``Block``          ``forward(stream, ctx)`` on a :class:`ResidualStream`
``StreamStage``    ``forward(stream, ctx)`` between the embedding and the first block
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Mapping

import torch


# --------------------------------------------------------------------- data
@dataclass(frozen=True)
class PartSpec:
    """A part named by kind, with its sizes and constants."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""  # weight-name prefix relative to the enclosing block


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part reads from the checkpoint, by name relative to its prefix."""
    name: str
    shape: tuple[int, ...]
    init: str = "normal"       # random mode: "normal" (std), "ones", "zeros"
    std: float = 0.02
    role: str = "matrix"       # "matrix": kept as stored (bf16 / fp32); "vector": widened to fp32;
                               # "int_table": integer table kept as int32
    optional: bool = False     # may be absent from the file (then the part copes)


@dataclass(frozen=True)
class CacheSpec:
    """What a mixer keeps per token: for each of ``kv_heads`` heads a key of ``head_dim`` elements and a
    value of ``value_dim`` elements (None: as wide as the key; 0: keys only, e.g. one latent vector).

    ``window``: None keeps every token; w > 0 means a query at position p reads
    keys p-w+1 .. p only, so pages wholly behind the window may be given back.
    """
    kv_heads: int
    head_dim: int
    window: int | None = None
    value_dim: int | None = None

    @property
    def value_width(self) -> int:
        return self.head_dim if self.value_dim is None else self.value_dim

    @property
    def elements_per_token(self) -> int:
        return self.kv_heads * (self.head_dim + self.value_width)


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size (it does not grow with tokens)."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class KVBinding:
    """The cache one layer call reads and, unless ``writes`` is False, writes."""
    pool: torch.Tensor          # this cache layer's pages: [pages, 2, kv_heads, page_size, head_dim] when keys and
                                # values are equally wide, else the flat pages [pages, elements of a page]
    block_table: torch.Tensor   # [slots, max_pages] int32, on the device
    page_size: int
    window: int | None
    writes: bool = True
    keys: torch.Tensor | None = None     # [pages, kv_heads, page_size, head_dim], a view of the pages
    values: torch.Tensor | None = None   # [pages, kv_heads, page_size, value width], a view of the pages


@dataclass
class LayerContext:
    """What a part sees of the running step."""
    batch: Any                          # engine.batch.StepBatch
    kv: KVBinding | None = None
    state: torch.Tensor | None = None   # [slots, *StateSpec.shape] of this layer, or None
    error_word: torch.Tensor | None = None
    layer_index: int = 0


class ResidualStream:
    """The 32-bit residual sum plus the not-yet-added output of the last part.

    Keeping the last output pending lets a norm fuse the add with itself: one
    pass reads the pending delta and the residual, writes the new residual and
    the normalised rows.
    """

    def __init__(self, residual: torch.Tensor, dtype: torch.dtype) -> None:
        self.residual = residual        # [tokens, hidden] float32
        self.pending: torch.Tensor | None = None
        self.dtype = dtype              # activation dtype of normalised rows

    def normed(self, norm: "Norm", rows: torch.Tensor | None = None) -> torch.Tensor:
        n = self.residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.residual.shape[1]), dtype=self.dtype, device=self.residual.device)
        if self.pending is None:
            norm.forward(self.residual, out, rows)
        else:
            norm.add_forward(self.pending, self.residual, out, rows)
            if rows is None:
                self.pending = None
        return out

    def add(self, delta: torch.Tensor) -> None:
        if self.pending is not None:
            raise RuntimeError("a delta is already pending; a norm must fold it in first")
        self.pending = delta


# --------------------------------------------------------------- interfaces
class Part:
    """Common to all parts: declared weights and their binding."""

    def __init__(self, *, dtype: torch.dtype, device: torch.device) -> None:
        self.dtype = dtype
        self.device = device

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        """Take the tensors named by :meth:`weight_specs` (already on the device)."""


class Norm(Part):
    def forward(self, residual: torch.Tensor, out: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError

    def add_forward(self, delta: torch.Tensor, residual: torch.Tensor, out: torch.Tensor,
                    rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def encode_and_store(self, qkv: torch.Tensor, q_out: torch.Tensor, ctx: LayerContext, heads: int,
                         kv_heads: int, head_dim: int) -> torch.Tensor:
        """Encode positions into q (and k), and write k, v to ``ctx.kv`` if it writes."""
        raise NotImplementedError


class Mixer(Part):
    # ``capturable``: the forward only launches kernels on the current stream and reads the batch through its
    # device arrays, so a decode step that contains it may be captured in a CUDA graph.  Left unset, a mixer
    # without a StateSpec counts as capturable and one with a StateSpec does not (it is taken to walk
    # ``ctx.batch.entries`` on the host); a model with any mixer that is not runs its decode steps uncaptured.
    def cache_spec(self) -> CacheSpec | None:
        return None

    def state_spec(self) -> StateSpec | None:
        return None

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        raise NotImplementedError

    def named_parts(self) -> list[tuple[str, Part]]:
        """(prefix relative to the block, part) for every part that owns weights."""
        raise NotImplementedError


class StreamStage(Part):
    """Something done to the residual stream once, after the embedding and before the first block: a learned
    absolute position table added to it, a multiplier, a norm.  ``ctx`` carries the batch (positions, slots)."""

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        raise NotImplementedError


# ----------------------------------------------------------------- registry
_KINDS = ("mixer", "feed_forward", "norm", "position", "block", "stream_stage")
_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {kind: {} for kind in _KINDS}


def register_part(category: str, kind: str, factory: Callable[..., Part], *, replace: bool = False) -> None:
    if category not in _REGISTRY:
        raise ValueError(f"unknown part category {category!r}; one of {_KINDS}")
    if kind in _REGISTRY[category] and not replace and _REGISTRY[category][kind] is not factory:
        raise ValueError(f"{category} kind {kind!r} is already registered")
    _REGISTRY[category][kind] = factory


def unregister_part(category: str, kind: str) -> None:
    _REGISTRY.get(category, {}).pop(kind, None)


def build_part(category: str, spec: PartSpec, *, dtype: torch.dtype, device: torch.device, **extra: Any) -> Part:
    _ensure_builtin()
    table = _REGISTRY[category]
    if spec.kind not in table:
        raise ValueError(f"no {category} of kind {spec.kind!r}; registered: {sorted(table)}")
    return table[spec.kind](**dict(spec.params), **extra, dtype=dtype, device=device)


def registered_parts(category: str) -> tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(_REGISTRY[category]))


_loaded = False


def _ensure_builtin() -> None:
    global _loaded
    if _loaded:
        return
    _loaded = True
    from torchinferno_b200.parts import attention, block, mlp, norm, rope  # noqa: F401
