"""A model as data: parts by kind, a list of blocks and the order they run in.

``layers`` are the distinct blocks (each owns weights).  ``schedule`` is the
order of execution: a list of :class:`LayerCall` that may name a layer twice
and says which cache layer the call uses; a call with ``writes_cache=False``
reads what an earlier call stored there.  ``cache_layers`` is the number of
distinct cache layers the schedule addresses.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from torchinferno_b200.parts.base import PartSpec


@dataclass(frozen=True)
class BlockSpec:
    block: PartSpec                 # category "block"; its params hold the PartSpecs of its parts
    prefix: str                     # weight-name prefix of the layer, e.g. "model.layers.3."


@dataclass(frozen=True)
class LayerCall:
    layer: int                      # index into ModelSpec.layers
    cache: int | None = None        # cache layer this call uses (None: the mixer keeps no keys)
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding_name: str             # tensor name of the [vocab, hidden] table
    layers: tuple[BlockSpec, ...]
    schedule: tuple[LayerCall, ...]
    final_norm: PartSpec            # prefix holds its full name prefix
    head_name: str | None           # tensor name of the [vocab, hidden] output matrix
    tie_head_to_embedding: bool = False
    after_embedding: PartSpec | None = None   # category "stream_stage"; prefix holds its full name prefix
    config: Mapping[str, Any] = field(default_factory=dict)  # the config.json this came from

    def __post_init__(self) -> None:
        for call in self.schedule:
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"schedule names layer {call.layer}, but there are {len(self.layers)}")
        written: set[int] = set()
        for call in self.schedule:
            if call.cache is None:
                continue
            if call.writes_cache:
                if call.cache in written:
                    raise ValueError(f"cache layer {call.cache} is written by two layer calls")
                written.add(call.cache)
            elif call.cache not in written:
                raise ValueError(f"cache layer {call.cache} is read before any call writes it")

    @property
    def cache_layers(self) -> int:
        ids = [call.cache for call in self.schedule if call.cache is not None]
        return max(ids) + 1 if ids else 0
