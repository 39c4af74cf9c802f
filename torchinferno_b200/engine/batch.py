"""The ragged batch one step runs.

The reference's unified step pads rows to the longest entry and carries
``q_lens``, ``seq_lens``, ``write_positions`` and ``logit_positions``
(src/torchinferno/runtime/serving.py:2587-2600).  Here nothing is padded: all
tokens of the step lie on one axis, and an entry (one request's next tokens) is
a range of it.

Device arrays (int32, views into one uploaded buffer):
  token_ids[t], positions[t], token_slot[t]     per token
  q_start[e] (n_entries + 1), kv_start[e], slots[e]   per entry
  logit_rows[i], logit_slots[i]                 token rows whose logits are wanted, and the slot of their request
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import torch


@dataclass(frozen=True)
class StepEntry:
    """One request's share of a step: its next tokens and where logits are wanted."""
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()      # indices into ``tokens``
    seed: int = 0                 # sampling parameters, written into the request's record when this step opens it
    temperature: float = 0.0


@dataclass
class EntryPlacement:
    request_id: Hashable
    slot: int
    q_start: int
    q_len: int
    kv_start: int                 # tokens the request held before this step


@dataclass
class StepBatch:
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_slot: torch.Tensor
    q_start: torch.Tensor
    kv_start: torch.Tensor
    slots: torch.Tensor
    logit_rows: torch.Tensor
    logit_slots: torch.Tensor
    n_tokens: int
    n_entries: int
    n_logits: int
    max_q_len: int
    max_kv_len: int               # bound on the longest context (cached + new tokens) of an entry
    n_single: int = 0             # entries that bring one token
    n_multi: int = 0              # entries that bring more
    entries: list[EntryPlacement] = field(default_factory=list)
    h2d_bytes: int = 0


def build_batch(placements: list[EntryPlacement], tokens: list[Sequence[int]], wants: list[Sequence[int]],
                table_updates: list[tuple[list[int], list[int]]], device: torch.device
                ) -> tuple[StepBatch, list[tuple[torch.Tensor, torch.Tensor]]]:
    """Pack the step's integers into one host buffer, upload it once, and slice it."""
    token_ids: list[int] = []
    positions: list[int] = []
    token_slot: list[int] = []
    q_start = [0]
    kv_start: list[int] = []
    slots: list[int] = []
    logit_rows: list[int] = []
    logit_slots: list[int] = []
    for place, toks, want in zip(placements, tokens, wants):
        token_ids.extend(int(t) for t in toks)
        positions.extend(range(place.kv_start, place.kv_start + place.q_len))
        token_slot.extend([place.slot] * place.q_len)
        q_start.append(place.q_start + place.q_len)
        kv_start.append(place.kv_start)
        slots.append(place.slot)
        logit_rows.extend(place.q_start + int(w) for w in want)
        logit_slots.extend([place.slot] * len(want))
    sections = [token_ids, positions, token_slot, q_start, kv_start, slots, logit_rows, logit_slots]
    for index, value in table_updates:
        sections.extend((index, value))
    total = sum(len(s) for s in sections)
    use_cuda = device.type == "cuda"
    host = torch.empty(max(total, 1), dtype=torch.int32, pin_memory=use_cuda)
    flat: list[int] = []
    for section in sections:
        flat.extend(section)
    if flat:
        host[:total] = torch.tensor(flat, dtype=torch.int32)
    dev = host.to(device, non_blocking=use_cuda)
    views: list[torch.Tensor] = []
    offset = 0
    for section in sections:
        views.append(dev[offset: offset + len(section)])
        offset += len(section)
    batch = StepBatch(
        token_ids=views[0], positions=views[1], token_slot=views[2], q_start=views[3], kv_start=views[4],
        slots=views[5], logit_rows=views[6], logit_slots=views[7], n_tokens=len(token_ids), n_entries=len(placements),
        n_logits=len(logit_rows), max_q_len=max((p.q_len for p in placements), default=0),
        max_kv_len=max((p.kv_start + p.q_len for p in placements), default=0),
        n_single=sum(1 for p in placements if p.q_len == 1), n_multi=sum(1 for p in placements if p.q_len > 1),
        entries=placements, h2d_bytes=total * 4)
    updates = [(views[8 + 2 * i], views[9 + 2 * i]) for i in range(len(table_updates))]
    return batch, updates
