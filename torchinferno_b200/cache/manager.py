"""Paged key/value cache with per-request block tables, and fixed-size state slots.

What the reference does (src/torchinferno/runtime/paged.py:235-539): one pool
``[layers, pages, 2, page, kv_heads, head_dim]``, a LIFO free list whose first
pops are the lowest page ids (:276, :331, :537), one block table per request
shared by all layers (:236-239), ``reserve`` raising ``RuntimeError`` when pages
run out (:329-330), per-page reference counts (:286, :295-309), and the whole
future of a request reserved at admission
(src/torchinferno/runtime/paged_serving.py:1321-1322).

What is different here:

* cache layers are put in **groups** by what they keep (kv_heads, head_dim,
  window); every group has a pool, an allocator and block tables of its own;
* pages are taken as tokens arrive (:meth:`CacheManager.extend`), and a group
  with a window gives pages back as soon as the window has passed them
  (:meth:`CacheManager.release_behind_window`), all others when the request ends;
* one layer's pages are laid out ``[pages, 2, kv_heads, page_size, head_dim]``
  so that the keys of one head in one page are contiguous (keys and values may
  differ in width: a page then holds all its keys, then all its values);
* beside the pages there are **state slots**: every live request has a slot,
  and in it a fixed-size record on the device (``request_records``: length,
  next input token, sampling seed and temperature, count of drawn tokens),
  written whole when the request is opened, read by the decode step for its
  inputs and by the sampler for its parameters; and, for every layer call
  whose mixer asks for one, a fixed-size state tensor that is zeroed when the
  request is opened.

The manager is plain host code apart from the tensors it owns; block-table
changes are queued and applied on the device in one go before a step runs.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Hashable, Sequence

import torch

from torchinferno_b200.parts.base import CacheSpec, StateSpec


# A request's record: int32 words (the kernels' side: csrc/common.cuh TibRequestRecord).
RECORD_WORDS = 8
REC_LENGTH, REC_LAST_TOKEN, REC_SEED_LO, REC_SEED_HI, REC_TEMPERATURE, REC_DRAWN = range(6)


def _i32(value: int) -> int:
    """The low 32 bits of ``value`` as a signed integer."""
    value &= 0xFFFFFFFF
    return value - (1 << 32) if value >= (1 << 31) else value


class OutOfPages(RuntimeError):
    """No free page in some group; nothing was changed by the failed call."""


class CacheError(RuntimeError):
    """Misuse of the cache manager (unknown request, double free, ...)."""


class PageAllocator:
    """Free list and reference counts of one pool."""

    def __init__(self, num_pages: int) -> None:
        if num_pages < 1:
            raise ValueError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(reversed(range(num_pages)))  # pop() yields the lowest id first
        self._refs = [0] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        if self._refs[page] != 0:
            raise CacheError(f"page {page} was on the free list while held")
        self._refs[page] = 1
        return page

    def retain(self, page: int) -> None:
        """Another holder of a page that is already held (hook for sharing a prefix)."""
        if not 0 <= page < self.num_pages or self._refs[page] < 1:
            raise CacheError(f"page {page} is not held")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise CacheError(f"page {page} is outside the pool")
        if self._refs[page] < 1:
            raise CacheError(f"page {page} is freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        return self._refs[page]

    def free_pages(self) -> list[int]:
        return list(self._free)


@dataclass
class GroupBinding:
    pool: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    window: int | None
    keys: torch.Tensor | None = None
    values: torch.Tensor | None = None


@dataclass
class CacheGroup:
    spec: CacheSpec
    cache_layers: list[int]
    allocator: PageAllocator
    pool: torch.Tensor | None             # [layers_in_group, pages, elements of a page]: in a page all keys
                                          # [kv_heads, page_size, head_dim], then all values [kv_heads, page_size, value width]
    table_device: torch.Tensor | None     # [max_slots, max_pages] int32
    pending: dict[int, int] = field(default_factory=dict)    # flat index into table_device -> page id;
                                                             # the last change to an entry wins


@dataclass
class _Request:
    slot: int
    length: int = 0
    pages: list[list[int]] = field(default_factory=list)      # per group: page id per logical page, -1 once given back
    first_live: list[int] = field(default_factory=list)       # per group: first logical page still held


class CacheManager:
    def __init__(self, cache_specs: Sequence[CacheSpec], state_specs: Sequence[StateSpec | None], *,
                 page_size: int, num_pages: int, max_requests: int, max_request_tokens: int,
                 dtype: torch.dtype, device: torch.device | str, allocate_tensors: bool = True) -> None:
        if page_size < 1 or num_pages < 1 or max_requests < 1 or max_request_tokens < 1:
            raise ValueError("page_size, num_pages, max_requests and max_request_tokens must be positive")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.max_pages_per_request = -(-max_request_tokens // page_size)
        self.max_request_tokens = max_request_tokens
        self.dtype = dtype
        self.device = torch.device(device)
        self._tensors = allocate_tensors
        self.groups: list[CacheGroup] = []
        self._group_of_layer: list[tuple[int, int]] = []      # cache layer -> (group, index in group)
        by_spec: dict[CacheSpec, int] = {}
        for layer, spec in enumerate(cache_specs):
            if spec not in by_spec:
                by_spec[spec] = len(self.groups)
                self.groups.append(CacheGroup(spec, [], PageAllocator(num_pages), None, None))
            group = self.groups[by_spec[spec]]
            self._group_of_layer.append((by_spec[spec], len(group.cache_layers)))
            group.cache_layers.append(layer)
        for group in self.groups:
            if allocate_tensors:
                shape = (len(group.cache_layers), num_pages, page_size * group.spec.elements_per_token)
                group.pool = torch.zeros(shape, dtype=dtype, device=self.device)
                group.table_device = torch.full((max_requests, self.max_pages_per_request), -1,
                                                dtype=torch.int32, device=self.device)
        self.state_specs = list(state_specs)
        self.states: list[torch.Tensor | None] = []
        for spec in self.state_specs:
            if spec is None or not allocate_tensors:
                self.states.append(None)
            else:
                self.states.append(torch.zeros((max_requests, *spec.shape), dtype=spec.dtype, device=self.device))
        self.error_word = torch.zeros(1, dtype=torch.int32, device=self.device) if allocate_tensors else None
        # one record per slot; changes are queued like block-table changes (flat index -> word, the last wins)
        self.request_records = torch.zeros((max_requests, RECORD_WORDS), dtype=torch.int32, device=self.device) \
            if allocate_tensors else None
        self.pending_records: dict[int, int] = {}
        self._free_slots = list(reversed(range(max_requests)))
        self._requests: dict[Hashable, _Request] = {}

    # ------------------------------------------------------------ requests
    def __contains__(self, request_id: Hashable) -> bool:
        return request_id in self._requests

    @property
    def live_requests(self) -> list[Hashable]:
        return list(self._requests)

    def free_slots(self) -> int:
        return len(self._free_slots)

    def open(self, request_id: Hashable, *, seed: int = 0, temperature: float = 0.0) -> int:
        """Give the request a state slot and empty block tables; returns the slot.  Its record is written whole
        (length 0, no token, the sampling parameters given, nothing drawn) and its mixer states are zeroed:
        nothing of the slot's last holder is left."""
        if request_id in self._requests:
            raise CacheError(f"request {request_id!r} is already open")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        self._requests[request_id] = _Request(slot, 0, [[] for _ in self.groups], [0 for _ in self.groups])
        for state in self.states:
            if state is not None:
                state[slot].zero_()
        seed &= 0xFFFFFFFFFFFFFFFF
        temperature_bits = struct.unpack("<i", struct.pack("<f", float(temperature)))[0]
        words = {REC_LENGTH: 0, REC_LAST_TOKEN: -1, REC_SEED_LO: _i32(seed), REC_SEED_HI: _i32(seed >> 32),
                 REC_TEMPERATURE: temperature_bits, REC_DRAWN: 0}
        for word in range(RECORD_WORDS):
            self.pending_records[slot * RECORD_WORDS + word] = words.get(word, 0)
        return slot

    def set_record(self, request_id: Hashable, word: int, value: int) -> None:
        """Queue a change of one word of the request's record (applied on the device before the next step)."""
        if not 0 <= word < RECORD_WORDS:
            raise CacheError(f"a record has words 0..{RECORD_WORDS - 1}")
        self.pending_records[self._get(request_id).slot * RECORD_WORDS + word] = _i32(int(value))

    def set_sampling(self, request_id: Hashable, *, seed: int, temperature: float) -> None:
        """Queue new sampling parameters for the request's record."""
        seed &= 0xFFFFFFFFFFFFFFFF
        self.set_record(request_id, REC_SEED_LO, seed)
        self.set_record(request_id, REC_SEED_HI, seed >> 32)
        self.set_record(request_id, REC_TEMPERATURE, struct.unpack("<i", struct.pack("<f", float(temperature)))[0])

    def drain_record_updates(self) -> tuple[list[int], list[int]]:
        """Queued (flat index, word) changes of ``request_records``; clears the queue."""
        out = (list(self.pending_records.keys()), list(self.pending_records.values()))
        self.pending_records = {}
        return out

    def slot(self, request_id: Hashable) -> int:
        return self._get(request_id).slot

    def length(self, request_id: Hashable) -> int:
        return self._get(request_id).length

    def _get(self, request_id: Hashable) -> _Request:
        try:
            return self._requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not open") from None

    # --------------------------------------------------------------- pages
    def pages_needed(self, request_id: Hashable | None, n_tokens: int, length: int | None = None) -> list[int]:
        """New pages per group that ``n_tokens`` more tokens would take."""
        if request_id is not None and request_id in self._requests:
            request = self._requests[request_id]
            have = [len(pages) for pages in request.pages]
            length = request.length
        else:
            have = [0 for _ in self.groups]
            length = length or 0
        need_total = -(-(length + n_tokens) // self.page_size)
        return [max(0, need_total - h) for h in have]

    def can_extend(self, request_id: Hashable | None, n_tokens: int, length: int | None = None) -> bool:
        needed = self.pages_needed(request_id, n_tokens, length)
        return all(n <= g.allocator.num_free for n, g in zip(needed, self.groups))

    def free_pages(self) -> list[int]:
        return [g.allocator.num_free for g in self.groups]

    def extend(self, request_id: Hashable, n_tokens: int) -> int:
        """Make room for ``n_tokens`` more tokens; returns the position of the first.

        Either every group gets its pages or :class:`OutOfPages` is raised and
        nothing has changed.
        """
        request = self._get(request_id)
        if n_tokens < 0:
            raise ValueError("n_tokens must not be negative")
        start = request.length
        if start + n_tokens > self.max_request_tokens:
            raise CacheError(f"request {request_id!r} would hold {start + n_tokens} tokens; "
                             f"the limit is {self.max_request_tokens}")
        needed = self.pages_needed(request_id, n_tokens)
        for n, group in zip(needed, self.groups):
            if n > group.allocator.num_free:
                raise OutOfPages(f"request {request_id!r} needs {n} more pages of group {self.groups.index(group)}, "
                                 f"{group.allocator.num_free} are free")
        for gi, (n, group) in enumerate(zip(needed, self.groups)):
            for _ in range(n):
                page = group.allocator.alloc()
                logical = len(request.pages[gi])
                request.pages[gi].append(page)
                group.pending[request.slot * self.max_pages_per_request + logical] = page
        request.length = start + n_tokens
        return start

    def release_behind_window(self, request_id: Hashable) -> int:
        """Give back pages of windowed groups that no later query can read; returns how many."""
        request = self._get(request_id)
        released = 0
        for gi, group in enumerate(self.groups):
            window = group.spec.window
            if not window:
                continue
            # the next query stands at position `length` and reads keys >= length - window + 1
            first_needed_key = request.length - window + 1
            first_needed_page = max(0, first_needed_key) // self.page_size
            while request.first_live[gi] < min(first_needed_page, len(request.pages[gi])):
                logical = request.first_live[gi]
                page = request.pages[gi][logical]
                if page >= 0:
                    group.allocator.release(page)
                    request.pages[gi][logical] = -1
                    group.pending[request.slot * self.max_pages_per_request + logical] = -1
                    released += 1
                request.first_live[gi] += 1
        return released

    def close(self, request_id: Hashable) -> None:
        """The request is over: its pages and its slot are free again."""
        request = self._get(request_id)
        for gi, group in enumerate(self.groups):
            for logical, page in enumerate(request.pages[gi]):
                if page >= 0:
                    group.allocator.release(page)
                    group.pending[request.slot * self.max_pages_per_request + logical] = -1
        del self._requests[request_id]
        self._free_slots.append(request.slot)

    def block_table(self, request_id: Hashable, group: int = 0) -> list[int]:
        return list(self._get(request_id).pages[group])

    # -------------------------------------------------------------- device
    def drain_table_updates(self) -> list[tuple[list[int], list[int]]]:
        """Queued (flat index, page id) changes of every group's device table; clears the queues.

        Every index appears once (they are applied by one scatter launch, whose writes are unordered)."""
        out = []
        for group in self.groups:
            out.append((list(group.pending.keys()), list(group.pending.values())))
            group.pending = {}
        return out

    def kv_binding(self, cache_layer: int) -> GroupBinding:
        gi, li = self._group_of_layer[cache_layer]
        group = self.groups[gi]
        spec, pages, page = group.spec, group.pool[li], self.page_size
        key_elems = spec.kv_heads * page * spec.head_dim
        keys = pages[:, :key_elems].unflatten(1, (spec.kv_heads, page, spec.head_dim))
        values = pages[:, key_elems:].unflatten(1, (spec.kv_heads, page, spec.value_width)) if spec.value_width else None
        if spec.value_width == spec.head_dim:
            pages = pages.view(self.num_pages, 2, spec.kv_heads, page, spec.head_dim)
        return GroupBinding(pages, group.table_device, page, spec.window, keys, values)

    def group_of_layer(self, cache_layer: int) -> int:
        return self._group_of_layer[cache_layer][0]

    def state(self, call_index: int) -> torch.Tensor | None:
        return self.states[call_index] if call_index < len(self.states) else None

    def kv_bytes_per_token(self) -> int:
        element = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.cache_layers) * g.spec.elements_per_token * element for g in self.groups)

    # --------------------------------------------------------------- audit
    def audit(self) -> None:
        """Raise unless every page is either free or held by exactly one table entry."""
        for gi, group in enumerate(self.groups):
            held: dict[int, int] = {}
            for rid, request in self._requests.items():
                for page in request.pages[gi]:
                    if page >= 0:
                        held[page] = held.get(page, 0) + 1
            free = group.allocator.free_pages()
            if len(set(free)) != len(free):
                raise CacheError(f"group {gi}: a page is on the free list twice")
            for page, count in held.items():
                if count != group.allocator.refcount(page):
                    raise CacheError(f"group {gi}: page {page} held {count} times, refcount {group.allocator.refcount(page)}")
                if page in set(free):
                    raise CacheError(f"group {gi}: page {page} is both held and free")
            if len(held) + len(free) != group.allocator.num_pages:
                raise CacheError(f"group {gi}: {group.allocator.num_pages - len(held) - len(free)} pages are lost")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a state slot is held twice or both held and free")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a state slot is lost")
