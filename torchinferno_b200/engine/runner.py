"""The step function: run a batch of (request, its next tokens) from the cache.

One call serves whole prompts, portions of prompts cut anywhere, single decoded
tokens, and any mix of them (the reference's closest thing is
``_step_online_unified``: src/torchinferno/runtime/serving.py:2366-2765, with
its forward at src/torchinferno/models/llama3/tensor_parallel.py:6919-7139).
It runs only the tokens it is given, appends their keys and values to the
pages of their requests, and returns fp32 logits for the wanted token rows, in
the order of the entries and of each entry's ``want``.
"""
from __future__ import annotations

from typing import Hashable, Iterable, Sequence

import torch

from torchinferno_b200.cache.manager import CacheManager, OutOfPages
from torchinferno_b200.engine.batch import EntryPlacement, StepBatch, StepEntry, build_batch
from torchinferno_b200.kernels import ops


class StepError(RuntimeError):
    pass


class ModelRunner:
    def __init__(self, model, cache: CacheManager, *, check_errors: bool = True) -> None:
        self.model = model
        self.cache = cache
        self.check_errors = check_errors
        self.last_batch: StepBatch | None = None
        self.steps = 0

    # --------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; returns logits [sum(len(e.want)), vocab] in fp32 on the device."""
        cache, spec = self.cache, self.model.spec
        seen: set[Hashable] = set()
        for entry in entries:
            if entry.request_id in seen:
                raise StepError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            if len(entry.tokens) < 1:
                raise StepError(f"request {entry.request_id!r} brings no tokens")
            for token in entry.tokens:
                if not 0 <= int(token) < spec.vocab_size:
                    raise StepError(f"token id {token} of request {entry.request_id!r} is outside the vocabulary "
                                    f"(size {spec.vocab_size})")
            for w in entry.want:
                if not 0 <= int(w) < len(entry.tokens):
                    raise StepError(f"request {entry.request_id!r} wants logits at {w}, but brings {len(entry.tokens)} tokens")
            held = cache.length(entry.request_id) if entry.request_id in cache else 0
            if held + len(entry.tokens) > spec.max_positions:
                raise StepError(f"request {entry.request_id!r} would reach position {held + len(entry.tokens) - 1}; "
                                f"the model's limit is {spec.max_positions} positions")
        # Room for everything, or nothing is changed.
        need = [0] * len(cache.groups)
        new_requests = 0
        for entry in entries:
            known = entry.request_id in cache
            new_requests += 0 if known else 1
            for g, n in enumerate(cache.pages_needed(entry.request_id if known else None, len(entry.tokens))):
                need[g] += n
        free = cache.free_pages()
        for g, (n, f) in enumerate(zip(need, free)):
            if n > f:
                raise OutOfPages(f"the step needs {n} new pages of cache group {g}, {f} are free")
        if new_requests > cache.free_slots():
            raise StepError(f"the step opens {new_requests} requests, {cache.free_slots()} slots are free")

        placements: list[EntryPlacement] = []
        row = 0
        for entry in entries:
            if entry.request_id not in cache:
                cache.open(entry.request_id)
            start = cache.extend(entry.request_id, len(entry.tokens))
            placements.append(EntryPlacement(entry.request_id, cache.slot(entry.request_id), row, len(entry.tokens), start))
            row += len(entry.tokens)
        batch, updates = build_batch(placements, [e.tokens for e in entries], [e.want for e in entries],
                                     cache.drain_table_updates(), cache.device)
        for group, (index, value) in zip(cache.groups, updates):
            if index.numel():
                ops.scatter_i32(group.table_device, index, value)
        self.last_batch = batch
        logits = self.model.forward(batch, cache)
        for entry in entries:
            cache.release_behind_window(entry.request_id)
        self.steps += 1
        if self.check_errors:
            self.raise_on_device_error()
        return logits

    def end(self, request_ids: Iterable[Hashable]) -> None:
        """These requests are finished: what they hold is given back."""
        for request_id in request_ids:
            if request_id in self.cache:
                self.cache.close(request_id)

    def raise_on_device_error(self) -> None:
        word = int(self.cache.error_word.item())
        if word:
            self.cache.error_word.zero_()
            raise StepError(f"a kernel met a page id outside its pool (code {word:#x}); the step's result is invalid")
