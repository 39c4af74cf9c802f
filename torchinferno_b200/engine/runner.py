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

from torchinferno_b200.cache.manager import REC_LAST_TOKEN, REC_LENGTH, CacheManager, OutOfPages
from torchinferno_b200.engine.batch import EntryPlacement, StepBatch, StepEntry, build_batch
from torchinferno_b200.kernels import gemm, ops


class StepError(RuntimeError):
    pass


class _DecodeGraph:
    """The forward pass of a pure decode batch of ``n`` requests, captured once and replayed.

    The reference replays whole-step decode graphs over static buffers that are refilled outside
    the graph (src/torchinferno/runtime/paged_serving.py:333-397) and pads the batch by repeating a
    row; here a graph is captured per exact batch size, so no padded row ever touches the cache.
    The static integers are: token ids, positions (also the number of cached tokens, since each
    request brings one token), slots (also the slot of each token), and the fixed ranges
    q_start = 0..n and logit_rows = 0..n-1.  Only the slots come from the host, and only when the set of
    requests changes: the pass begins with a kernel that reads every request's next token and position from
    its record on the device and moves the record on (``ops.decode_inputs``).
    """

    def __init__(self, n: int, device: torch.device, max_kv_len: int) -> None:
        self.n = n
        self.buffer = torch.zeros(5 * n + 1, dtype=torch.int32, device=device)
        self.token_ids, self.positions, self.slots = (self.buffer[i * n:(i + 1) * n] for i in range(3))
        self.q_start = self.buffer[3 * n: 4 * n + 1]
        self.logit_rows = self.buffer[4 * n + 1: 5 * n + 1]
        self.q_start.copy_(torch.arange(n + 1, dtype=torch.int32))
        self.logit_rows.copy_(torch.arange(n, dtype=torch.int32))
        self.batch = StepBatch(
            token_ids=self.token_ids, positions=self.positions, token_slot=self.slots, q_start=self.q_start,
            kv_start=self.positions, slots=self.slots, logit_rows=self.logit_rows, logit_slots=self.slots, n_tokens=n, n_entries=n,
            n_logits=n, max_q_len=1, max_kv_len=max_kv_len, n_single=n, n_multi=0, entries=[])
        self.graph: torch.cuda.CUDAGraph | None = None
        self.logits: torch.Tensor | None = None
        self.launches = 0          # kernels of this library inside the graph
        self.host_slots: list[int] | None = None     # what self.slots holds


class ModelRunner:
    def __init__(self, model, cache: CacheManager, *, check_errors: bool = True, use_cuda_graphs: bool = True) -> None:
        self.model = model
        self.cache = cache
        self.check_errors = check_errors
        self.last_batch: StepBatch | None = None
        self.steps = 0
        # what the steps so far did, and the last one alone (same keys): tokens run, pages taken from and given
        # back to the pools, bytes copied to the device, steps that replayed a captured graph
        self.counters = {"steps": 0, "tokens": 0, "pages_taken": 0, "pages_freed": 0, "h2d_bytes": 0, "graph_steps": 0}
        self.last_step: dict[str, int] = {}
        # a part that walks the step's entries on the host cannot be captured: no graph for such a model
        self.use_cuda_graphs = use_cuda_graphs
        self._graph_ok = model.capturable()
        self._graphs: dict[int, _DecodeGraph] = {}
        self._graph_generation = gemm.generation()
        gemm.set_error_word(cache.error_word)   # bounded waits of the tcgen05 kernels report here
        self.graph_replays = 0

    # --------------------------------------------------------------- step
    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Run one batch; returns logits [sum(len(e.want)), vocab] in fp32 on the device.  A pure decode batch
        that replays a captured graph returns that graph's own output buffer: it holds these logits until the
        next step of the same batch size."""
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

        if (self.use_cuda_graphs and self._graph_ok and cache.device.type == "cuda"
                and all(len(e.tokens) == 1 and tuple(e.want) == (0,) for e in entries)):
            return self._decode_step(entries)

        placements: list[EntryPlacement] = []
        row = 0
        free_before = cache.free_pages()
        for entry in entries:
            if entry.request_id not in cache:
                cache.open(entry.request_id, seed=entry.seed, temperature=entry.temperature)
            start = cache.extend(entry.request_id, len(entry.tokens))
            # (the record's length after the step is the position of the token a sampler would draw from it)
            cache.set_record(entry.request_id, REC_LENGTH, start + len(entry.tokens))
            placements.append(EntryPlacement(entry.request_id, cache.slot(entry.request_id), row, len(entry.tokens), start))
            row += len(entry.tokens)
        batch, updates = build_batch(placements, [e.tokens for e in entries], [e.want for e in entries],
                                     cache.drain_table_updates() + [cache.drain_record_updates()], cache.device)
        targets = [group.table_device for group in cache.groups] + [cache.request_records]
        for target, (index, value) in zip(targets, updates):
            if index.numel():
                ops.scatter_i32(target, index, value)
        self.last_batch = batch
        free_mid = cache.free_pages()
        logits = self.model.forward(batch, cache)
        for entry in entries:
            cache.release_behind_window(entry.request_id)
        self.steps += 1
        self._count(batch, free_before, free_mid, False)
        if self.check_errors:
            self.raise_on_device_error()
        return logits

    def _count(self, batch: StepBatch, free_before: list[int], free_mid: list[int], graph: bool) -> None:
        """Per-step counters: ``free_before`` / ``free_mid`` are the free pages before the step took its pages and
        after (before windows gave pages back)."""
        free_after = self.cache.free_pages()
        self.last_step = {"steps": 1, "tokens": batch.n_tokens, "pages_taken": sum(b - m for b, m in zip(free_before, free_mid)),
                          "pages_freed": sum(a - m for a, m in zip(free_after, free_mid)), "h2d_bytes": batch.h2d_bytes,
                          "graph_steps": int(graph)}
        for key, value in self.last_step.items():
            self.counters[key] += value

    # ------------------------------------------------------- decode graphs
    def _apply_table_updates(self) -> int:
        """Upload and apply queued changes of the block tables and of the requests' records; returns the bytes
        copied to the device."""
        copied = 0
        targets = [group.table_device for group in self.cache.groups] + [self.cache.request_records]
        for target, (index, value) in zip(targets, self.cache.drain_table_updates() + [self.cache.drain_record_updates()]):
            if not index:
                continue
            host = torch.tensor([index, value], dtype=torch.int32).pin_memory()
            dev = host.to(self.cache.device, non_blocking=True)
            ops.scatter_i32(target, dev[0], dev[1])
            copied += host.numel() * 4
        return copied

    def _set_slots(self, g: _DecodeGraph, slots: list[int]) -> int:
        """Make ``g`` run the requests in these slots; returns the bytes copied (none while the set stays)."""
        if g.host_slots == slots:
            return 0
        g.slots.copy_(torch.tensor(slots, dtype=torch.int32).pin_memory(), non_blocking=True)
        g.host_slots = list(slots)
        return 4 * len(slots)

    def _graph_for(self, n: int) -> _DecodeGraph:
        if self._graph_generation != gemm.generation():
            # a weight was bound or a kernel choice changed: captured passes hold what was chosen before
            self._graphs.clear()
            self._graph_generation = gemm.generation()
        if n not in self._graphs:
            self._graphs[n] = _DecodeGraph(n, self.cache.device, self.cache.max_request_tokens)
        return self._graphs[n]

    def _run_decode_graph(self, g: _DecodeGraph) -> torch.Tensor:
        """Logits [n, vocab] for the decode batch described by ``g``'s static buffers."""
        records = self.cache.request_records
        if g.graph is None:
            # First use at this batch size: run once outside a graph (this also does every lazy
            # set-up of libraries and kernels), then capture the same pass for later steps.
            ops.decode_inputs(records, g.slots, g.token_ids, g.positions)
            logits = self.model.forward(g.batch, self.cache)
            torch.cuda.synchronize(self.cache.device)
            before = ops.launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                ops.decode_inputs(records, g.slots, g.token_ids, g.positions)
                g.logits = self.model.forward(g.batch, self.cache)
            g.launches = ops.launch_count() - before
            g.graph = graph
            return logits
        g.graph.replay()
        self.graph_replays += 1
        return g.logits

    def decode_ahead(self, request_ids: Sequence[Hashable]) -> torch.Tensor:
        """One decode step fed from the device: every request's input token is the one the sampler last drew for
        it (``ops.sample_records`` left it in the request's record); the host need not have read it yet.
        Otherwise as :meth:`step` with one token and ``want=(0,)`` per request."""
        cache = self.cache
        if not (self.use_cuda_graphs and self._graph_ok and cache.device.type == "cuda"):
            raise StepError("decode_ahead needs the captured decode pass (a CUDA device, graphs on, no per-request host state)")
        if len(set(request_ids)) != len(request_ids):
            raise StepError("decode_ahead takes distinct requests")
        need = [0] * len(cache.groups)
        for request_id in request_ids:
            if request_id not in cache:
                raise StepError(f"request {request_id!r} is not open")
            if cache.length(request_id) + 1 > self.model.spec.max_positions:
                raise StepError(f"request {request_id!r} is at the model's limit of {self.model.spec.max_positions} positions")
            for g, n in enumerate(cache.pages_needed(request_id, 1)):
                need[g] += n
        for g, (n, f) in enumerate(zip(need, cache.free_pages())):
            if n > f:
                raise OutOfPages(f"the step needs {n} new pages of cache group {g}, {f} are free")
        return self._decode_step([StepEntry(r, (0,), (0,)) for r in request_ids], fed_by_device=True)

    def _decode_step(self, entries: Sequence[StepEntry], fed_by_device: bool = False) -> torch.Tensor:
        cache = self.cache
        n = len(entries)
        g = self._graph_for(n)
        starts = []
        free_before = cache.free_pages()
        for entry in entries:
            if entry.request_id not in cache:
                cache.open(entry.request_id, seed=entry.seed, temperature=entry.temperature)
            starts.append(cache.extend(entry.request_id, 1))
            if not fed_by_device:       # the host names the token (and, for good measure, where it stands)
                cache.set_record(entry.request_id, REC_LAST_TOKEN, int(entry.tokens[0]))
                cache.set_record(entry.request_id, REC_LENGTH, starts[-1])
        slots = [cache.slot(e.request_id) for e in entries]
        g.batch.h2d_bytes = self._set_slots(g, slots) + self._apply_table_updates()
        g.batch.entries = [EntryPlacement(e.request_id, s, i, 1, st) for i, (e, s, st) in enumerate(zip(entries, slots, starts))]
        self.last_batch = g.batch
        free_mid = cache.free_pages()
        logits = self._run_decode_graph(g)
        for entry in entries:
            cache.release_behind_window(entry.request_id)
        self.steps += 1
        self._count(g.batch, free_before, free_mid, True)
        if self.check_errors:
            self.raise_on_device_error()
        return logits

    def decode_loop(self, request_ids: Sequence[Hashable], tokens: Sequence[int], steps: int, *,
                    temperature: Sequence[float] | None = None, seeds: Sequence[int] | None = None) -> torch.Tensor:
        """Decode ``steps`` tokens for each request without a host round trip per token.

        Every request must be open; ``tokens[i]`` is its next input token (the last one drawn, not
        yet in the cache).  Each step runs the captured decode pass, which takes its inputs from the
        requests' records, and draws the next tokens into those records; the host only runs ahead with
        page bookkeeping.  ``temperature`` / ``seeds`` replace the sampling parameters the requests
        were opened with.  Returns the drawn tokens [steps, n] (int32, on the device).  Nothing stops a
        request early.
        """
        cache = self.cache
        n = len(request_ids)
        if not (self._graph_ok and cache.device.type == "cuda"):
            raise StepError("decode_loop needs a CUDA device and a model without per-request host state")
        g = self._graph_for(n)
        for i, request_id in enumerate(request_ids):
            cache.set_record(request_id, REC_LAST_TOKEN, int(tokens[i]))
            cache.set_record(request_id, REC_LENGTH, cache.length(request_id))
            if temperature is not None or seeds is not None:
                cache.set_sampling(request_id, seed=0 if seeds is None else int(seeds[i]),
                                   temperature=0.0 if temperature is None else float(temperature[i]))
        self._set_slots(g, [cache.slot(r) for r in request_ids])
        history = torch.empty((steps, n), dtype=torch.int32, device=cache.device)
        sampled = torch.empty(n, dtype=torch.int32, device=cache.device)
        for step in range(steps):
            for request_id in request_ids:
                cache.extend(request_id, 1)
            self._apply_table_updates()
            logits = self._run_decode_graph(g)
            ops.sample_records(logits, sampled, cache.request_records, g.slots, history[step])
            for request_id in request_ids:
                cache.release_behind_window(request_id)
            self.steps += 1
        return history

    def end(self, request_ids: Iterable[Hashable]) -> None:
        """These requests are finished: what they hold is given back."""
        for request_id in request_ids:
            if request_id in self.cache:
                self.cache.close(request_id)

    def raise_on_device_error(self) -> None:
        word = int(self.cache.error_word.item())
        if word:
            self.cache.error_word.zero_()
            raise StepError(f"a kernel reported an error (code {word:#x}: 0x7c.... a bounded wait of a tcgen05 kernel ran out, "
                            f"else a page id outside its pool); the step's result is invalid")
