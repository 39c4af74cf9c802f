"""Continuous batching above the step function: admit, cut prompts, decode, finish, free.

Reference behaviour this follows:

* a per-step token budget spent on running requests first, then on admissions;
  a decode costs one token, an unfinished prompt ``min(remaining, chunk, budget)``
  (``TokenBudgetScheduler``: src/torchinferno/runtime/scheduler.py:438-609);
* the chunk that completes a prompt is the one that yields the first new token
  (scheduler.py:566-569; src/torchinferno/runtime/serving.py:2666-2681);
* arrival order for admission, head-of-line blocking when the head does not
  fit (src/torchinferno/runtime/paged_serving.py:1300-1305);
* a request ends when it has ``max_new_tokens`` tokens or its last token is a
  stop token, which is still emitted (src/torchinferno/runtime/serving.py:11571-11581).

Where it differs: the reference reserves a request's whole future at admission,
so a live request can never run out of pages and nothing is ever preempted
(paged_serving.py:1321-1322).  Here pages are taken as tokens arrive, which
admits more requests, and **when pages run out the youngest running request is
preempted**: its pages and slot are given back and it returns to the head of the
waiting queue, to be recomputed later from its prompt plus the tokens it had
generated.  Seeded sampling is keyed by position, so the recomputed request
continues exactly as it would have.  A request that could never fit the pool
even alone is refused at submission.

The scheduler is host code over a :class:`CacheManager`; it never touches the
device and is tested on the CPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable

from torchinferno_b200.cache.manager import CacheManager


UNKNOWN_TOKEN = -1   # input token of a step planned ahead: the token the running step is still drawing


@dataclass(eq=False)     # (a request is itself: membership tests and removals go by identity, not by comparing fields)
class SchedulerRequest:
    request_id: Hashable
    prompt: list[int]
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    stop_token_ids: tuple[int, ...] = ()
    # progress
    generated: list[int] = field(default_factory=list)
    computed: int = 0            # tokens of (prompt + generated) whose keys are in the cache
    admitted_at: int = -1        # admission counter; larger is younger
    preemptions: int = 0
    finish_reason: str | None = None
    # The request's record on the device holds its last token: the sampler drew it in the last step that ran the
    # request.  Kept by whoever runs the steps; false again after a preemption, and after a recomputation that ends
    # one token short of the sequence (that token is known, so nothing is drawn for it).
    token_on_device: bool = False

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.generated

    @property
    def prefilling(self) -> bool:
        """More than one token is still to be computed (a prompt or a recomputation)."""
        return self.computed < len(self.prompt) + len(self.generated) - (1 if self.generated else 0)


@dataclass(frozen=True)
class PlannedEntry:
    request_id: Hashable
    tokens: tuple[int, ...]
    start: int                   # position of the first token
    samples: bool                # the step's logits at the last token yield this request's next token
    kind: str                    # "prefill" or "decode"


@dataclass(frozen=True)
class StepPlan:
    step: int
    entries: tuple[PlannedEntry, ...]
    preempted: tuple[Hashable, ...] = ()
    admitted: tuple[Hashable, ...] = ()

    @property
    def scheduled_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


@dataclass(frozen=True)
class TokenEvent:
    request_id: Hashable
    token: int | None
    index: int
    finished: bool
    finish_reason: str | None = None


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batch_size: int = 64, max_step_tokens: int = 8192,
                 prefill_chunk_size: int | None = 2048) -> None:
        if max_batch_size < 1 or max_step_tokens < 1:
            raise ValueError("max_batch_size and max_step_tokens must be positive")
        if prefill_chunk_size is not None and prefill_chunk_size < 1:
            raise ValueError("prefill_chunk_size must be positive")
        self.cache = cache
        self.max_batch_size = min(max_batch_size, cache.max_requests)
        self.max_step_tokens = max_step_tokens
        self.prefill_chunk_size = prefill_chunk_size
        self.waiting: deque[SchedulerRequest] = deque()
        self.running: list[SchedulerRequest] = []
        self._by_id: dict[Hashable, SchedulerRequest] = {}
        self._admissions = 0
        self._step = 0
        self.stats = {"steps": 0, "preemptions": 0, "admitted": 0, "finished": 0,
                      "prefill_tokens": 0, "decode_tokens": 0}

    # ----------------------------------------------------------- requests
    def submit(self, request: SchedulerRequest) -> None:
        if request.request_id in self._by_id:
            raise ValueError(f"duplicate request_id: {request.request_id!r}")
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if request.max_new_tokens < 0:
            raise ValueError("max_new_tokens must be non-negative")
        most = len(request.prompt) + max(0, request.max_new_tokens - 1)  # the last token is never fed back
        if most > self.cache.max_request_tokens:
            raise ValueError(f"request {request.request_id!r} needs room for {most} tokens; "
                             f"the limit per request is {self.cache.max_request_tokens}")
        if -(-most // self.cache.page_size) > self.cache.num_pages:
            raise ValueError(f"request {request.request_id!r} could never fit the cache pool, even alone")
        self._by_id[request.request_id] = request
        self.waiting.append(request)

    def request(self, request_id: Hashable) -> SchedulerRequest | None:
        """The live request of this id (waiting or running), or None once it has finished."""
        return self._by_id.get(request_id)

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def cancel(self, request_id: Hashable) -> TokenEvent | None:
        request = self._by_id.get(request_id)
        if request is None or request.finish_reason is not None:
            return None
        if request in self.running:
            self.running.remove(request)
            if request_id in self.cache:
                self.cache.close(request_id)
        else:
            self.waiting.remove(request)
        return self._finish(request, "cancelled", None)

    # --------------------------------------------------------------- plan
    def plan(self) -> StepPlan:
        """Decide the next step.  Changes only the queues (admission, preemption), never the cache
        of a request that stays: pages are taken when the plan runs."""
        cache = self.cache
        budget = self.max_step_tokens
        room = list(cache.free_pages())          # pages still unclaimed by this plan, per group
        entries: list[PlannedEntry] = []
        preempted: list[Hashable] = []
        admitted: list[Hashable] = []
        planned: set[Hashable] = set()

        def claim(request: SchedulerRequest, n_tokens: int) -> bool:
            known = request.request_id in cache
            need = cache.pages_needed(request.request_id if known else None, n_tokens,
                                      length=None if known else request.computed)
            if any(n > r for n, r in zip(need, room)):
                return False
            for g, n in enumerate(need):
                room[g] -= n
            return True

        def fitting_tokens(request: SchedulerRequest, wanted: int) -> int:
            """The most tokens <= wanted whose pages fit in ``room``."""
            known = request.request_id in cache
            held = cache.length(request.request_id) if known else 0
            best = wanted
            for g, r in enumerate(room):
                pages_held = len(cache.block_table(request.request_id, g)) if known else 0
                capacity = (pages_held + r) * cache.page_size - held
                best = min(best, capacity)
            return max(0, best)

        def preempt_youngest(protect: SchedulerRequest | None) -> bool:
            """Give back the pages of the youngest running request that is not yet planned."""
            candidates = [r for r in self.running if r.request_id not in planned and r is not protect]
            if not candidates:
                candidates = [r for r in self.running if r.request_id not in planned]
            if not candidates:
                return False
            victim = max(candidates, key=lambda r: r.admitted_at)
            self.running.remove(victim)
            if victim.request_id in cache:
                freed_before = cache.free_pages()
                cache.close(victim.request_id)
                for g, (after, before) in enumerate(zip(cache.free_pages(), freed_before)):
                    room[g] += after - before
            victim.computed = 0
            victim.preemptions += 1
            victim.token_on_device = False
            self.waiting.appendleft(victim)
            preempted.append(victim.request_id)
            self.stats["preemptions"] += 1
            return True

        # 1. running requests, oldest first: decodes cost one token, unfinished prompts a portion
        for request in sorted(self.running, key=lambda r: r.admitted_at):
            if request not in self.running or budget <= 0:
                continue
            if not request.prefilling:
                fits = claim(request, 1)
                while not fits:
                    if not preempt_youngest(protect=request) or request not in self.running:
                        break
                    fits = claim(request, 1)
                if not fits:
                    continue
                entries.append(PlannedEntry(request.request_id, (request.tokens[-1],), request.computed, True, "decode"))
                planned.add(request.request_id)
                budget -= 1
            else:
                entry = self._portion(request, budget, fitting_tokens, claim)
                if entry is not None:
                    entries.append(entry)
                    planned.add(request.request_id)
                    budget -= len(entry.tokens)

        # 2. admissions in arrival order; the head of the queue blocks those behind it
        while self.waiting and budget > 0 and len(self.running) < self.max_batch_size and cache.free_slots() > len(admitted):
            request = self.waiting[0]
            entry = self._portion(request, budget, fitting_tokens, claim)
            if entry is None:
                break
            self.waiting.popleft()
            request.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(request)
            admitted.append(request.request_id)
            self.stats["admitted"] += 1
            entries.append(entry)
            planned.add(request.request_id)
            budget -= len(entry.tokens)

        # 3. nothing can move although requests are running: free the youngest and try again next step
        if not entries and self.running:
            preempt_youngest(protect=None)

        plan = StepPlan(self._step, tuple(entries), tuple(preempted), tuple(admitted))
        self._step += 1
        return plan

    def _portion(self, request: SchedulerRequest, budget: int, fitting_tokens, claim) -> PlannedEntry | None:
        tokens = request.tokens
        # everything but a pending last generated token is "prompt" for the cache
        target = len(tokens)
        remaining = target - request.computed
        count = min(remaining, budget)
        if self.prefill_chunk_size is not None:
            count = min(count, self.prefill_chunk_size)
        count = min(count, fitting_tokens(request, count))
        if count <= 0 or not claim(request, count):
            return None
        start = request.computed
        chunk = tuple(tokens[start:start + count])
        completes = start + count == target
        return PlannedEntry(request.request_id, chunk, start, completes, "prefill")

    # ---------------------------------------------------------- run ahead
    def plan_ahead(self, running: StepPlan) -> StepPlan | None:
        """The step after ``running``, decided before ``running``'s tokens are known, or None.

        ``running`` has been launched but not committed.  If every running request draws a token
        in it and goes on afterwards unless that token is a stop token, the next step is a decode
        of the same requests in the same order, whose input tokens exist only on the device yet:
        each entry carries ``UNKNOWN_TOKEN``.  Anything that needs a decision (a request waiting, a
        request that ends by length, pages that would run out) returns None: the caller then
        commits ``running`` first and plans as usual.  A request that does stop in ``running`` has
        been run one token too far; :meth:`commit` skips its entry.
        """
        if self.waiting or not running.entries or len(running.entries) != len(self.running):
            return None
        need = [0] * len(self.cache.free_pages())
        entries = []
        live = {id(r) for r in self.running}
        for entry in running.entries:
            request = self._by_id.get(entry.request_id)
            if (request is None or id(request) not in live or not entry.samples
                    or len(request.generated) + 2 > request.max_new_tokens
                    or entry.request_id not in self.cache
                    or self.cache.length(entry.request_id) != entry.start + len(entry.tokens)):
                return None
            for g, n in enumerate(self.cache.pages_needed(entry.request_id, 1)):
                need[g] += n
            entries.append(PlannedEntry(entry.request_id, (UNKNOWN_TOKEN,), entry.start + len(entry.tokens), True, "decode"))
        if any(n > f for n, f in zip(need, self.cache.free_pages())):
            return None
        plan = StepPlan(self._step, tuple(entries))
        self._step += 1
        return plan

    # ------------------------------------------------------------- commit
    def commit(self, plan: StepPlan, sampled: dict[Hashable, int]) -> list[TokenEvent]:
        """Record what the step computed and the tokens drawn; finish and free what is done.
        Entries of requests that ended since the plan was made (a stop token or a cancellation
        while a step planned ahead was running) are skipped."""
        events: list[TokenEvent] = []
        for entry in plan.entries:
            request = self._by_id.get(entry.request_id)
            if request is None or request.finish_reason is not None:
                continue
            request.computed = entry.start + len(entry.tokens)
            self.stats["decode_tokens" if entry.kind == "decode" else "prefill_tokens"] += len(entry.tokens)
            if not entry.samples:
                continue
            if request.max_new_tokens == 0:
                events.append(self._retire(request, "length", None))
                continue
            token = int(sampled[entry.request_id])
            request.generated.append(token)
            index = len(request.generated) - 1
            if token in request.stop_token_ids:
                events.append(self._retire(request, "stop", token))
            elif len(request.generated) >= request.max_new_tokens:
                events.append(self._retire(request, "length", token))
            else:
                events.append(TokenEvent(request.request_id, token, index, False))
        self.stats["steps"] += 1
        return events

    def _retire(self, request: SchedulerRequest, reason: str, token: int | None) -> TokenEvent:
        if request in self.running:
            self.running.remove(request)
        if request.request_id in self.cache:
            self.cache.close(request.request_id)
        return self._finish(request, reason, token)

    def _finish(self, request: SchedulerRequest, reason: str, token: int | None) -> TokenEvent:
        request.finish_reason = reason
        self.stats["finished"] += 1
        del self._by_id[request.request_id]
        return TokenEvent(request.request_id, token, max(0, len(request.generated) - 1), True, reason)
