"""The Python entry point: ``InferenceEngine`` over scheduler, step function and sampler.

Interface as in the reference (src/torchinferno/engine/engine.py:35-54, 91-151):
``InferenceEngine.from_config(EngineConfig)``, ``generate(request)``,
``generate_stream(request)``, ``cancel(request_id)``, ``close()``, context
manager.  ``generate_many`` runs several requests together through the
continuous-batching scheduler.  Tokens go in and come out as host integers;
text prompts need a tokenizer (``EngineConfig.tokenizer`` or the model folder's
``tokenizer.json``, through the optional ``tokenizers`` package as in
src/torchinferno/tokenization.py:7-61).
"""
from __future__ import annotations

from pathlib import Path
from typing import Hashable, Iterable, Iterator, Sequence

import torch

from torchinferno_b200.config import registry
from torchinferno_b200.config.engine_config import EngineConfig
from torchinferno_b200.config.model_config import read_config_json
from torchinferno_b200.engine.batch import StepEntry
from torchinferno_b200.engine.factory import load_model, make_runner
from torchinferno_b200.engine.runner import StepError
from torchinferno_b200.engine.scheduler import Scheduler, SchedulerRequest, StepPlan, TokenEvent, UNKNOWN_TOKEN
from torchinferno_b200.kernels import gemm, ops
from torchinferno_b200.engine.types import GenerateOutput, GenerateRequest, SamplingConfig, TokenOutput, Usage
from torchinferno_b200.sampling.sampler import Sampler, SamplingParams


class _Launched:
    """A step that runs on the device: its plan, the drawn tokens there and on their way to the host."""

    def __init__(self, plan: StepPlan, requests: list, drawing: list, device_tokens: torch.Tensor | None,
                 error_word: torch.Tensor) -> None:
        self.plan, self.requests, self.drawing, self.device_tokens = plan, requests, drawing, device_tokens
        self.host_tokens: torch.Tensor | None = None
        self.arrived: torch.cuda.Event | None = None
        if device_tokens is not None and device_tokens.numel():
            # the tokens and, behind them, the kernels' error word (a page id outside its pool, a bounded wait
            # that ran out): one more small copy instead of a synchronising read after every step
            self.host_tokens = torch.empty(device_tokens.numel() + 1, dtype=torch.int32, pin_memory=True)
            self.host_tokens[:-1].copy_(device_tokens.reshape(-1), non_blocking=True)
            self.host_tokens[-1:].copy_(error_word.reshape(-1)[:1], non_blocking=True)
            self.arrived = torch.cuda.Event()
            self.arrived.record()

    def tokens(self) -> dict[Hashable, int]:
        """Wait for the copy to the host and return {request: token}."""
        if self.host_tokens is None:
            return {}
        self.arrived.synchronize()
        *tokens, error = self.host_tokens.tolist()
        if error:
            raise StepError(f"a kernel reported an error during the step (code {error:#x}); its tokens are invalid")
        return {e.request_id: int(t) for e, t in zip(self.drawing, tokens)}


class InferenceEngine:
    def __init__(self, model, config: EngineConfig, tokenizer=None) -> None:
        self.model = model
        self.config = config
        self.tokenizer = tokenizer
        limit = model.spec.max_positions if config.max_model_len is None else min(config.max_model_len, model.spec.max_positions)
        if config.num_pages is not None:
            num_pages = config.num_pages
        else:
            tokens = config.kv_cache_tokens or _default_cache_tokens(model, config, limit)
            num_pages = -(-tokens // config.page_size) + config.max_batch_size
        self.runner = make_runner(model, page_size=config.page_size, num_pages=num_pages,
                                  max_requests=config.max_batch_size, max_request_tokens=limit, check_errors=False)
        self.runner.use_cuda_graphs = config.use_cuda_graphs and not config.profile_kernels
        if config.profile_kernels:
            ops.set_kernel_timers(True)
        gemm.set_backend(config.gemm_backend)
        self.scheduler = Scheduler(self.runner.cache, max_batch_size=config.max_batch_size,
                                   max_step_tokens=config.max_num_batched_tokens,
                                   prefill_chunk_size=config.prefill_chunk_size)
        self.sampler = Sampler(model.device)
        self._requests: dict[Hashable, GenerateRequest] = {}
        self._cancelled: set[Hashable] = set()
        self._closed = False
        self._ahead: _Launched | None = None      # a step launched before the one before it was committed
        self.stats = {"steps": 0, "steps_ahead": 0, "tokens": 0, "h2d_bytes": 0, "d2h_bytes": 0}

    # -------------------------------------------------------- construction
    @classmethod
    def from_config(cls, config: EngineConfig) -> "InferenceEngine":
        wanted = None
        if config.model_kind != "auto":
            wanted = registry.entry_for_kind(config.model_kind)
            if wanted is None:
                raise ValueError(f"model_kind={config.model_kind!r} is not registered; 'auto' or one of {list(registry.known_kinds())}")
        gemm.set_backend(config.gemm_backend)   # decides the layout the weights are bound in
        gemm.set_few_rows_choice(config.few_rows_choice)
        if wanted is not None:
            named = registry.resolve_architecture(read_config_json(config.model))
            if named is not wanted:
                raise ValueError(f"model_kind={config.model_kind!r} names {wanted.name}, but {config.model}/config.json names {named.name}")
        model = load_model(config.model, dtype=config.dtype, device=config.device or "cuda:0")
        return cls(model, config, _load_tokenizer(config))

    def __enter__(self) -> "InferenceEngine":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def warm_up(self, batch_sizes: Iterable[int] | None = None) -> list[int]:
        """Capture the decode step for these numbers of running requests (default: every number up to
        ``max_batch_size``) now instead of at the first step that meets them: a decode step is captured per exact
        batch size (no padded rows), and a capture in the middle of serving costs that step several times its
        usual time.  Runs throw-away requests of two tokens each; needs the cache empty.  Returns the sizes captured."""
        runner, cache = self.runner, self.runner.cache
        if cache.live_requests or self.scheduler.has_work():
            raise RuntimeError("warm_up needs an idle engine")
        if not (runner.use_cuda_graphs and runner._graph_ok and cache.device.type == "cuda"):
            return []
        sizes = sorted({int(n) for n in (batch_sizes if batch_sizes is not None else range(1, self.config.max_batch_size + 1))
                        if 1 <= int(n) <= min(self.config.max_batch_size, cache.max_requests)}, reverse=True)
        done = []
        with torch.inference_mode():
            for n in sizes:
                if any(n > free for free in cache.free_pages()):      # (a page per request is the least it takes)
                    continue
                ids = [("warm-up", i) for i in range(n)]
                runner.step([StepEntry(r, (0,), ()) for r in ids])           # one token each, then a decode step of n
                runner.step([StepEntry(r, (0,), (0,)) for r in ids])
                runner.step([StepEntry(r, (0,), (0,)) for r in ids])         # (the second one replays the captured step)
                runner.end(ids)
                done.append(n)
            torch.cuda.synchronize(cache.device)
        if cache.error_word is not None:
            cache.error_word.zero_()
        return done

    def kernel_times(self, reset: bool = False) -> dict[str, dict[str, float]]:
        """With ``profile_kernels``: milliseconds and launches per kernel class of the layers run so far (norm, qkv,
        rope_append, attention_prefill, attention_decode, o, gate_up, swiglu, down); and the step counters."""
        return {**ops.read_kernel_timers(reset), "counters": dict(self.runner.counters)}

    def close(self) -> None:
        if self._closed:
            return
        if self.config.profile_kernels:
            ops.set_kernel_timers(False)
        for request_id in list(self._requests):
            self.cancel(request_id)
        self._ahead = None
        self._closed = True

    # ------------------------------------------------------------ requests
    def _prompt_ids(self, request: GenerateRequest) -> list[int]:
        if request.prompt_token_ids is not None:
            return list(request.prompt_token_ids)
        if self.tokenizer is None:
            raise ValueError("a text prompt needs a tokenizer; give prompt_token_ids or EngineConfig.tokenizer")
        if request.prompt is not None:
            return list(self.tokenizer.encode(request.prompt).ids)
        text = "".join(f"{m.get('role', 'user')}: {m.get('content', '')}\n" for m in request.messages)
        return list(self.tokenizer.encode(text).ids)

    def _decode(self, ids: Sequence[int]) -> str:
        return "" if self.tokenizer is None or not ids else self.tokenizer.decode(list(ids))

    def submit(self, request: GenerateRequest) -> None:
        if self._closed:
            raise RuntimeError("the engine is closed")
        prompt = self._prompt_ids(request)
        sampling = request.sampling
        self.scheduler.submit(SchedulerRequest(
            request.request_id, prompt, sampling.max_tokens, sampling.temperature,
            sampling.seed if sampling.seed else self.config.seed, sampling.stop_token_ids))
        self._requests[request.request_id] = request

    def cancel(self, request_id: Hashable) -> bool:
        """Stop a request; its pages are given back (src/torchinferno/engine/engine.py:87-89)."""
        if request_id not in self._requests:
            return False
        self._cancelled.add(request_id)
        self.scheduler.cancel(request_id)
        self._requests.pop(request_id, None)
        return True

    # ---------------------------------------------------------------- step
    def step(self) -> list[TokenEvent]:
        """Plan one step, run it, draw tokens, and return what happened.

        With ``async_scheduling`` a decode step whose successor needs no decision (the same
        requests go on, pages suffice, nobody waits) has that successor launched before its own
        tokens are read: the device feeds the drawn tokens to the next step itself, and the host
        reads them while that step runs.  A request that draws a stop token has then been run one
        token too far; that row is dropped.
        """
        current, self._ahead = self._ahead, None
        if current is not None:
            # requests that ended while the step ran (a stop token, a cancellation) drop out of it
            live = tuple(e for e, r in zip(current.plan.entries, current.requests)
                         if self.scheduler.request(e.request_id) is r)
            if not live:
                current = None
            elif len(live) < len(current.plan.entries):
                current.plan = StepPlan(current.plan.step, live)
        if current is None:
            plan = self.scheduler.plan()
            if not plan.entries:
                return []
            current = self._launch(_longest_first(plan), False)
        if self.config.async_scheduling and current.device_tokens is not None and self.runner.use_cuda_graphs:
            ahead = self.scheduler.plan_ahead(current.plan)
            if ahead is not None and len(current.drawing) == len(ahead.entries):
                self._ahead = self._launch(_longest_first(ahead), True)
                self.stats["steps_ahead"] += 1
        try:
            tokens = current.tokens()
        except StepError:
            self._abandon(current.plan)
            raise
        return self.scheduler.commit(current.plan, tokens)

    def _launch(self, plan: StepPlan, ahead: bool) -> _Launched:
        """Start a step on the device.  ``ahead``: the plan was made before the tokens of the step before it
        were read; they are on the device, in the requests' records."""
        runner, cache = self.runner, self.runner.cache
        with torch.inference_mode():
            # a step of decoded tokens only takes its inputs from the requests' records on the device, where the
            # sampler left them: nothing but new block-table entries is copied.  (Not every decoded token is there: a
            # recomputation after a preemption may end one token short of the sequence, and that last token, which
            # the host knows, was never drawn on the device since.)
            requests = [self.scheduler.request(e.request_id) for e in plan.entries]
            fed_by_device = ahead or (runner.use_cuda_graphs and runner._graph_ok
                                      and all(e.kind == "decode" and e.request_id in cache and r is not None and r.token_on_device
                                              for e, r in zip(plan.entries, requests)))
            try:
                if fed_by_device:
                    logits = runner.decode_ahead([e.request_id for e in plan.entries])
                else:
                    assert all(t != UNKNOWN_TOKEN for e in plan.entries for t in e.tokens)
                    entries = []
                    for e in plan.entries:
                        request = self.scheduler.request(e.request_id)
                        entries.append(StepEntry(e.request_id, e.tokens, (len(e.tokens) - 1,) if e.samples else (),
                                                 seed=request.seed, temperature=request.temperature))
                    logits = runner.step(entries)
            except StepError:
                self._abandon(plan)
                raise
            batch = runner.last_batch
            for planned, placed in zip(plan.entries, batch.entries):
                if placed.kv_start != planned.start:
                    self._abandon(plan)
                    raise StepError(f"request {planned.request_id!r} was planned at position {planned.start} "
                                    f"but its cache stands at {placed.kv_start}")
            self.stats["steps"] += 1
            self.stats["h2d_bytes"] += batch.h2d_bytes
            self.stats["tokens"] += batch.n_tokens
            drawing = [e for e in plan.entries if e.samples]
            for e, r in zip(plan.entries, requests):
                if r is not None:
                    r.token_on_device = e.samples      # (the sampler below leaves the token it draws in the record)
            if not drawing:
                return _Launched(plan, requests, [], None, cache.error_word)
            tokens = self.sampler.sample_records(logits, cache.request_records, batch.logit_slots)
            self.stats["d2h_bytes"] += tokens.numel() * tokens.element_size() + 4    # (and the error word)
            return _Launched(plan, requests, drawing, tokens, cache.error_word)

    def _abandon(self, plan: StepPlan | None) -> None:
        """A step failed: its requests (and those of a step launched ahead) are cancelled and give back what
        they hold, and the device's error word is cleared, so that the engine can go on with the rest."""
        ahead, self._ahead = self._ahead, None
        for p in (plan, None if ahead is None else ahead.plan):
            for entry in (() if p is None else p.entries):
                self.scheduler.cancel(entry.request_id)
                self._requests.pop(entry.request_id, None)
        if self.runner.cache.error_word is not None:
            self.runner.cache.error_word.zero_()

    # ------------------------------------------------------------ generate
    def generate_stream(self, request: GenerateRequest) -> Iterator[TokenOutput]:
        """Yield one ``TokenOutput`` per token, then a final one with ``finished`` and ``usage``."""
        self.submit(request)
        prompt_tokens = len(self.scheduler.request(request.request_id).prompt)
        emitted: list[int] = []
        reason = None
        while reason is None:
            if request.request_id in self._cancelled:
                reason = "cancelled"
                break
            for event in self.step():
                if event.request_id != request.request_id:
                    continue
                if event.token is not None:
                    emitted.append(event.token)
                    yield TokenOutput(request.request_id, event.token, self._decode([event.token]), len(emitted) - 1)
                if event.finished:
                    reason = event.finish_reason
            if reason is None and not self.scheduler.has_work():
                reason = "cancelled" if request.request_id in self._cancelled else "length"
        self._requests.pop(request.request_id, None)
        self._cancelled.discard(request.request_id)
        yield TokenOutput(request.request_id, None, "", len(emitted), True, reason, Usage(prompt_tokens, len(emitted)))

    def generate(self, request: GenerateRequest) -> GenerateOutput:
        tokens: list[int] = []
        final = None
        for out in self.generate_stream(request):
            if out.finished:
                final = out
            elif out.token_id is not None:
                tokens.append(out.token_id)
        return GenerateOutput(request.request_id, tuple(tokens), self._decode(tokens), final.finish_reason, final.usage)

    def generate_many(self, requests: Iterable[GenerateRequest]) -> list[GenerateOutput]:
        """Run requests together (continuous batching); results in the order given."""
        requests = list(requests)
        for request in requests:
            self.submit(request)
        prompts = {r.request_id: len(self.scheduler.request(r.request_id).prompt) for r in requests}
        tokens: dict[Hashable, list[int]] = {r.request_id: [] for r in requests}
        reasons: dict[Hashable, str] = {}
        while len(reasons) < len(requests) and self.scheduler.has_work():
            for event in self.step():
                if event.request_id not in tokens:
                    continue
                if event.token is not None:
                    tokens[event.request_id].append(event.token)
                if event.finished:
                    reasons[event.request_id] = event.finish_reason
        outputs = []
        for r in requests:
            self._requests.pop(r.request_id, None)
            ids = tokens[r.request_id]
            outputs.append(GenerateOutput(r.request_id, tuple(ids), self._decode(ids),
                                          reasons.get(r.request_id, "cancelled"), Usage(prompts[r.request_id], len(ids))))
        return outputs


def _longest_first(plan: StepPlan) -> StepPlan:
    """A step of decoded tokens only, longest context first: the decode attention kernel gives every (request, kv
    head) a block, the hardware hands blocks out in order, and a long context that starts last is the step's tail.
    (The order is stable from step to step, so the captured step's slots stay as they are.)"""
    if len(plan.entries) < 2 or any(e.kind != "decode" for e in plan.entries):
        return plan
    ordered = tuple(sorted(plan.entries, key=lambda e: -e.start))
    return plan if ordered == plan.entries else StepPlan(plan.step, ordered, plan.preempted, plan.admitted)


def _default_cache_tokens(model, config: EngineConfig, limit: int) -> int:
    """The pool when no size is given: room for every request at its longest, but no more than
    ``cache_memory_fraction`` of the device memory that is free once the weights are loaded (the reference sizes
    its pool as max_active x ceil(max_seq / page) + 8 pages whatever that costs:
    src/torchinferno/runtime/paged_serving.py:749-752)."""
    wanted = config.max_batch_size * limit
    if model.device.type != "cuda":
        return wanted
    per_token = sum(spec.elements_per_token for spec in model.cache_requirements()) * torch.empty((), dtype=model.dtype).element_size()
    free, _ = torch.cuda.mem_get_info(model.device)
    fits = int(free * config.cache_memory_fraction) // max(1, per_token)
    if fits < config.page_size:
        raise RuntimeError(f"no room for a cache: {free / 2**30:.1f} GiB are free and a token takes {per_token} bytes")
    return min(wanted, fits)


def _load_tokenizer(config: EngineConfig):
    path = config.tokenizer
    if path is None:
        candidate = Path(config.model) / "tokenizer.json"
        if not candidate.is_file():
            return None
        path = str(candidate)
    elif Path(path).is_dir():
        path = str(Path(path) / "tokenizer.json")
    try:
        from tokenizers import Tokenizer
    except ImportError as exc:
        raise RuntimeError("text prompts need the optional 'tokenizers' package") from exc
    return Tokenizer.from_file(path)


def generate(model_dir: str, prompt_token_ids: Sequence[int], *, max_new_tokens: int = 16, temperature: float = 0.0,
             seed: int = 0, dtype: str = "auto", stop_token_ids: Sequence[int] = (), **engine_options) -> list[int]:
    """One call from a model folder and prompt ids to new token ids (the shape of the reference's
    ``model.generate(input_ids, max_new_tokens=, temperature=)``: src/torchinferno/models/llama3/pipeline.py:404-433)."""
    config = EngineConfig(model=str(model_dir), dtype=dtype, **engine_options)
    with InferenceEngine.from_config(config) as engine:
        out = engine.generate(GenerateRequest("generate-0", prompt_token_ids=list(prompt_token_ids),
                                              sampling=SamplingConfig(max_new_tokens, temperature, tuple(stop_token_ids), seed)))
    return list(out.token_ids)
