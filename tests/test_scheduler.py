"""The scheduler's decisions on the CPU: portions under a token budget, decode first, admission,
finishing, and what happens when pages run out (the youngest running request is preempted and
recomputed).  A fake step function stands in for the model: the next token is a function of the
request's whole token sequence, so a recomputed request must continue as if nothing had happened."""
import torch

import pytest

from torchinferno_b200.cache.manager import CacheManager
from torchinferno_b200.engine.scheduler import Scheduler, SchedulerRequest
from torchinferno_b200.parts.base import CacheSpec


def make(num_pages=16, page_size=4, max_requests=4, max_request_tokens=64, **kw):
    cache = CacheManager([CacheSpec(1, 8)], [None], page_size=page_size, num_pages=num_pages, max_requests=max_requests,
                         max_request_tokens=max_request_tokens, dtype=torch.float32, device="cpu", allocate_tensors=False)
    return cache, Scheduler(cache, **kw)


def next_token(tokens):
    return (sum(tokens) * 31 + len(tokens) * 7) % 101


def run_plan(cache, sched, plan, seen):
    """What the step function does to the cache, and a deterministic 'model'."""
    sampled = {}
    for entry in plan.entries:
        if entry.request_id not in cache:
            cache.open(entry.request_id)
        assert cache.extend(entry.request_id, len(entry.tokens)) == entry.start
        seen.setdefault(entry.request_id, {})
        for i, tok in enumerate(entry.tokens):
            seen[entry.request_id][entry.start + i] = tok
        if entry.samples:
            history = [seen[entry.request_id][p] for p in range(entry.start + len(entry.tokens))]
            sampled[entry.request_id] = next_token(history)
    cache.audit()
    return sampled


def drive(cache, sched, max_steps=500):
    seen, outputs, plans = {}, {}, []
    for _ in range(max_steps):
        if not sched.has_work():
            break
        plan = sched.plan()
        plans.append(plan)
        for rid in plan.preempted:
            seen.pop(rid, None)
        for event in sched.commit(plan, run_plan(cache, sched, plan, seen)):
            if event.token is not None:
                outputs.setdefault(event.request_id, []).append(event.token)
            if event.finished:
                outputs.setdefault(event.request_id, [])
                outputs[event.request_id].append(event.finish_reason)
    assert not sched.has_work(), "the scheduler did not finish"
    return outputs, plans


def expected(prompt, n, stop=()):
    toks, out = list(prompt), []
    for _ in range(n):
        t = next_token(toks)
        toks.append(t), out.append(t)
        if t in stop:
            return out + ["stop"]
    return out + ["length"]


def test_prompt_is_cut_under_chunk_and_budget_and_emits_once_complete():
    cache, sched = make(max_step_tokens=8, prefill_chunk_size=5)
    sched.submit(SchedulerRequest("a", list(range(12)), 3))
    outputs, plans = drive(cache, sched)
    shape = [[(e.kind, e.start, len(e.tokens), e.samples) for e in p.entries] for p in plans]
    assert shape == [[("prefill", 0, 5, False)], [("prefill", 5, 5, False)], [("prefill", 10, 2, True)],
                     [("decode", 12, 1, True)], [("decode", 13, 1, True)]]
    assert outputs["a"] == expected(range(12), 3)
    assert cache.free_pages() == [16] and not cache.live_requests


def test_decode_goes_before_waiting_prefill_and_budget_is_shared():
    cache, sched = make(max_step_tokens=6, prefill_chunk_size=None)
    sched.submit(SchedulerRequest("a", [1, 2, 3], 4))
    plan0 = sched.plan()
    sched.commit(plan0, run_plan(cache, sched, plan0, s := {}))
    sched.submit(SchedulerRequest("b", list(range(9)), 2))
    plan1 = sched.plan()
    assert [(e.request_id, e.kind, len(e.tokens)) for e in plan1.entries] == [("a", "decode", 1), ("b", "prefill", 5)]
    assert plan1.admitted == ("b",) and plan1.scheduled_tokens == 6
    sched.commit(plan1, run_plan(cache, sched, plan1, s))
    plan2 = sched.plan()
    assert [(e.request_id, e.kind, e.start, len(e.tokens), e.samples) for e in plan2.entries] == \
        [("a", "decode", 4, 1, True), ("b", "prefill", 5, 4, True)]


def test_stop_token_is_emitted_and_ends_the_request():
    cache, sched = make()
    prompt = [5, 6, 7]
    want = expected(prompt, 6)
    stop = want[2]
    sched.submit(SchedulerRequest("a", prompt, 6, stop_token_ids=(stop,)))
    outputs, _ = drive(cache, sched)
    assert outputs["a"] == want[:3] + ["stop"] == expected(prompt, 6, (stop,))


def test_zero_and_one_new_tokens():
    cache, sched = make()
    sched.submit(SchedulerRequest("z", [1, 2], 0))
    sched.submit(SchedulerRequest("o", [1, 2], 1))
    outputs, plans = drive(cache, sched)
    assert outputs["z"] == ["length"] and outputs["o"] == expected([1, 2], 1) and len(plans) == 1


def test_admission_is_in_arrival_order_and_limited_by_rows():
    cache, sched = make(max_requests=2, max_batch_size=2, max_step_tokens=64)
    for name in "abc":
        sched.submit(SchedulerRequest(name, [1, 2, 3], 2))
    plan = sched.plan()
    assert plan.admitted == ("a", "b") and [e.request_id for e in plan.entries] == ["a", "b"]
    sched.commit(plan, run_plan(cache, sched, plan, s := {}))
    plan = sched.plan()                      # a and b finish with their second token
    sched.commit(plan, run_plan(cache, sched, plan, s))
    plan = sched.plan()
    assert plan.admitted == ("c",)


def test_head_of_queue_blocks_when_its_first_portion_has_no_page():
    cache, sched = make(num_pages=4, page_size=4, max_step_tokens=64, prefill_chunk_size=None)
    sched.submit(SchedulerRequest("a", list(range(14)), 2))          # takes all four pages
    plan = sched.plan()
    sched.commit(plan, run_plan(cache, sched, plan, s := {}))
    sched.submit(SchedulerRequest("b", [1] * 6, 1))
    sched.submit(SchedulerRequest("c", [1], 1))
    plan = sched.plan()
    assert plan.admitted == () and [e.request_id for e in plan.entries] == ["a"]


def test_a_prompt_portion_shrinks_to_the_pages_that_are_free():
    cache, sched = make(num_pages=5, page_size=4, max_step_tokens=64, prefill_chunk_size=None)
    sched.submit(SchedulerRequest("a", list(range(11)), 6))          # three pages
    plan = sched.plan()
    sched.commit(plan, run_plan(cache, sched, plan, s := {}))
    sched.submit(SchedulerRequest("b", list(range(20)), 1))
    plan = sched.plan()                                              # a decodes within its third page
    assert [(e.request_id, len(e.tokens)) for e in plan.entries] == [("a", 1), ("b", 8)]


def test_running_out_of_pages_preempts_the_youngest_which_is_recomputed():
    cache, sched = make(num_pages=6, page_size=4, max_step_tokens=64, prefill_chunk_size=None)
    prompts = {"old": list(range(1, 8)), "young": list(range(20, 29))}
    sched.submit(SchedulerRequest("old", prompts["old"], 14))
    sched.submit(SchedulerRequest("young", prompts["young"], 10))
    outputs, plans = drive(cache, sched)
    assert sched.stats["preemptions"] >= 1
    assert all(p.preempted in ((), ("young",)) for p in plans)       # never the older request
    first = next(i for i, p in enumerate(plans) if p.preempted)
    # the preempted request comes back later as one prefill over prompt + what it had generated
    back = next(e for p in plans[first:] for e in p.entries if e.request_id == "young" and e.kind == "prefill")
    assert back.start == 0 and len(back.tokens) > len(prompts["young"])
    assert outputs["old"] == expected(prompts["old"], 14)
    assert outputs["young"] == expected(prompts["young"], 10)        # same tokens as without preemption
    assert cache.free_pages() == [6]


def test_many_requests_on_a_small_pool_all_finish_with_the_right_tokens():
    cache, sched = make(num_pages=10, page_size=4, max_requests=4, max_step_tokens=16, prefill_chunk_size=6)
    wants = {}
    for i in range(9):
        prompt = [(i * 13 + j) % 97 for j in range(3 + 4 * (i % 4))]
        sched.submit(SchedulerRequest(i, prompt, 5 + i % 3))
        wants[i] = expected(prompt, 5 + i % 3)
    outputs, plans = drive(cache, sched, max_steps=2000)
    assert outputs == wants
    assert all(p.scheduled_tokens <= 16 for p in plans)
    assert all(len(e.tokens) <= 6 for p in plans for e in p.entries if e.kind == "prefill")
    assert cache.free_pages() == [10] and sched.stats["finished"] == 9


def test_requests_that_can_never_fit_are_refused_at_submission():
    cache, sched = make(num_pages=3, page_size=4, max_request_tokens=64)
    with pytest.raises(ValueError, match="never fit"):
        sched.submit(SchedulerRequest("big", [1] * 10, 5))
    cache, sched = make(max_request_tokens=8)
    with pytest.raises(ValueError, match="limit per request"):
        sched.submit(SchedulerRequest("long", [1] * 8, 2))
    with pytest.raises(ValueError, match="prompt token"):
        sched.submit(SchedulerRequest("empty", [], 2))
    sched.submit(SchedulerRequest("ok", [1], 2))
    with pytest.raises(ValueError, match="duplicate"):
        sched.submit(SchedulerRequest("ok", [1], 2))


def test_cancel_frees_pages_and_row():
    cache, sched = make()
    sched.submit(SchedulerRequest("a", [1, 2, 3, 4, 5], 50))
    sched.submit(SchedulerRequest("b", [1], 50))
    plan = sched.plan()
    sched.commit(plan, run_plan(cache, sched, plan, {}))
    event = sched.cancel("a")
    assert event.finished and event.finish_reason == "cancelled" and "a" not in cache
    assert sched.cancel("a") is None
    sched.cancel("b")
    assert cache.free_pages() == [16] and not sched.has_work()


def drive_ahead(cache, sched, max_steps=500):
    """As ``drive``, but as the engine does with async scheduling: the next step is planned and 'launched'
    before the running one is committed, whenever ``plan_ahead`` allows it."""
    from torchinferno_b200.engine.scheduler import UNKNOWN_TOKEN
    seen, outputs, ahead_steps = {}, {}, 0
    launched = None            # (plan, sampled) of a step that runs but is not yet committed
    for _ in range(max_steps):
        if launched is None:
            if not sched.has_work():
                break
            plan = sched.plan()
            for rid in plan.preempted:
                seen.pop(rid, None)
            launched = (plan, run_plan(cache, sched, plan, seen))
        plan, sampled = launched
        launched = None
        ahead = sched.plan_ahead(plan)
        if ahead is not None:
            ahead_steps += 1
            assert [e.request_id for e in ahead.entries] == [e.request_id for e in plan.entries]
            assert all(e.tokens == (UNKNOWN_TOKEN,) for e in ahead.entries)
            # the device feeds the drawn tokens in; the fake model does the same
            fed = type(ahead)(ahead.step, tuple(type(e)(e.request_id, (sampled[e.request_id],), e.start, True, "decode")
                                                for e in ahead.entries))
            launched = (ahead, run_plan(cache, sched, fed, seen))
        for event in sched.commit(plan, sampled):
            if event.token is not None:
                outputs.setdefault(event.request_id, []).append(event.token)
            if event.finished:
                outputs.setdefault(event.request_id, []).append(event.finish_reason)
        if launched is not None and not any(sched.request(e.request_id) is not None for e in launched[0].entries):
            launched = None
        cache.audit()
    assert not sched.has_work(), "the scheduler did not finish"
    return outputs, ahead_steps


def test_planning_ahead_gives_the_same_tokens_and_skips_a_request_that_stopped():
    prompts = {"a": [3, 1, 4, 1, 5], "b": [9, 2, 6], "c": [5, 3, 5, 8, 9, 7]}
    stop = (expected(prompts["b"], 6)[3],)          # b stops at its fourth token, mid-flight
    want = {"a": expected(prompts["a"], 9), "b": expected(prompts["b"], 9, stop), "c": expected(prompts["c"], 7)}
    assert want["b"][-1] == "stop"
    cache, sched = make(num_pages=32)
    for rid, prompt in prompts.items():
        sched.submit(SchedulerRequest(rid, list(prompt), 9 if rid != "c" else 7, stop_token_ids=stop if rid == "b" else ()))
    outputs, ahead_steps = drive_ahead(cache, sched)
    assert outputs == want
    assert ahead_steps >= 4
    assert cache.free_pages() == [32] and cache.free_slots() == 4


def test_planning_ahead_declines_when_a_decision_is_needed():
    cache, sched = make(num_pages=8, page_size=4, max_requests=2)
    sched.submit(SchedulerRequest("a", [1, 2, 3], 20))
    seen = {}
    plan = sched.plan()
    sampled = run_plan(cache, sched, plan, seen)
    sched.submit(SchedulerRequest("b", [4, 5], 4))
    assert sched.plan_ahead(plan) is None                     # somebody waits: admission is a decision
    sched.cancel("b")
    ahead = sched.plan_ahead(plan)
    assert ahead is not None and ahead.entries[0].start == 3
    sched.commit(plan, sampled)
    # a request that ends by length after the running step is not run further
    cache2, sched2 = make()
    sched2.submit(SchedulerRequest("x", [1, 2], 2))
    p0 = sched2.plan()
    s0 = run_plan(cache2, sched2, p0, {})
    assert sched2.plan_ahead(p0) is not None                  # one more token is still to come after this one
    sched2.commit(p0, s0)
    p1 = sched2.plan()
    run_plan(cache2, sched2, p1, {"x": {0: 1, 1: 2}})
    assert sched2.plan_ahead(p1) is None                      # p1 draws the last token
    # pages: both requests fill their last page, and none is free for the tokens after
    cache3, sched3 = make(num_pages=3, page_size=4, max_requests=2)
    sched3.submit(SchedulerRequest("y", list(range(8)), 3))
    sched3.submit(SchedulerRequest("z", list(range(4)), 3))
    p = sched3.plan()
    assert len(p.entries) == 2
    run_plan(cache3, sched3, p, {})
    assert cache3.free_pages() == [0] and sched3.plan_ahead(p) is None
