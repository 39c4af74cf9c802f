"""Generation through the Python entry point and the command line, long decoding, and the first tokens
of a sequence, against the plain implementation."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama
from conftest import TINY
from gpu_common import BF16_REL, check_rows, need_gpu, plain_logits, requests_for
from replay_util import InProcessReplayer, gather, peak_tokens, trace_tail_decode

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def engine_for(folder, dtype, **options):
    from torchinferno_b200.config.engine_config import EngineConfig
    from torchinferno_b200.engine.engine import InferenceEngine
    return InferenceEngine.from_config(EngineConfig(model=str(folder), dtype=dtype, **options))


def requests(prompts, max_tokens, temperature=0.0, seeds=None, stop=()):
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    return [GenerateRequest(f"g{i}", prompt_token_ids=p, sampling=SamplingConfig(
        max_tokens, temperature, stop, 0 if seeds is None else seeds[i])) for i, p in enumerate(prompts)]


def test_greedy_generation_equals_the_plain_implementation_fp32(model_folders):
    """Tiny A: prompts of 7, 13 and 1 tokens, pages of 4, eight greedy tokens each, all together."""
    need_gpu()
    config, seed = TINY["A"]
    prompts = list(requests_for(config, seed, [7, 13, 1]).values())
    cfg, weights = plain_llama.read_model_folder(model_folders["A"])
    want = [plain_llama.generate_greedy(cfg, weights, p, 8) for p in prompts]
    with engine_for(model_folders["A"], "float32", page_size=4, max_batch_size=4) as engine:
        outs = engine.generate_many(requests(prompts, 8))
        assert [list(o.token_ids) for o in outs] == want
        assert all(o.finish_reason == "length" and o.usage.completion_tokens == 8 for o in outs)
        assert [o.usage.prompt_tokens for o in outs] == [7, 13, 1]
        # one at a time through generate(), and streamed
        single = engine.generate(requests(prompts[:1], 8)[0])
        assert list(single.token_ids) == want[0]
        streamed = list(engine.generate_stream(requests(prompts[1:2], 8)[0]))
        assert [t.token_id for t in streamed[:-1]] == want[1] and streamed[-1].finished and streamed[-1].finish_reason == "length"
        assert [t.index for t in streamed[:-1]] == list(range(8))
        # a stop token ends the request and is emitted
        stopped = engine.generate(requests(prompts[:1], 8, stop=(want[0][3],))[0])
        assert list(stopped.token_ids) == want[0][:want[0].index(want[0][3]) + 1] and stopped.finish_reason == "stop"
        assert engine.runner.cache.free_pages() == [engine.runner.cache.num_pages]


def test_async_scheduling_gives_the_same_tokens(model_folders):
    """Tiny B, fp32: the same requests (greedy and seeded sampling, one of them ending at a stop token while
    the step after it already runs, another cancelled in flight) with the next step launched ahead of the
    host and without; and a request id used again at once."""
    need_gpu()
    config, seed = TINY["B"]
    prompts = list(requests_for(config, seed, [5, 17, 3]).values())
    results = {}
    for ahead in (False, True):
        with engine_for(model_folders["B"], "float32", page_size=16, max_batch_size=4, async_scheduling=ahead) as engine:
            greedy = engine.generate_many(requests(prompts, 20))
            stop = (greedy[1].token_ids[7],)
            stopped = engine.generate_many(requests(prompts, 20, stop=stop))
            again = engine.generate(requests(prompts[:1], 6)[0])      # the id "g0" once more, right after
            warm = engine.generate_many(requests(prompts, 14, temperature=0.7, seeds=[11, 12, 13]))
            # cancel one of two requests while steps are in flight
            for r in requests(prompts[:2], 12):
                engine.submit(r)
            got = []
            for i in range(40):
                for event in engine.step():
                    if event.request_id == "g0" and event.token is not None:
                        got.append(event.token)
                if i == 4:
                    engine.cancel("g1")
                if not engine.scheduler.has_work():
                    break
            results[ahead] = ([o.token_ids for o in greedy], [(o.token_ids, o.finish_reason) for o in stopped],
                              again.token_ids, [o.token_ids for o in warm], got)
            assert engine.stats["steps_ahead"] > 20 if ahead else engine.stats["steps_ahead"] == 0
            engine.step()                                             # a step left in flight is dropped
            assert engine.runner.cache.free_pages() == [engine.runner.cache.num_pages]
            engine.runner.cache.audit()
    assert results[True] == results[False]
    assert any(reason == "stop" for _, reason in results[True][1])
    assert results[True][2] == results[True][0][0][:6] and results[True][4] == list(results[True][0][0][:12])


def test_programmatic_dependent_launch_changes_no_token(model_folders):
    """Tiny D in bfloat16 (TMA decode attention, tcgen05 prefill attention, swap-AB output projection, all launched
    so that they may start while the kernel before drains): the same requests with that switched off."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    config, seed = TINY["D"]
    prompts = list(requests_for(config, seed, [70, 9, 33]).values())
    got = {}
    try:
        for on in (True, False):
            ops.set_dependent_launch(on)
            with engine_for(model_folders["D"], "bfloat16", page_size=16, max_batch_size=4, prefill_chunk_size=32) as engine:
                got[on] = [o.token_ids for o in engine.generate_many(requests(prompts, 24))]
    finally:
        ops.set_dependent_launch(True)
    assert got[True] == got[False]


def test_many_requests_on_a_tight_pool_do_not_depend_on_how_they_are_scheduled(model_folders):
    """Tiny B, fp32: forty requests of random lengths (1..90 prompt tokens, 1..40 new tokens, some at a temperature,
    some with a stop token that really occurs), more than the slots and pages hold at once, so that requests wait,
    are cut into portions, are preempted and recomputed.  Every way of running them (async scheduling on and off,
    large and small token budgets and portions, pools of two sizes) must give each request the tokens it gets when
    it runs alone."""
    need_gpu()
    import random
    config, seed = TINY["B"]
    rng = random.Random(7)
    lengths = [rng.randint(1, 90) for _ in range(40)]
    prompts = list(requests_for(config, seed, lengths).values())
    budgets = [rng.randint(1, 40) for _ in prompts]
    temps = [0.0 if rng.random() < 0.6 else 0.9 for _ in prompts]

    def make(stops):
        from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
        return [GenerateRequest(f"q{i}", prompt_token_ids=p, sampling=SamplingConfig(budgets[i], temps[i], stops[i], 100 + i))
                for i, p in enumerate(prompts)]

    with engine_for(model_folders["B"], "float32", page_size=16, max_batch_size=2, kv_cache_tokens=512) as engine:
        alone = [engine.generate(r) for r in make([()] * len(prompts))]
        # a stop token that occurs: the token in the middle of what the request generates alone
        stops = [(o.token_ids[len(o.token_ids) // 2],) if i % 3 == 0 and len(o.token_ids) > 2 else () for i, o in enumerate(alone)]
        want = [engine.generate(r) for r in make(stops)]
    assert any(o.finish_reason == "stop" for o in want) and any(o.finish_reason == "length" for o in want)
    ways = [dict(async_scheduling=True, max_batch_size=8, kv_cache_tokens=400, max_num_batched_tokens=64, prefill_chunk_size=24),
            dict(async_scheduling=False, max_batch_size=8, kv_cache_tokens=400, max_num_batched_tokens=64, prefill_chunk_size=24),
            dict(async_scheduling=True, max_batch_size=5, kv_cache_tokens=260, max_num_batched_tokens=33, prefill_chunk_size=7),
            dict(async_scheduling=True, max_batch_size=16, kv_cache_tokens=2000, max_num_batched_tokens=4096, prefill_chunk_size=2048)]
    preempted = 0
    for options in ways:
        with engine_for(model_folders["B"], "float32", page_size=16, **options) as engine:
            got = engine.generate_many(make(stops))
            preempted += engine.scheduler.stats["preemptions"]
            engine.runner.cache.audit()
            assert engine.runner.cache.free_pages() == [engine.runner.cache.num_pages]
        assert [(o.token_ids, o.finish_reason) for o in got] == [(o.token_ids, o.finish_reason) for o in want], options
    assert preempted > 0                                   # the tight pools really ran out


def _random_round(model_folders, draw):
    """Draw number ``draw`` of a random search over schedules, in float32: a tiny configuration, 8 to 30 requests
    of random lengths, budgets, temperatures and (for some) a stop token that occurs, run once with room and once
    under a random schedule on a pool that may be tight.  Returns (tokens and reasons with room, the same under the
    schedule, the schedule, preemptions)."""
    import random
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    rng = random.Random(1000 + draw)
    name = rng.choice("ABCDE")
    config, seed = TINY[name]
    top = min(120, config["max_position_embeddings"] // 2)
    n = rng.randint(8, 30)
    lengths = [rng.randint(1, top) for _ in range(n)]
    prompts = list(requests_for(config, seed + draw, lengths).values())
    budgets = [rng.randint(1, min(40, config["max_position_embeddings"] - l - 1)) for l in lengths]
    temps = [0.0 if rng.random() < 0.5 else rng.choice([0.5, 0.9, 1.3]) for _ in prompts]
    page = rng.choice([4, 8, 16, 32])

    def make(stops):
        return [GenerateRequest(f"s{i}", prompt_token_ids=p, sampling=SamplingConfig(budgets[i], temps[i], stops[i], 7000 + 13 * i + draw))
                for i, p in enumerate(prompts)]

    with engine_for(model_folders[name], "float32", page_size=page, max_batch_size=4, kv_cache_tokens=4096) as engine:
        roomy = engine.generate_many(make([()] * n))
        stops = [(o.token_ids[len(o.token_ids) // 2],) if rng.random() < 0.3 and len(o.token_ids) > 2 else () for o in roomy]
        want = engine.generate_many(make(stops))
    longest = max(l + b for l, b in zip(lengths, budgets))
    need = -(-longest // page) * page
    way = dict(async_scheduling=rng.random() < 0.7, max_batch_size=rng.randint(1, 12),
               kv_cache_tokens=max(need + page, rng.randint(need, 6 * need)), max_num_batched_tokens=rng.randint(8, 200),
               prefill_chunk_size=rng.randint(2, 64), page_size=page)
    with engine_for(model_folders[name], "float32", **way) as engine:
        got = engine.generate_many(make(stops))
        preemptions = engine.scheduler.stats["preemptions"]
        engine.runner.cache.audit()
        assert engine.runner.cache.free_pages() == [engine.runner.cache.num_pages]
    return [(o.token_ids, o.finish_reason) for o in want], [(o.token_ids, o.finish_reason) for o in got], way, preemptions


@pytest.mark.parametrize("draw", [395, 95, 70, 285])
def test_a_recomputation_that_ends_one_token_short_feeds_that_token_from_the_host(model_folders, draw):
    """Draws of the random search below that found this: a preempted request whose recomputation, cut into portions,
    ends exactly one token short of its sequence goes on with a decode step for the token it had last generated.
    That token is known to the host and was never drawn on the device since the request was opened again, so the
    step must take it from the host, not from the request's record (which then held no token: the embedding of "no
    token" is NaN, and the request went on with token 0)."""
    need_gpu()
    want, got, way, preemptions = _random_round(model_folders, draw)
    assert preemptions > 0
    assert got == want, way


def test_random_schedules_give_every_request_the_tokens_it_gets_with_room(model_folders):
    """Thirty draws of the random search (other than the ones above): whatever the schedule, in float32 every request
    gets exactly the tokens and the finish reason it gets with room; no page is lost on the way."""
    need_gpu()
    preempted = 0
    for draw in range(30):
        want, got, way, preemptions = _random_round(model_folders, draw)
        preempted += preemptions
        assert got == want, (draw, way)
    assert preempted > 20


def test_schedules_in_bfloat16_on_the_default_path_give_the_same_tokens(model_folders):
    """Config D (head size 64: tcgen05 prompt attention, TMA decode attention, the native block call, captured
    decode steps, steps launched ahead) in bfloat16 with the library's products, which makes the kernels of a row
    the same under every schedule: thirty requests (some at a temperature, some with a stop token that occurs)
    on pools so tight that requests wait, are cut and are preempted.  Every schedule must give every request
    the tokens of every other schedule."""
    need_gpu()
    import random
    config, seed = TINY["D"]
    rng = random.Random(11)
    lengths = [rng.randint(1, 200) for _ in range(30)]
    prompts = list(requests_for(config, seed, lengths).values())
    budgets = [rng.randint(2, 40) for _ in prompts]
    temps = [0.0 if rng.random() < 0.5 else 0.8 for _ in prompts]

    def make(stops):
        from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
        return [GenerateRequest(f"q{i}", prompt_token_ids=p, sampling=SamplingConfig(budgets[i], temps[i], stops[i], 500 + i))
                for i, p in enumerate(prompts)]

    base = dict(gemm_backend="library", page_size=16)
    with engine_for(model_folders["D"], "bfloat16", max_batch_size=8, kv_cache_tokens=4096, **base) as engine:
        roomy = engine.generate_many(make([()] * len(prompts)))
    stops = [(o.token_ids[len(o.token_ids) // 2],) if i % 3 == 0 and len(o.token_ids) > 2 else () for i, o in enumerate(roomy)]
    ways = [dict(async_scheduling=True, max_batch_size=8, kv_cache_tokens=4096, max_num_batched_tokens=4096),
            dict(async_scheduling=False, max_batch_size=8, kv_cache_tokens=4096, max_num_batched_tokens=4096),
            dict(async_scheduling=True, max_batch_size=8, kv_cache_tokens=640, max_num_batched_tokens=96, prefill_chunk_size=40),
            dict(async_scheduling=False, max_batch_size=6, kv_cache_tokens=560, max_num_batched_tokens=64, prefill_chunk_size=24),
            dict(async_scheduling=True, max_batch_size=3, kv_cache_tokens=480, max_num_batched_tokens=33, prefill_chunk_size=7)]
    results, preempted, ahead = [], 0, 0
    for options in ways:
        with engine_for(model_folders["D"], "bfloat16", **base, **options) as engine:
            got = engine.generate_many(make(stops))
            preempted += engine.scheduler.stats["preemptions"]
            ahead += engine.stats["steps_ahead"]
            engine.runner.cache.audit()
            assert engine.runner.cache.free_pages() == [engine.runner.cache.num_pages]
            assert engine.runner.graph_replays > 0
        results.append([(o.token_ids, o.finish_reason) for o in got])
    assert any(r == "stop" for _, r in results[0]) and any(r == "length" for _, r in results[0])
    # Single-token rows are multiplied by the same library kernel whatever the batch, but a prompt portion's
    # rows are not (the kernel changes with the row count), so a token may differ where two schedules cut a
    # prompt differently and two logits lie within rounding of each other.  Equal cuts must give equal tokens.
    assert results[0] == results[1], "async scheduling changed a token"
    agree = [sum(a == b for a, b in zip(results[0], other)) for other in results[2:]]
    assert min(agree) >= len(prompts) - 3, agree
    assert preempted > 0 and ahead > 20


def test_warm_up_captures_the_decode_steps_ahead_of_serving_and_changes_no_token(model_folders):
    """warm_up() captures the decode step for every batch size it is given with throw-away requests; afterwards the
    cache is empty, serving replays those captures from its first decode step on, and the tokens are those of an
    engine that was not warmed up."""
    need_gpu()
    config, seed = TINY["D"]
    prompts = list(requests_for(config, seed, [30, 5, 17]).values())
    with engine_for(model_folders["D"], "bfloat16", page_size=16, max_batch_size=4, gemm_backend="library") as engine:
        cold = engine.generate_many(requests(prompts, 12, 0.7, [1, 2, 3]))
    with engine_for(model_folders["D"], "bfloat16", page_size=16, max_batch_size=4, gemm_backend="library") as engine:
        assert engine.warm_up() == [4, 3, 2, 1]
        cache = engine.runner.cache
        assert sorted(engine.runner._graphs) == [1, 2, 3, 4] and all(g.graph is not None for g in engine.runner._graphs.values())
        assert cache.free_pages() == [cache.num_pages] and not cache.live_requests
        cache.audit()
        replays = engine.runner.graph_replays
        warm = engine.generate_many(requests(prompts, 12, 0.7, [1, 2, 3]))
        assert engine.runner.graph_replays - replays >= 11          # (every decode step of the run was a replay)
        with pytest.raises(RuntimeError, match="idle"):
            engine.submit(requests(prompts[:1], 4)[0])
            engine.warm_up([2])
    assert [o.token_ids for o in warm] == [o.token_ids for o in cold]


def test_the_engine_sees_an_error_word_that_a_kernel_set_and_goes_on_without_the_failed_requests(model_folders):
    """The kernels report a page id outside its pool or a bounded wait that ran out in one device word; the
    engine reads it with the step's tokens.  Here the word is set from the host (no kernel is made to fail).
    The step's requests are cancelled and give their pages back, the word is cleared, and the next request
    generates what it should."""
    need_gpu()
    from torchinferno_b200.engine.runner import StepError
    config, seed = TINY["A"]
    prompt = list(requests_for(config, seed, [9]).values())[0]
    cfg, weights = plain_llama.read_model_folder(model_folders["A"])
    with engine_for(model_folders["A"], "float32", page_size=4, max_batch_size=2) as engine:
        engine.submit(requests([prompt], 6)[0])
        engine.step()
        engine.runner.cache.error_word.fill_(0x7C0031)
        with pytest.raises(StepError, match="0x7c0031"):
            for _ in range(3):
                engine.step()
        cache = engine.runner.cache
        assert int(cache.error_word.item()) == 0 and not engine.scheduler.has_work()
        assert cache.free_pages() == [cache.num_pages] and not cache.live_requests
        again = engine.generate(requests([prompt], 6)[0])
        assert list(again.token_ids) == plain_llama.generate_greedy(cfg, weights, prompt, 6)


@pytest.mark.parametrize("ahead", [True, False])
def test_a_sampled_decode_step_copies_only_new_block_table_entries_to_the_device(model_folders, ahead):
    """Seed, temperature, position and the last drawn token of every request live in its record on the device:
    a decode step at a temperature takes its inputs and the sampler its parameters from there.  Over decode
    steps that need no new page nothing at all goes from the host to the device; a step in which a request
    crosses into a new page brings that one block-table entry (index and page id)."""
    need_gpu()
    config, seed = TINY["B"]
    prompts = list(requests_for(config, seed, [20, 37, 5]).values())
    with engine_for(model_folders["B"], "float32", page_size=16, max_batch_size=4, async_scheduling=ahead) as engine:
        for r in requests(prompts, 40, 0.7, [5, 6, 7]):
            engine.submit(r)
        while any(r.prefilling for r in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        engine.step()                                        # (the first decode step brings the slots of its requests)
        per_step = []
        for _ in range(30):
            lengths = {r.request_id: engine.runner.cache.length(r.request_id) for r in engine.scheduler.running}
            before = engine.stats["h2d_bytes"]
            engine.step()
            new_pages = sum(1 for rid, n in lengths.items() if engine.runner.cache.length(rid) > n and n % 16 == 0)
            per_step.append((engine.stats["h2d_bytes"] - before, new_pages))
        assert all(copied == 8 * pages for copied, pages in per_step), per_step
        assert any(pages for _, pages in per_step) and any(not pages for _, pages in per_step)


def test_a_slot_used_again_carries_nothing_over(tmp_path, model_folders):
    """A request that takes the slot of one that has ended starts from a whole new record (length, token, seed,
    temperature, count of drawn tokens) and zeroed mixer state: its tokens are those it draws in a fresh engine."""
    need_gpu()
    from torchinferno_b200.cache.manager import REC_DRAWN, REC_LENGTH, REC_SEED_LO
    config, seed = TINY["B"]
    first, second = list(requests_for(config, seed, [33, 12]).values())
    with engine_for(model_folders["B"], "float32", page_size=16, max_batch_size=1) as engine:
        engine.generate(requests([first], 9, 0.9, [1234])[0])
        cache = engine.runner.cache
        torch.cuda.synchronize()
        left = cache.request_records[0].tolist()              # (one slot: the record the first request leaves behind)
        assert left[REC_LENGTH] >= 33 + 8 and left[REC_DRAWN] == 9 and left[REC_SEED_LO] == 1234
        reused = engine.generate(requests([second], 9, 0.6, [77])[0])
        torch.cuda.synchronize()
        now = cache.request_records[0].tolist()
        assert now[REC_SEED_LO] == 77 and now[REC_DRAWN] == 9 and now[REC_LENGTH] in (12 + 8, 12 + 9)
    with engine_for(model_folders["B"], "float32", page_size=16, max_batch_size=1) as engine:
        fresh = engine.generate(requests([second], 9, 0.6, [77])[0])
    assert reused.token_ids == fresh.token_ids
    # and the state tensors of a mixer that keeps some: the cache manager zeroes the slot when it is opened
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.parts.base import CacheSpec, StateSpec
    manager = CacheManager([CacheSpec(1, 16)], [StateSpec((5,)), None], page_size=4, num_pages=8, max_requests=2,
                           max_request_tokens=32, dtype=torch.float32, device="cuda")
    slot = manager.open("a")
    manager.states[0][slot] = 3.0
    manager.close("a")
    assert manager.open("b") == slot and manager.states[0][slot].abs().sum().item() == 0.0


def test_seeded_temperature_generation_fp32(model_folders):
    """Tiny B: five prompts (1, 5, 17, 40, 96 tokens), pages of 16, portions of 32, twelve tokens at
    temperature 0.8.  Each token must be the Gumbel-max choice of the plain logits for the engine's own
    prefix with the request's seed, and must not depend on batching."""
    need_gpu()
    config, seed = TINY["B"]
    prompts = list(requests_for(config, seed, [1, 5, 17, 40, 96]).values())
    cfg, weights = plain_llama.read_model_folder(model_folders["B"])
    seeds = [11, 12, 13, 14, 15]
    with engine_for(model_folders["B"], "float32", page_size=16, prefill_chunk_size=32, max_num_batched_tokens=64) as engine:
        together = engine.generate_many(requests(prompts, 12, 0.8, seeds))
        alone = [engine.generate(r) for r in requests(prompts, 12, 0.8, seeds)]
    assert [o.token_ids for o in together] == [o.token_ids for o in alone]
    for prompt, out, s in zip(prompts, together, seeds):
        ids = list(prompt) + list(out.token_ids)
        logits = plain_llama.forward(cfg, weights, ids[:-1]).numpy()
        for i, tok in enumerate(out.token_ids):
            pos = len(prompt) + i
            scores = plain_llama.gumbel_scores(logits[pos - 1], 0.8, s, pos)
            assert scores[tok] >= scores.max() - 1e-4, (pos, tok, int(scores.argmax()))
    assert len({o.token_ids for o in together}) == 5


@pytest.mark.parametrize("name", ["A", "C", "D"])
def test_greedy_generation_bf16_follows_the_plain_logits(model_folders, name):
    """In bfloat16 a near-tie may go the other way, so each generated token is checked against the plain
    logits of the engine's own prefix: it is the plain implementation's own choice nearly always, and where it
    is not, it is one of the plain implementation's three best and its logit is within the engine's own
    error bound (twice the bfloat16 tolerance: one for either logit) of the best."""
    need_gpu()
    config, seed = TINY[name]
    prompts = list(requests_for(config, seed, [7, 13, 1, 60]).values())
    cfg, weights = plain_llama.read_model_folder(model_folders[name])
    with engine_for(model_folders[name], "bfloat16", page_size=16) as engine:
        outs = engine.generate_many(requests(prompts, 10))
    same = total = 0
    for prompt, out in zip(prompts, outs):
        ids = list(prompt) + list(out.token_ids)
        logits = plain_llama.forward(cfg, weights, ids[:-1]).numpy()
        for i, tok in enumerate(out.token_ids):
            row = logits[len(prompt) + i - 1]
            assert row[tok] >= row.max() - 2 * BF16_REL * np.abs(logits).max()
            assert tok in np.argsort(row)[-3:], (tok, np.argsort(row)[-3:])
            same += int(tok == int(row.argmax()))
            total += 1
    assert same >= 0.85 * total, f"only {same} of {total} tokens are the plain implementation's choice"


def test_preemption_on_a_small_pool_does_not_change_the_tokens(model_folders):
    need_gpu()
    config, seed = TINY["B"]
    prompts = list(requests_for(config, seed + 1, [30, 45, 20, 33, 50, 12]).values())
    with engine_for(model_folders["B"], "float32", page_size=16, max_batch_size=8) as engine:
        roomy = engine.generate_many(requests(prompts, 40, 0.7, list(range(6))))
    with engine_for(model_folders["B"], "float32", page_size=16, max_batch_size=8, num_pages=11) as engine:
        tight = engine.generate_many(requests(prompts, 40, 0.7, list(range(6))))
        assert engine.scheduler.stats["preemptions"] > 0
        engine.runner.cache.audit()
        assert engine.runner.cache.free_pages() == [11]
    assert [o.token_ids for o in tight] == [o.token_ids for o in roomy]


def test_cancel_gives_pages_back(model_folders):
    need_gpu()
    with engine_for(model_folders["A"], "float32", page_size=4) as engine:
        stream = engine.generate_stream(requests([[1, 2, 3, 4, 5]], 50)[0])
        first = [next(stream) for _ in range(3)]
        assert all(not t.finished for t in first)
        assert engine.cancel("g0")
        rest = list(stream)
        assert rest[-1].finished and rest[-1].finish_reason == "cancelled"
        assert engine.runner.cache.free_pages() == [engine.runner.cache.num_pages]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(model_folders, dtype):
    """One request decoded token by token for hundreds of steps, over many pages."""
    need_gpu()
    config, seed = TINY["C"]
    reqs = requests_for(config, seed + 3, [620])
    steps, index = trace_tail_decode(reqs, tail=500)
    replayer = InProcessReplayer(model_folders["C"], dtype, max_tokens=peak_tokens(steps))
    check_rows(gather(replayer.run(steps), index), model_folders["C"], reqs, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(model_folders, dtype):
    """Positions 0, 1, 2 one by one: the first token has nothing before it, the pages are new."""
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    for name in ("A", "B"):
        config, seed = TINY[name]
        reqs = requests_for(config, seed + 5, [4, 4])
        replayer = InProcessReplayer(model_folders[name], dtype, max_tokens=128)
        rows = {}
        with torch.inference_mode():
            for pos in range(4):
                out = replayer.runner.step([StepEntry(k, [v[pos]], [0]) for k, v in reqs.items()]).cpu().numpy()
                for i, k in enumerate(reqs):
                    rows[(k, pos)] = [out[i]]
        check_rows(rows, model_folders[name], reqs, dtype)


def test_step_refuses_bad_input_and_reports_no_room(model_folders):
    need_gpu()
    from torchinferno_b200.cache.manager import OutOfPages
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.runner import StepError
    replayer = InProcessReplayer(model_folders["A"], "float32", max_tokens=64)
    runner = replayer.runner
    with torch.inference_mode():
        with pytest.raises(StepError, match="vocabulary"):
            runner.step([StepEntry("a", [256], [0])])
        with pytest.raises(StepError, match="twice"):
            runner.step([StepEntry("a", [1], [0]), StepEntry("a", [2], [0])])
        with pytest.raises(StepError, match="wants logits"):
            runner.step([StepEntry("a", [1, 2], [2])])
        with pytest.raises(StepError, match="no tokens"):
            runner.step([StepEntry("a", [], [])])
        runner.step([StepEntry("a", [1] * 40, [])])
        with pytest.raises(OutOfPages):
            runner.step([StepEntry("b", [1] * 20, []), StepEntry("a", [1] * 10, [])])
        assert runner.cache.length("a") == 40 and "b" not in runner.cache      # nothing changed
        runner.cache.audit()
        with pytest.raises(StepError, match="limit"):
            runner.step([StepEntry("c", [1] * 129, [])])


def test_command_line(model_folders, tmp_path):
    need_gpu()
    folder = model_folders["A"]
    cfg, weights = plain_llama.read_model_folder(folder)
    cli = [sys.executable, str(ROOT / "bin" / "torchinferno-b200")]
    out = subprocess.run(cli + ["generate", str(folder), "--input-ids", "5", "17", "3", "--new-tokens", "6", "--dtype", "float32",
                                "--page-size", "4"], capture_output=True, text=True, check=True).stdout
    line = next(l for l in out.splitlines() if l.startswith("output_ids="))
    assert json.loads(line.split("=", 1)[1]) == [5, 17, 3] + plain_llama.generate_greedy(cfg, weights, [5, 17, 3], 6)
    captured = tmp_path / "logits.json"
    subprocess.run(cli + ["capture-logits", str(folder), str(captured), "--input-ids", "9", "8", "7", "--dtype", "float32"], check=True,
                   capture_output=True)
    got = json.loads(captured.read_text())["logits"]
    assert np.allclose(got, plain_llama.forward(cfg, weights, [9, 8, 7])[-1].numpy(), atol=2e-5)
    ok = subprocess.run(cli + ["validate-logits", str(folder), str(captured), "--dtype", "float32"], capture_output=True, text=True)
    assert ok.returncode == 0 and "ok" in ok.stdout
    smoke = subprocess.run(cli + ["serve-smoke", "--dtype", "bfloat16"], capture_output=True, text=True, check=True).stdout
    assert smoke.count("finish_reason=length") == 3
