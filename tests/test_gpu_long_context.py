"""Logits and attention rows where the benchmark runs: 32 query heads on 8 key/value heads of 128, pages of 16,
contexts of 2,048 to 8,200 tokens, with the context splits the engine itself chooses, against the plain
implementation; and the engine at the 8B layer sizes on a 2,048-token prompt followed by 64 decoded tokens.
(The plain implementation computes only the compared rows of a long sequence: same formulas, fewer rows.)"""
import math

import numpy as np
import pytest
import torch

import plain_llama
from gpu_common import BF16_REL_LARGE, need_gpu, note_worst
from test_gpu_kernels import dev, fill_pages, paged_layout, rnd
from test_gpu_large_layers import LARGE

pytestmark = pytest.mark.gpu
HEADS, KV_HEADS, D, PAGE = 32, 8, 128, 16


def long_case(entries, standout=None, seed=0):
    """entries: (kv_start, q_len).  Pages, queries and the float64 rows wanted for them."""
    lengths = [s + n for s, n in entries]
    pool, table, slots = paged_layout(len(entries), lengths, PAGE, KV_HEADS, D, torch.bfloat16, seed=seed)
    q_rows, refs, q_start = [], [], [0]
    for e, (start, n) in enumerate(entries):
        total = start + n
        k, v = rnd(KV_HEADS, total, D, dtype=torch.bfloat16, seed=seed + e), rnd(KV_HEADS, total, D, dtype=torch.bfloat16, seed=seed + 50 + e)
        q = rnd(HEADS, n, D, dtype=torch.bfloat16, seed=seed + 100 + e)
        if standout is not None and standout < total:
            # one far key whose score (about 12) stands out from the others (about N(0, 1)) for every query that sees it
            u = torch.ones(D) / math.sqrt(D)
            q = (q.float() * 0.2 + 8.0 * u).to(torch.bfloat16)
            k[:, standout] = (12.0 * math.sqrt(D) / 8.0 * u).to(torch.bfloat16)
            v[:, standout] = (v[:, standout].float() + 7).to(torch.bfloat16)
        fill_pages(pool, table, slots[e], k, v)
        q_rows.append(q.transpose(0, 1).reshape(n, HEADS * D))
        ref = plain_llama.causal_attention(q.double(), k.double(), v.double(), HEADS // KV_HEADS, rows=range(start, total))
        refs.append(ref.transpose(0, 1).reshape(n, HEADS * D))
        q_start.append(q_start[-1] + n)
    i32 = lambda xs: dev(torch.tensor(xs, dtype=torch.int32))
    args = (dev(torch.cat(q_rows)), dev(pool), None, i32(q_start), i32([s for s, _ in entries]), i32(slots), dev(table), len(entries))
    return args, torch.cat(refs), lengths


@pytest.mark.parametrize("contexts, standout", [
    ([2048], None), ([4096], 0), ([8200], 4000), ([8200], 0),            # one request: 16, 16 and 32 context parts
    ([2048, 3000, 4096, 2500, 4001, 2049, 3999, 4095], 2047),              # eight requests: 4 parts each
    ([2048 + 7 * i for i in range(64)], None),                             # sixty-four: one part each
    ([8200, 100, 8193, 4097], 4000)])
def test_tma_decode_attention_at_the_benchmarks_contexts(contexts, standout):
    need_gpu()
    from torchinferno_b200.kernels import ops
    entries = [(c - 1, 1) for c in contexts]
    args, ref, lengths = long_case(entries, standout, seed=len(contexts))
    splits = ops.decode_num_splits(len(entries), HEADS, KV_HEADS, max(lengths))
    assert splits == {1: 32 if max(lengths) > 8192 else 16, 8: 4, 64: 1, 4: 8}[len(entries)]
    out = torch.full_like(args[0], float("nan"))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.decode_attention(args[0], args[1], out, *args[3:], HEADS, KV_HEADS, D, 1.0 / math.sqrt(D), max(lengths),
                         kernel="tma", error_word=err)          # (splits and parts as the engine's step chooses them)
    assert int(err) == 0 and torch.isfinite(out).all()
    if standout is not None:
        assert ref.abs().max() > 3
    assert torch.allclose(out.cpu().double(), ref, atol=6e-2 if standout is not None else 2e-2, rtol=2e-2), \
        (out.cpu().double() - ref).abs().max()


@pytest.mark.parametrize("entries, standout", [
    ([(0, 2048)], None), ([(0, 2048)], 0), ([(1500, 548)], 3), ([(4096, 300), (0, 700)], 4000), ([(7900, 300)], 0),
    ([(7900, 300), (8199, 1), (2047, 1)], 4000)])
def test_tcgen05_prefill_attention_at_the_benchmarks_contexts(entries, standout):
    need_gpu()
    from torchinferno_b200.kernels import ops
    args, ref, lengths = long_case(entries, standout, seed=7)
    out = torch.full_like(args[0], float("nan"))
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    singles = sum(1 for _, n in entries if n == 1)
    scale = 1.0 / math.sqrt(D)
    ops.prefill_attention_tcgen05(args[0], args[1], out, *args[3:], max(n for _, n in entries), HEADS, KV_HEADS, D, scale,
                                  skip_single=singles > 0, error_word=err)
    if singles:
        ops.decode_attention(args[0], args[1], out, *args[3:], HEADS, KV_HEADS, D, scale, max(lengths), kernel="tma", error_word=err)
    assert int(err) == 0 and torch.isfinite(out).all()
    assert torch.allclose(out.cpu().double(), ref, atol=6e-2 if standout is not None else 2e-2, rtol=2e-2), \
        (out.cpu().double() - ref).abs().max()


# ------------------------------------------------------------------ the engine at the 8B layer sizes
PROMPT, DECODED = 2048, 64


@pytest.fixture(scope="module")
def long_folder(tmp_path_factory):
    from torchinferno_b200.weights.random_init import write_random_model
    folder = tmp_path_factory.mktemp("large_long")
    write_random_model(LARGE, folder, seed=9)
    return folder


@pytest.fixture(scope="module")
def long_reference(long_folder):
    """Tokens and the plain logits (float32 on the CPU) at the last prompt position and at every decoded one."""
    g = torch.Generator().manual_seed(2048)
    tokens = torch.randint(0, LARGE["vocab_size"], (PROMPT + DECODED,), generator=g).tolist()
    config, weights = plain_llama.read_model_folder(long_folder, dtype=torch.float32)
    rows = list(range(PROMPT - 1, PROMPT + DECODED))
    with torch.inference_mode():
        want = plain_llama.forward(config, weights, tokens, rows=rows).double().numpy()
    return tokens, rows, want


@pytest.mark.parametrize("cut", ["whole", "1500+548"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_2048_token_prompt_and_64_decoded_tokens_at_the_8b_layer_sizes(long_folder, long_reference, dtype, cut):
    """The prompt whole or as 1,500 + 548 tokens, then 64 tokens one by one (the captured decode step, context
    parts merged in the kernel): the logits at the prompt's last position and at every decoded one."""
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import load_model, make_runner
    tokens, rows, want = long_reference
    model = load_model(long_folder, dtype=dtype)
    runner = make_runner(model, page_size=16, max_tokens=PROMPT + DECODED + 16, max_requests=2)
    got = []
    with torch.inference_mode():
        if cut == "whole":
            got.append(runner.step([StepEntry("r", tokens[:PROMPT], [PROMPT - 1])]).cpu())
        else:
            assert runner.step([StepEntry("r", tokens[:1500], [])]).shape[0] == 0
            got.append(runner.step([StepEntry("r", tokens[1500:PROMPT], [PROMPT - 1501])]).cpu())
        for t in tokens[PROMPT:PROMPT + DECODED]:
            got.append(runner.step([StepEntry("r", [t], [0])]).cpu())
        runner.end(["r"])
    if dtype == "bfloat16":
        assert runner.graph_replays >= DECODED - 1
    got = torch.cat(got)[:len(rows)].double().numpy()
    assert np.isfinite(got).all()
    err = np.abs(got - want[:len(got)]).max(axis=1)
    # (the plain implementation runs in float32 here, so in 32-bit its own rounding counts too)
    bound = (1e-4 if dtype == "float32" else BF16_REL_LARGE) * np.abs(want).max()
    note_worst(f"8B layer sizes, 2048-token prompt {cut} + 64 decoded, {dtype}", err.max() / bound)
    assert err.max() <= bound, f"{dtype} {cut}: row {int(err.argmax())} is off by {err.max():.3e} > {bound:.3e}"
    del runner, model
    torch.cuda.empty_cache()
