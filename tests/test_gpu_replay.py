"""Replay of the same requests cut in different ways, in 32-bit and in bfloat16, against the plain
implementation: whole; most in one step and the last 32 tokens one by one; in portions of changing
size down to two tokens; and mixed, up to four live requests with so few pages that they are used again."""
import numpy as np
import pytest
import torch

from conftest import TINY
from gpu_common import check_rows, need_gpu, requests_for
from replay_util import (InProcessReplayer, gather, peak_tokens, run_trace_program, trace_mixed, trace_portions,
                         trace_tail_decode, trace_whole)

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [7, 13, 1, 97, 128, 64, 2, 50], "B": [1, 5, 17, 40, 96, 211, 130, 64], "C": [3, 129, 70, 256, 31, 16, 200, 65],
           "D": [1, 64, 65, 300, 17, 129, 2, 700], "E": [5, 128, 63, 257, 1, 90, 420, 33]}
NAMES = ["A", "B", "C", "D", "E"]


def _requests(name):
    config, seed = TINY[name]
    return requests_for(config, seed, LENGTHS[name])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_every_way_of_cutting_agrees_with_the_plain_implementation(model_folders, name, dtype):
    need_gpu()
    folder, requests = model_folders[name], _requests(name)
    rows = {}
    for maker in (trace_whole, trace_tail_decode, trace_portions):
        steps, index = maker(requests)
        replayer = InProcessReplayer(folder, dtype, max_tokens=peak_tokens(steps))
        rows[maker.__name__] = gather(replayer.run(steps), index)
        check_rows(rows[maker.__name__], folder, requests, dtype)
        assert replayer.runner.cache.free_pages() == [replayer.runner.cache.num_pages]
    if dtype == "float32":
        # the 32-bit kernels keep each row's arithmetic independent of the cut: bit-equal
        whole = rows["trace_whole"]
        for other in ("trace_tail_decode", "trace_portions"):
            for key, got in rows[other].items():
                assert np.array_equal(got[0], whole[key][0]), f"{other} differs from whole at {key}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_on_a_tight_pool(model_folders, name, dtype, seed):
    need_gpu()
    folder, requests = model_folders[name], _requests(name)
    steps, index = trace_mixed(requests, seed=seed)
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"] if any(len(o["tokens"]) == 1 for o in s["entries"]))
    peak = peak_tokens(steps)
    assert peak < sum(-(-len(t) // 64) * 64 for t in requests.values())      # pages must be used again
    replayer = InProcessReplayer(folder, dtype, max_tokens=peak)
    rows = gather(replayer.run(steps), index)
    check_rows(rows, folder, requests, dtype)
    cache = replayer.runner.cache
    assert cache.free_pages() == [cache.num_pages] and not cache.live_requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_folders, tmp_path, dtype):
    """bin/trace_run itself: the file protocol, `done` lines, page reuse, both dtypes."""
    need_gpu()
    folder, requests = model_folders["B"], _requests("B")
    steps, index = trace_mixed(requests, seed=3)
    extra, extra_index = trace_tail_decode({"r4": requests["r4"]}, tail=8)
    for s in extra:                       # append after the mixed part, with later step numbers
        s["step"] += len(steps)
    index.update({(st + len(steps), row): key for (st, row), key in extra_index.items()})
    steps = steps + extra
    steps.insert(3, {"step": 1000, "entries": [], "end": []})      # a step that brings nothing
    results = run_trace_program(folder, dtype, peak_tokens(steps), steps, tmp_path / "out")
    check_rows(gather(results, index), folder, requests, dtype)


def test_peaky_attention_shows_a_lost_key(model_folders, tmp_path):
    """Random weights give nearly flat attention, which would hide a lost key among hundreds.
    With q and k projections scaled up the scores spread, so every key counts."""
    need_gpu()
    from safetensors.torch import load_file, save_file
    import shutil
    folder = tmp_path / "peaky"
    shutil.copytree(model_folders["C"], folder)
    tensors = load_file(str(folder / "model.safetensors"))
    for key in tensors:
        if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
            tensors[key] = (tensors[key].float() * 12).to(torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    config, seed = TINY["C"]
    requests = requests_for(config, seed + 7, [300, 77, 130, 610])
    for maker in (trace_whole, trace_portions, trace_mixed):
        steps, index = maker(requests)
        replayer = InProcessReplayer(folder, "float32", max_tokens=peak_tokens(steps))
        check_rows(gather(replayer.run(steps), index), folder, requests, "float32")


@pytest.mark.parametrize("name", ["D", "E"])
def test_peaky_attention_in_bfloat16_on_the_tensor_core_kernels(model_folders, tmp_path, name):
    """The same in bfloat16 at head sizes 64 and 128, where prompt portions run on the tcgen05 kernel and single
    tokens on the TMA decode kernel, through the engine's own dispatch, block tables and context splits, whole,
    in portions and mixed on a tight pool.  With nearly flat attention a lost key moves a logit by less than the
    bfloat16 tolerance; with the scores spread it does not."""
    need_gpu()
    from safetensors.torch import load_file, save_file
    import shutil
    folder = tmp_path / "peaky"
    shutil.copytree(model_folders[name], folder)
    tensors = load_file(str(folder / "model.safetensors"))
    for key in tensors:
        if key.endswith("q_proj.weight") or key.endswith("k_proj.weight"):
            tensors[key] = (tensors[key].float() * 4).to(torch.bfloat16)
    save_file(tensors, str(folder / "model.safetensors"))
    config, seed = TINY[name]
    requests = requests_for(config, seed + 7, [300, 77, 130, 610, 64, 1000])
    # What a lost key would cost here: the plain logits with one early key hidden from every later query leave the
    # true ones by many times the tolerance (measured: 20 times; with the unscaled weights it is under one).  The
    # scale is as large as bfloat16 allows: queries and keys rounded to 8 bits move a score by score / 256, and at
    # four times the scale of the weights that alone takes 0.4 of the tolerance, at six times more than all of it.
    import plain_llama
    from gpu_common import BF16_REL, plain_logits
    true_attention = plain_llama.causal_attention

    def one_key_lost(q, k, v, group, window=None, rows=None):
        out = true_attention(q, k, v, group, window, rows)
        if k.shape[1] > 40:                              # queries after position 5 do not see key 5
            keep = [i for i in range(k.shape[1]) if i != 5]
            out[:, 6:] = true_attention(q[:, 6:], k[:, keep], v[:, keep], group, None, rows=range(5, k.shape[1] - 1))
        return out
    cfg, weights = plain_llama.read_model_folder(folder)
    truth = plain_logits(folder, requests["r0"])
    plain_llama.causal_attention = one_key_lost
    try:
        lossy = plain_llama.forward(cfg, weights, requests["r0"]).numpy()
    finally:
        plain_llama.causal_attention = true_attention
    assert np.abs(lossy - truth).max() > 5 * BF16_REL * np.abs(truth).max()
    for maker in (trace_whole, trace_portions, trace_mixed):
        steps, index = maker(requests)
        replayer = InProcessReplayer(folder, "bfloat16", max_tokens=peak_tokens(steps))
        check_rows(gather(replayer.run(steps), index), folder, requests, "bfloat16")


def test_two_processes_write_the_same_bits(model_folders, tmp_path):
    """bin/trace_run twice, in two processes, on the same trace in bfloat16 with the default choice of kernels:
    the files are equal byte for byte (which kernel multiplies few rows is decided once per GPU model and shape
    and kept beside the built library, not timed anew by every process)."""
    need_gpu()
    folder, requests = model_folders["D"], _requests("D")
    steps, _ = trace_mixed(requests, seed=5)
    first = run_trace_program(folder, "bfloat16", peak_tokens(steps), steps, tmp_path / "one")
    second = run_trace_program(folder, "bfloat16", peak_tokens(steps), steps, tmp_path / "two")
    assert first.keys() == second.keys() and len(first) > 10
    for step in first:
        assert np.array_equal(first[step], second[step]), f"step {step} differs between two processes"


@pytest.mark.parametrize("backend", ["tcgen05", "library"])
def test_bf16_projections_on_either_gemm_backend(model_folders, backend):
    """The hand-written tcgen05 products (swap-AB for few rows, 128 x 256 tiles for many) and cuBLAS
    must both carry the engine: same traces, same tolerance."""
    need_gpu()
    from torchinferno_b200.kernels import gemm, ops
    folder, requests = model_folders["D"], _requests("D")
    gemm.set_backend(backend)
    try:
        launches = ops.launch_count()
        for maker in (trace_whole, trace_tail_decode, trace_mixed):
            steps, index = maker(requests)
            replayer = InProcessReplayer(folder, "bfloat16", max_tokens=peak_tokens(steps))
            check_rows(gather(replayer.run(steps), index), folder, requests, "bfloat16")
        assert ops.launch_count() > launches
    finally:
        gemm.set_backend("auto")
