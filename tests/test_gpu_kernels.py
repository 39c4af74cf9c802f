"""Each CUDA kernel alone against a plain PyTorch reference (float64 on the CPU), at sizes other
than the engine's tiny models: widths that are no power of two, head sizes in steps of 16, odd
group sizes, page sizes from 1 up, windows, ragged batches."""
import math

import pytest
import torch

import plain_llama
from gpu_common import need_gpu

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=1e-2, rtol=1.6e-2)


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype else t.to("cuda")


def as_ref(t):
    return t.detach().cpu().double()


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


# ------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [100, 4096, 5000])
def test_embedding(dtype, hidden):
    need_gpu()
    from torchinferno_b200.kernels import ops
    table = rnd(37, hidden, dtype=dtype)
    ids = torch.tensor([3, 36, 0, 3, 40, -1], dtype=torch.int32)
    out = torch.empty(6, hidden, device="cuda")
    ops.embedding(dev(ids), dev(table), out)
    assert torch.equal(out[:4].cpu(), table[ids[:4].long()].float())
    assert torch.isnan(out[4:]).all()                      # ids outside the table must show


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, hidden, eps", [(5, 100, 1e-5), (3, 4096, 1e-6), (2, 5000, 3e-6), (1, 24, 1e-2)])
def test_add_rmsnorm(dtype, rows, hidden, eps):
    need_gpu()
    from torchinferno_b200.kernels import ops
    res0, delta, w = rnd(rows, hidden, scale=3), rnd(rows, hidden, dtype=dtype, seed=1), 1 + 0.2 * rnd(hidden, seed=2)
    # plain norm of the residual
    res = dev(res0.clone())
    out = torch.empty(rows, hidden, dtype=dtype, device="cuda")
    ops.add_rmsnorm(None, res, dev(w), eps, out)
    want = plain_llama.rms_norm(res0.double(), w.double(), eps)
    assert torch.allclose(as_ref(out), want, **tol(dtype)) and torch.equal(res.cpu(), res0)
    # fused add: the residual is updated in 32-bit, the normed rows leave in dtype
    ops.add_rmsnorm(dev(delta), res, dev(w), eps, out)
    summed = res0 + delta.float()
    assert torch.equal(res.cpu(), summed)
    assert torch.allclose(as_ref(out), plain_llama.rms_norm(summed.double(), w.double(), eps), **tol(dtype))
    # rows: only the picked rows, residual untouched
    pick = torch.tensor([rows - 1, 0, rows - 1], dtype=torch.int32)
    out3 = torch.empty(3, hidden, dtype=dtype, device="cuda")
    before = res.clone()
    ops.add_rmsnorm(dev(delta), res, dev(w), eps, out3, rows=dev(pick))
    want3 = plain_llama.rms_norm((summed + delta.float()).double(), w.double(), eps)[pick.long()]
    assert torch.allclose(as_ref(out3), want3, **tol(dtype)) and torch.equal(res, before)
    # rows of the activation type
    x = rnd(rows, hidden, dtype=dtype, seed=5)
    ops.rmsnorm(dev(x), dev(w), eps, out)
    assert torch.allclose(as_ref(out), plain_llama.rms_norm(x.double(), w.double(), eps), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, inter", [(7, 200), (1, 14336), (33, 17)])
def test_swiglu(dtype, rows, inter):
    need_gpu()
    from torchinferno_b200.kernels import ops
    gu = rnd(rows, 2 * inter, dtype=dtype, scale=3)
    out = torch.empty(rows, inter, dtype=dtype, device="cuda")
    ops.swiglu(dev(gu), out)
    g, u = gu.double()[:, :inter], gu.double()[:, inter:]
    assert torch.allclose(as_ref(out), g / (1 + torch.exp(-g)) * u, **tol(dtype))


def test_cast_and_scatter():
    need_gpu()
    from torchinferno_b200.kernels import ops
    x = rnd(1000, 3)
    y = ops.cast(dev(x), torch.empty(1000, 3, dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(y.cpu(), x.to(torch.bfloat16))
    assert torch.equal(ops.cast(y, torch.empty(1000, 3, device="cuda")).cpu(), x.to(torch.bfloat16).float())
    table = torch.full((4, 5), -1, dtype=torch.int32, device="cuda")
    ops.scatter_i32(table, dev(torch.tensor([7, 0, 19, 99], dtype=torch.int32)), dev(torch.tensor([70, 1, 190, 5], dtype=torch.int32)))
    want = torch.full((20,), -1, dtype=torch.int32)
    want[7], want[0], want[19] = 70, 1, 190
    assert torch.equal(table.cpu().view(-1), want)


# ------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("m, n, k", [(1, 64, 64), (37, 129, 100), (130, 67, 257), (5, 1000, 4096)])
@pytest.mark.parametrize("wdtype", DTYPES)
def test_gemm_f32_is_true_fp32_and_row_independent(m, n, k, wdtype):
    need_gpu()
    from torchinferno_b200.kernels import ops
    x, w = rnd(m, k, scale=2), rnd(n, k, dtype=wdtype, seed=3)
    out = ops.gemm_f32(dev(x), dev(w), torch.empty(m, n, device="cuda"))
    want = x.double() @ w.double().T
    # fp32 accumulation over k terms: error far below what a tf32 or bf16 product would leave
    assert (as_ref(out) - want).abs().max() <= 4e-7 * math.sqrt(k) * (x.abs().max() * w.float().abs().max()).item() * math.sqrt(k)
    one = ops.gemm_f32(dev(x[m // 2: m // 2 + 1].contiguous()), dev(w), torch.empty(1, n, device="cuda"))
    assert torch.equal(one[0], out[m // 2])               # a row does not depend on the rows beside it


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (1, 8, 64), (200, 520, 192), (77, 1000, 4096), (300, 264, 1024), (2048, 512, 14336)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05(m, n, k, out_dtype):
    """The TMA / tcgen05 / TMEM product against float64, with rows and columns that do not fill the
    128 x 256 tiles, a long K (many trips round the stage ring), and both output types."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, scale=0.05, seed=3)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_tcgen05(dev(x), dev(w), torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda"), err)
    assert int(err) == 0                                   # no bounded wait ran out
    want = (x.cuda().double() @ w.cuda().double().T).cpu()
    bound = (1e-2 if out_dtype == torch.bfloat16 else 2e-5) * want.abs().max() + 1e-6
    assert (as_ref(out) - want).abs().max() <= bound
    with pytest.raises(ops.KernelError, match="size"):     # K must be a multiple of 64
        ops.gemm_tcgen05(dev(rnd(4, 96, dtype=torch.bfloat16)), dev(rnd(8, 96, dtype=torch.bfloat16)), torch.empty(4, 8, dtype=out_dtype, device="cuda"))


@pytest.mark.parametrize("m, n, k", [(256, 256, 64), (1, 8, 64), (200, 520, 192), (77, 1000, 4096), (600, 264, 1024), (2048, 512, 14336),
                                     (515, 1288, 512)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_on_pairs_of_sms(m, n, k, out_dtype):
    """The `cta_group::2` product (two blocks per 256 x 256 tile) against float64: one tile, rows and columns that
    do not fill the tiles (among them tiles whose second block has no rows at all), a long K, more tiles than
    pairs of SMs take in one round, and both output types."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, scale=0.05, seed=3)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.gemm_tcgen05_2cta(dev(x), dev(w), torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda"), err)
    assert int(err) == 0                                   # no bounded wait ran out
    want = (x.cuda().double() @ w.cuda().double().T).cpu()
    bound = (1e-2 if out_dtype == torch.bfloat16 else 2e-5) * want.abs().max() + 1e-6
    assert (as_ref(out) - want).abs().max() <= bound
    with pytest.raises(ops.KernelError, match="size"):     # K must be a multiple of 64
        ops.gemm_tcgen05_2cta(dev(rnd(4, 96, dtype=torch.bfloat16)), dev(rnd(8, 96, dtype=torch.bfloat16)), torch.empty(4, 8, dtype=out_dtype, device="cuda"))


@pytest.mark.parametrize("m, n, k, splits", [(8, 128, 64, 0), (1, 8, 64, 1), (8, 6144, 4096, 0), (16, 4096, 4096, 4), (5, 1000, 4096, 0),
                                             (8, 4096, 14336, 8), (33, 520, 192, 3), (64, 264, 1024, 0), (17, 28672, 512, 0),
                                             (48, 136, 9472, 5)])
@pytest.mark.parametrize("w_kn", [False, True])
def test_gemm_tcgen05_swapab(m, n, k, splits, w_kn):
    """The few-rows product (weights as the 128-row operand, K split over a cluster) against float64: one tile, a
    ragged last tile, every padding of the rows, splits chosen and forced, more tiles than clusters, and the weights
    stored [out, in] (K-major operand) as well as [in, out] (MN-major operand); both output types."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, scale=0.05, seed=3)
    want = (x.cuda().double() @ w.cuda().double().T).cpu()
    wd = dev(w.t().contiguous()) if w_kn else dev(w)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for out_dtype in (torch.bfloat16, torch.float32):
        out = ops.gemm_tcgen05_swapab(dev(x), wd, torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda"), err,
                                      splits=splits, w_kn=w_kn)
        assert int(err) == 0                               # no bounded wait ran out
        bound = (1e-2 if out_dtype == torch.bfloat16 else 2e-5) * want.abs().max() + 1e-6
        assert (as_ref(out) - want).abs().max() <= bound
    with pytest.raises(ops.KernelError, match="size"):     # at most 64 rows
        ops.gemm_tcgen05_swapab(dev(rnd(65, 64, dtype=torch.bfloat16)), dev(rnd(8, 64, dtype=torch.bfloat16)),
                                torch.empty(65, 8, dtype=torch.bfloat16, device="cuda"))


def test_few_rows_kernel_is_chosen_by_measurement_and_either_choice_is_right():
    """Weights that leave their few-rows kernel open get it from tune_few_rows (the hand-written kernel up to 0, 4, 8,
    16, 32 or 64 rows, with the tile width and K split that measured fastest): one decision per shape, kept for the
    process and on disk, the same for every weight of the shape; a slice of the weight inherits it; whichever kernel
    was chosen, and whichever is forced, the product is right at few and at many rows; and so is silu(gate) * up
    of a weight bound with the SwiGLU epilogue, fused or not."""
    need_gpu()
    from torchinferno_b200.kernels import gemm
    from torchinferno_b200.kernels.gemm import LinearWeight, linear, linear_swiglu
    n, k = 1160, 2048
    ws = [rnd(n, k, dtype=torch.bfloat16, scale=0.05, seed=i) for i in range(3)]
    open_weights = [LinearWeight(dev(w), few_rows_tcgen05=None) for w in ws]
    assert all(w.few_rows == 0 for w in open_weights)                     # the library until measured
    decisions = gemm.tune_few_rows()
    key = (n, k, open_weights[0].tensor.device, "none")
    rows, features, splits = decisions[key]
    assert rows in (0, 4, 8, 16, 32, 64) and features in (128, 256) and 0 <= splits <= 8
    assert all((w.few_rows, w.features, w.splits) == decisions[key] for w in open_weights)
    later = LinearWeight(dev(ws[0]), few_rows_tcgen05=None)
    assert gemm.tune_few_rows()[key] == decisions[key] and later.few_rows == open_weights[0].few_rows
    gemm._tuned.pop(key)                                                   # a new process reads what this one stored
    again = [LinearWeight(dev(w), few_rows_tcgen05=None) for w in ws]      # (as many weights of the shape as were measured)
    assert gemm.tune_few_rows()[key] == decisions[key] and again[0].splits == splits
    forced = [LinearWeight(dev(ws[0]), few_rows_tcgen05=True), LinearWeight(dev(ws[0]), few_rows_tcgen05=False)]
    assert [w.few_rows for w in forced] == [LinearWeight.FEW_ROWS, 0] and LinearWeight.FEW_ROWS == 64
    configured = LinearWeight(dev(ws[0]), few_rows_tcgen05=True)
    configured.features, configured.splits = 128, 4
    glu = [LinearWeight(dev(ws[0][:1152]), few_rows_tcgen05=flag, epilogue="swiglu") for flag in (True, False)]
    glu[0].splits = 1
    for m in (1, 4, 5, 8, 9, 16, 17, 33, 64, 65, 200):
        x = rnd(m, k, dtype=torch.bfloat16, seed=50 + m)
        want = x.double() @ ws[0].double().T
        for weight in (open_weights[0], later, configured, *forced):
            out = linear(dev(x), weight)
            assert (as_ref(out) - want).abs().max() <= 1e-2 * want.abs().max() + 1e-6
            part = linear(dev(x), weight.rows(64, 1096))
            assert (as_ref(part) - want[:, 64:1096]).abs().max() <= 1e-2 * want.abs().max() + 1e-6
        gate, up = want[:, 0:1152:2], want[:, 1:1152:2]
        act = gate / (1 + torch.exp(-gate)) * up
        for weight in glu:
            got = linear_swiglu(dev(x), weight)
            assert got.shape == (m, 576) and (as_ref(got) - act).abs().max() <= 1.5e-2 * act.abs().max() + 1e-6


@pytest.mark.parametrize("m, n, k", [(1, 256, 64), (8, 6144, 4096), (16, 28672, 4096), (5, 1000, 4096), (33, 520, 192), (64, 4096, 4096)])
def test_gemm_decode_every_tile_width_split_and_epilogue(m, n, k):
    """The few-rows kernel on [in, out] weights: tiles of 128 features with K shared by 1 to 8 blocks of a cluster,
    tiles of 256 features unsplit, bf16 and fp32 results, and the SwiGLU epilogue on interleaved gate/up columns,
    against float64; NaN in the output buffer beforehand shows what was not written."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(k, n, dtype=torch.bfloat16, scale=0.05, seed=3)
    want = x.double() @ w.double()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ran = 0
    for features in (128, 256):
        for splits in (1, 2, 3, 5, 8):
            if not ops.gemm_decode_supports(m, n, k, features, splits):
                continue
            for out_dtype in (torch.bfloat16, torch.float32):
                out = ops.gemm_decode(dev(x), dev(w), torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda"),
                                      features=features, splits=splits, error_word=err)
                bound = (1e-2 if out_dtype == torch.bfloat16 else 1e-4) * want.abs().max() + 1e-6
                assert (as_ref(out) - want).abs().max() <= bound, (features, splits, out_dtype)
                ran += 1
        if n % 16 == 0:
            gate, up = want[:, 0::2], want[:, 1::2]
            act = gate / (1 + torch.exp(-gate)) * up
            out = ops.gemm_decode(dev(x), dev(w), torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device="cuda"),
                                  features=features, splits=1, epilogue=ops.DG_SWIGLU, error_word=err)
            assert (as_ref(out) - act).abs().max() <= 1e-2 * act.abs().max() + 1e-6
    assert ran >= 4 and int(err) == 0
    assert not ops.gemm_decode_supports(65, n, k) and not ops.gemm_decode_supports(m, n, k, 256, 2)
    assert not ops.gemm_decode_supports(m, n, k, 128, 2, ops.DG_SWIGLU) and not ops.gemm_decode_supports(m, n, k + 8)
    with pytest.raises(ops.KernelError, match="size"):
        ops.gemm_decode(dev(x), dev(w), torch.empty(m, n, dtype=torch.bfloat16, device="cuda"), features=256, splits=2)


def _records(rows):
    """A record table [slots, 8] from {slot: (length, last token, seed, temperature, drawn)}."""
    import struct
    table = torch.zeros(max(rows) + 1, 8, dtype=torch.int32)
    for slot, (length, last, seed, temperature, drawn) in rows.items():
        seed &= 0xFFFFFFFFFFFFFFFF
        words = [length, last, seed & 0xFFFFFFFF, seed >> 32, struct.unpack("<I", struct.pack("<f", temperature))[0], drawn]
        table[slot, :6] = torch.tensor([w - (1 << 32) if w >= (1 << 31) else w for w in words], dtype=torch.int64).to(torch.int32)
    return table


def test_decode_inputs_come_from_the_requests_records_which_move_on():
    """The first kernel of a captured decode step: request i of the step sits in slot slots[i]; its next token and
    its position come from its record, whose length moves one on.  Records of other slots, the other words of a
    record and the tails of longer buffers stay as they are; a slot outside the table yields token -1."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    i32 = lambda xs: dev(torch.tensor(xs, dtype=torch.int32))
    table = _records({0: (4, 100, 7, 0.5, 1), 1: (9, 9, 9, 0.0, 9), 2: (511, 300, -3, 1.5, 2), 5: (0, 200, 1 << 40, 0.0, 0)})
    before, records = table.clone(), dev(table)
    tokens, positions = i32([7, 8, 9, 77]), i32([-1, -1, -1, 55])
    ops.decode_inputs(records, i32([2, 5, 0]), tokens, positions)
    assert tokens.tolist() == [300, 200, 100, 77] and positions.tolist() == [511, 0, 4, 55]
    after = records.cpu()
    assert after[:, 0].tolist() == [5, 9, 512, 0, 0, 1]
    assert torch.equal(after[:, 1:], before[:, 1:])
    ops.decode_inputs(records, i32([6, 1]), tokens, positions)           # slot 6 is outside the table
    assert tokens.tolist()[:2] == [-1, 9] and positions.tolist()[:2] == [0, 9]
    with pytest.raises(ops.KernelError, match="shorter"):
        ops.decode_inputs(records, i32([0, 1, 2]), i32([1]), positions)


def test_sampling_from_records_is_sampling_with_the_same_parameters_given_by_hand():
    """The sampler reads temperature, seed and the position of the drawn token (the request's length) from the
    record of each row's request, draws what the explicit form draws, and leaves the token in the record."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    logits = dev(torch.randn(4, 1000, generator=g) * 3)
    rows = {3: (17, -1, 12345678901234567, 0.8, 0), 1: (40, 5, -99, 1.3, 7), 0: (5, 5, 3, 0.0, 2), 6: (1, 1, 1, 0.7, 0)}
    records = dev(_records(rows))
    slots = dev(torch.tensor([3, 0, 1, 6], dtype=torch.int32))
    out, history = torch.empty(4, dtype=torch.int32, device="cuda"), torch.full((6,), -1, dtype=torch.int32, device="cuda")
    ops.sample_records(logits, out, records, slots, history)
    order = [3, 0, 1, 6]
    as_i64 = lambda s: ((s & 0xFFFFFFFFFFFFFFFF) ^ (1 << 63)) - (1 << 63)
    want = ops.sample(logits, torch.empty(4, dtype=torch.int32, device="cuda"),
                      dev(torch.tensor([rows[s][3] for s in order])), dev(torch.tensor([as_i64(rows[s][2]) for s in order])),
                      dev(torch.tensor([rows[s][0] for s in order], dtype=torch.int32)))
    assert out.tolist() == want.tolist() and history.tolist() == want.tolist() + [-1, -1]
    assert out.tolist()[1] == int(logits[1].argmax())                    # temperature 0 is greedy
    after = records.cpu()
    for row, slot in enumerate(order):
        assert after[slot, 1].item() == want[row].item() and after[slot, 5].item() == rows[slot][4] + 1
        assert after[slot, 0].item() == rows[slot][0]                    # the length is the decode step's to move


@pytest.mark.parametrize("m, n, k", [(1, 72, 40), (8, 4096, 4096), (17, 1000, 264), (300, 136, 2048)])
@pytest.mark.parametrize("w_kn", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_library_gemm_both_layouts(m, n, k, w_kn, out_dtype):
    """cuBLAS called from the engine's library (its own handle and workspace): weights stored [out, in] and
    [in, out], bf16 and fp32 results, against float64."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    x, w = rnd(m, k, dtype=torch.bfloat16), rnd(n, k, dtype=torch.bfloat16, scale=0.05, seed=3)
    ops.library_gemm_ready(torch.device("cuda", torch.cuda.current_device()))
    out = ops.library_gemm(dev(x), dev(w.t().contiguous()) if w_kn else dev(w),
                           torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda"), w_kn=w_kn)
    want = x.double() @ w.double().T
    bound = (1e-2 if out_dtype == torch.bfloat16 else 2e-5) * want.abs().max() + 1e-6
    assert (as_ref(out) - want).abs().max() <= bound


# -------------------------------------------------------------- RoPE + KV
def paged_layout(n_requests, lengths, page_size, kv_heads, d, dtype, spare_pages=3, seed=0):
    """A pool with NaN everywhere, shuffled page ids, and block tables for the given lengths."""
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-n // page_size) for n in lengths]
    total = sum(pages_per) + spare_pages
    order = torch.randperm(total, generator=g).tolist()
    width = max(pages_per) + 1
    table = torch.full((n_requests + 2, width), -1, dtype=torch.int32)
    slots = torch.randperm(n_requests + 2, generator=g)[:n_requests].tolist()
    for r, slot in enumerate(slots):
        for p in range(pages_per[r]):
            table[slot, p] = order.pop()
    pool = torch.full((total, 2, kv_heads, page_size, d), float("nan"), dtype=dtype)
    return pool, table, slots


def fill_pages(pool, table, slot, k, v, start=0):
    """k, v: [kv_heads, T, d] written at positions start.. of the request in ``slot``."""
    p = pool.shape[3]
    for t in range(k.shape[1]):
        pos = start + t
        page = int(table[slot, pos // p])
        pool[page, 0, :, pos % p] = k[:, t]
        pool[page, 1, :, pos % p] = v[:, t]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, d, rot, inter, page", [
    (4, 2, 16, None, False, 4), (5, 1, 48, None, False, 3), (3, 3, 80, 32, False, 16), (8, 2, 128, None, True, 16),
    (2, 1, 64, 0, False, 5)])
def test_rope_append(dtype, heads, kv_heads, d, rot, inter, page):
    need_gpu()
    from torchinferno_b200.kernels import ops
    from torchinferno_b200.parts.rope import rotary_frequencies
    rot_dim = d if rot is None else rot
    starts, lens = [0, 37, 5], [6, 1, 9]                 # three entries: a prompt start, a decode, a portion
    pool, table, slots = paged_layout(3, [s + n for s, n in zip(starts, lens)], page, kv_heads, d, dtype)
    positions = torch.tensor([s + i for s, n in zip(starts, lens) for i in range(n)], dtype=torch.int32)
    token_slot = torch.tensor([slots[e] for e, n in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    n = int(positions.numel())
    qkv = rnd(n, (heads + 2 * kv_heads) * d, dtype=dtype)
    scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 16}
    inv_freq = rotary_frequencies(rot_dim, 10000.0, scaling) if rot_dim else torch.zeros(0)
    pool_d, q_out = dev(pool), torch.empty(n, heads * d, dtype=dtype, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.rope_append(dev(qkv), q_out, pool_d, dev(positions), dev(token_slot), dev(table), dev(inv_freq),
                    heads, kv_heads, d, rot_dim=rot_dim, interleaved=inter, error_word=err)
    assert int(err) == 0

    def rotate(x):                                      # x [T, H, d] float64
        if rot_dim == 0:
            return x
        ang = (positions.float()[:, None] * inv_freq[None, :]).double()      # fp32 product, as the kernel
        c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
        out = x.clone()
        if inter:
            lo, hi = x[..., 0:rot_dim:2], x[..., 1:rot_dim:2]
            out[..., 0:rot_dim:2], out[..., 1:rot_dim:2] = lo * c - hi * s, hi * c + lo * s
        else:
            h = rot_dim // 2
            lo, hi = x[..., :h], x[..., h:rot_dim]
            out[..., :h], out[..., h:rot_dim] = lo * c - hi * s, hi * c + lo * s
        return out

    q, k, v = qkv.double().split([heads * d, kv_heads * d, kv_heads * d], dim=1)
    assert torch.allclose(as_ref(q_out).view(n, heads, d), rotate(q.view(n, heads, d)), **tol(dtype))
    want_k, got = rotate(k.reshape(n, kv_heads, d)), pool_d.cpu()
    written = torch.zeros(pool.shape[0], page, dtype=torch.bool)
    for t in range(n):
        pos, slot = int(positions[t]), int(token_slot[t])
        pg = int(table[slot, pos // page])
        written[pg, pos % page] = True
        assert torch.allclose(got[pg, 0, :, pos % page].double(), want_k[t], **tol(dtype))
        assert torch.equal(got[pg, 1, :, pos % page], v.reshape(n, kv_heads, d)[t].to(dtype))
    untouched = got.permute(0, 3, 1, 2, 4)[~written]
    assert torch.isnan(untouched).all()                 # nothing else in the pool was written
    # a page id outside the pool is reported, not written
    bad = table.clone()
    bad[slots[1], 37 // page] = pool.shape[0] + 5
    ops.rope_append(dev(qkv), q_out, pool_d, dev(positions), dev(token_slot), dev(bad), dev(inv_freq),
                    heads, kv_heads, d, rot_dim=rot_dim, interleaved=inter, error_word=err)
    assert int(err) != 0


# -------------------------------------------------------------- attention
def attention_case(dtype, heads, kv_heads, d, page, entries, window=0, seed=0, standout=None, kernel="simt", splits=None):
    """entries: list of (kv_start, q_len).  Returns kernel output and the float64 reference.

    kernel "simt": the CUDA-core kernel; "mma": the tensor-core pair (portions by the prefill kernel,
    single tokens by the split decode kernel, as the engine dispatches them); "mma_prefill": the
    prefill kernel alone for every entry; "tma": as "mma" with the single tokens by the TMA decode kernel.
    ``splits`` = (num_splits, chunk) forces a split."""
    from torchinferno_b200.kernels import ops
    lengths = [s + n for s, n in entries]
    pool, table, slots = paged_layout(len(entries), lengths, page, kv_heads, d, dtype, seed=seed)
    q_rows, refs, q_start = [], [], [0]
    group = heads // kv_heads
    for e, (start, n) in enumerate(entries):
        total = start + n
        k, v = rnd(kv_heads, total, d, dtype=dtype, seed=seed + e), rnd(kv_heads, total, d, dtype=dtype, seed=seed + 50 + e)
        q = rnd(heads, n, d, dtype=dtype, seed=seed + 100 + e)
        if standout is not None and standout < total:
            # every query shares a component along u, and one far key points along u: its score
            # (about 12) stands out from the others (about N(0, 1)) for every query that may see it
            u = torch.ones(d) / math.sqrt(d)
            q = (q.float() * 0.2 + 8.0 * u).to(dtype)
            k[:, standout] = (12.0 * math.sqrt(d) / 8.0 * u).to(dtype)
            v[:, standout] = (v[:, standout].float() + 7).to(dtype)
        fill_pages(pool, table, slots[e], k, v)
        q_rows.append(q.transpose(0, 1).reshape(n, heads * d))
        full_q = torch.zeros(heads, total, d, dtype=torch.float64)
        full_q[:, start:] = q.double()
        ref = plain_llama.causal_attention(full_q, k.double(), v.double(), group, window=window or None)[:, start:]
        refs.append(ref.transpose(0, 1).reshape(n, heads * d))
        q_start.append(q_start[-1] + n)
    q_all = torch.cat(q_rows)
    out = torch.empty_like(q_all, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    i32 = lambda xs: dev(torch.tensor(xs, dtype=torch.int32))
    scale, max_q = 1.0 / math.sqrt(d), max(n for _, n in entries)
    args = (dev(q_all), dev(pool), out, i32(q_start), i32([s for s, _ in entries]), i32(slots), dev(table), len(entries))
    if kernel == "simt":
        ops.paged_attention_simt(*args, max_q, heads, kv_heads, d, scale, window=window, error_word=err)
    elif kernel == "mma_prefill":
        ops.prefill_attention(*args, max_q, heads, kv_heads, d, scale, window=window)
    elif kernel == "tcgen05_prefill":
        ops.prefill_attention_tcgen05(*args, max_q, heads, kv_heads, d, scale, window=window, error_word=err)
    else:
        out.fill_(float("nan"))
        singles = sum(1 for _, n in entries if n == 1)
        if singles < len(entries):
            ops.prefill_attention(*args, max_q, heads, kv_heads, d, scale, window=window, skip_single=singles > 0)
        if singles:
            ns, ch = splits or (None, None)
            ops.decode_attention(*args, heads, kv_heads, d, scale, max(lengths), window=window, num_splits=ns, chunk=ch,
                                 kernel="tma" if kernel == "tma" else "cp_async", error_word=err)
    assert int(err) == 0
    return out.cpu(), torch.cat(refs)


ATTN_SHAPES = [  # heads, kv_heads, d, page
    (4, 2, 16, 4), (6, 3, 32, 16), (5, 1, 48, 3), (7, 7, 80, 1), (8, 2, 128, 16), (32, 1, 64, 64), (2, 1, 256, 16),
    (14, 2, 96, 5)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads, kv_heads, d, page", ATTN_SHAPES)
def test_paged_attention_ragged_batch(dtype, heads, kv_heads, d, page):
    need_gpu()
    entries = [(0, 70), (130, 1), (31, 2), (0, 1), (63, 33)]       # whole prompt, decode, tiny portion, first token, portion over block edges
    out, ref = attention_case(dtype, heads, kv_heads, d, page, entries)
    assert torch.isfinite(out).all()                              # NaN in unwritten slots must not leak
    assert torch.allclose(out.double(), ref, **(dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("window", [1, 5, 32, 33, 100])
def test_paged_attention_window_edges(window):
    need_gpu()
    entries = [(0, 90), (200, 1), (95, 7)]
    out, ref = attention_case(torch.float32, 4, 2, 32, 16, entries, window=window, seed=3)
    assert torch.allclose(out.double(), ref, atol=3e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("standout", [0, 3, 511, 512, 700])
def test_paged_attention_finds_one_far_key_among_hundreds(dtype, standout):
    need_gpu()
    entries = [(900, 1), (640, 70)]
    out, ref = attention_case(dtype, 8, 2, 64, 16, entries, seed=5, standout=standout)
    assert ref.abs().max() > 3                                    # the far key really dominates the reference
    assert torch.allclose(out.double(), ref, **(dict(atol=2e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=6e-2, rtol=2e-2)))


def test_paged_attention_rows_do_not_depend_on_the_batch():
    need_gpu()
    alone, _ = attention_case(torch.float32, 6, 3, 32, 16, [(40, 9)], seed=9)
    # same request (same seed → same q, k, v for entry 0) with others beside it
    mixed, _ = attention_case(torch.float32, 6, 3, 32, 16, [(40, 9), (0, 50), (77, 1)], seed=9)
    assert torch.equal(alone, mixed[:9])


BF16_ATTN = dict(atol=2e-2, rtol=2e-2)
MMA_SHAPES = [(4, 2, 64, 16), (8, 2, 128, 16), (32, 8, 128, 16), (3, 1, 64, 4), (6, 6, 128, 1), (40, 2, 64, 5), (7, 1, 128, 64),
              # head sizes that do not fill the 64- or 128-wide tiles
              (5, 1, 48, 16), (4, 2, 80, 8), (6, 2, 96, 16), (3, 3, 112, 4), (4, 4, 16, 16), (8, 2, 32, 3)]


@pytest.mark.parametrize("heads, kv_heads, d, page", MMA_SHAPES)
@pytest.mark.parametrize("kernel", ["mma", "mma_prefill"])
def test_tensor_core_attention_ragged_batch(heads, kv_heads, d, page, kernel):
    need_gpu()
    # a whole prompt over several tiles, decodes at short and long contexts, portions that start and
    # end off the tile edges, a first token, a two-token portion
    entries = [(0, 150), (130, 1), (31, 2), (0, 1), (63, 66), (700, 1), (64, 1), (255, 129)]
    out, ref = attention_case(torch.bfloat16, heads, kv_heads, d, page, entries, kernel=kernel)
    assert torch.isfinite(out).all()
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()


TC_SHAPES = [(4, 2, 64, 16), (8, 2, 128, 16), (32, 8, 128, 16), (3, 1, 64, 8), (6, 6, 128, 32), (16, 2, 64, 64), (7, 1, 128, 128)]


@pytest.mark.parametrize("heads, kv_heads, d, page", TC_SHAPES)
def test_tcgen05_prefill_attention_ragged_batch(heads, kv_heads, d, page):
    need_gpu()
    entries = [(0, 150), (130, 1), (31, 2), (0, 1), (63, 66), (700, 1), (64, 1), (255, 129), (0, 300)]
    out, ref = attention_case(torch.bfloat16, heads, kv_heads, d, page, entries, kernel="tcgen05_prefill")
    assert torch.isfinite(out).all()
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()


@pytest.mark.parametrize("window", [1, 5, 128, 129, 200])
def test_tcgen05_prefill_attention_window_edges(window):
    need_gpu()
    entries = [(0, 190), (300, 1), (95, 70), (63, 1), (120, 140)]
    out, ref = attention_case(torch.bfloat16, 4, 2, 64, 16, entries, window=window, seed=3, kernel="tcgen05_prefill")
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()


@pytest.mark.parametrize("standout", [0, 3, 511, 512, 700])
def test_tcgen05_prefill_attention_finds_one_far_key(standout):
    need_gpu()
    entries = [(900, 1), (640, 70)]
    out, ref = attention_case(torch.bfloat16, 8, 2, 64, 16, entries, seed=5, standout=standout, kernel="tcgen05_prefill")
    assert ref.abs().max() > 3
    assert torch.allclose(out.double(), ref, atol=6e-2, rtol=2e-2)


@pytest.mark.parametrize("splits", [(1, 1024), (2, 512), (3, 320), (16, 64), (9, 128), (1, 0), (2, 0), (5, 0), (32, 0)])
def test_split_decode_attention_is_the_same_for_every_split(splits):
    need_gpu()
    entries = [(900, 1), (0, 1), (63, 1), (64, 1), (517, 1)]
    out, ref = attention_case(torch.bfloat16, 8, 2, 128, 16, entries, kernel="mma", splits=splits, seed=2)
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()


TMA_SHAPES = [(4, 2, 64, 16), (8, 2, 128, 16), (32, 8, 128, 16), (3, 1, 64, 8), (6, 6, 128, 32), (32, 2, 64, 64), (7, 1, 128, 8),
              (12, 4, 128, 64)]


@pytest.mark.parametrize("heads, kv_heads, d, page", TMA_SHAPES)
def test_tma_decode_attention_ragged_batch(heads, kv_heads, d, page):
    """Single tokens by the TMA kernel (portions beside them by the mma.sync prefill kernel): contexts of 1, 64, 65
    tokens, ones that end in the middle of a page and of a tile, and a long one."""
    need_gpu()
    entries = [(0, 150), (130, 1), (31, 2), (0, 1), (63, 1), (700, 1), (64, 1), (255, 129), (1000, 1), (15, 1), (16, 1), (127, 1)]
    out, ref = attention_case(torch.bfloat16, heads, kv_heads, d, page, entries, kernel="tma")
    assert torch.isfinite(out).all()
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()


@pytest.mark.parametrize("splits", [(1, 1024), (2, 512), (3, 320), (16, 64), (9, 128), (1, 0), (2, 0), (5, 0), (32, 0)])
def test_tma_decode_attention_is_the_same_for_every_split(splits):
    need_gpu()
    entries = [(900, 1), (0, 1), (63, 1), (64, 1), (517, 1)]
    out, ref = attention_case(torch.bfloat16, 8, 2, 128, 16, entries, kernel="tma", splits=splits, seed=2)
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()
    other, _ = attention_case(torch.bfloat16, 8, 2, 128, 16, entries, kernel="mma", splits=splits, seed=2)
    assert torch.allclose(out.float(), other.float(), atol=4e-3, rtol=1e-2)     # the two kernels do the same arithmetic


@pytest.mark.parametrize("window", [1, 5, 64, 65, 200])
def test_tma_decode_attention_window_edges(window):
    need_gpu()
    entries = [(300, 1), (63, 1), (64, 1), (199, 1), (200, 1), (1, 1), (777, 1)]
    out, ref = attention_case(torch.bfloat16, 4, 2, 64, 16, entries, window=window, seed=3, kernel="tma")
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()


@pytest.mark.parametrize("standout", [0, 3, 511, 512, 700])
def test_tma_decode_attention_finds_one_far_key(standout):
    need_gpu()
    entries = [(900, 1), (701, 1)]
    out, ref = attention_case(torch.bfloat16, 8, 2, 64, 16, entries, seed=5, standout=standout, kernel="tma")
    assert ref.abs().max() > 3
    assert torch.allclose(out.double(), ref, atol=6e-2, rtol=2e-2)


@pytest.mark.parametrize("heads, kv_heads, d, page, rot, inter", [(8, 2, 128, 16, 128, False), (4, 2, 64, 8, 64, False), (32, 8, 128, 16, 128, False),
                                                                  (6, 1, 64, 32, 32, True), (4, 4, 128, 64, 0, False), (3, 1, 64, 16, 48, False)])
def test_tma_decode_attention_that_rotates_and_stores_the_newest_token_itself(heads, kv_heads, d, page, rot, inter):
    """One kernel from the rows of the qkv product (rotary encoding of q and k, the write of k and v into their pages,
    attention) gives bit for bit what the rotary kernel followed by the attention kernel gives: the same output and
    the same pages, with contexts that end at the first and last slot of a page and of a tile, and with 1, 4 and 16
    context parts."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    contexts = [1, 2, 64, 65, 16, 17, 700, 128, 333, 1000]
    n = len(contexts)
    pool, table, slots = paged_layout(n, contexts, page, kv_heads, d, torch.bfloat16, seed=9)
    for e, c in enumerate(contexts):                                  # older keys and values; the newest slot stays NaN
        if c > 1:
            fill_pages(pool, table, slots[e], rnd(kv_heads, c - 1, d, dtype=torch.bfloat16, seed=e), rnd(kv_heads, c - 1, d, dtype=torch.bfloat16, seed=40 + e))
    qkv = rnd(n, (heads + 2 * kv_heads) * d, dtype=torch.bfloat16, seed=77)
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / max(rot, 1)))) if rot else torch.zeros(0)
    i32 = lambda xs: dev(torch.tensor(xs, dtype=torch.int32))
    q_start, kv_start, slot_t, table_d = i32(list(range(n + 1))), i32([c - 1 for c in contexts]), i32(slots), dev(table)
    scale = 1.0 / math.sqrt(d)
    for splits in (1, 4, 16):
        pool_a, pool_b = dev(pool), dev(pool)
        q_rot = torch.empty(n, heads * d, dtype=torch.bfloat16, device="cuda")
        ops.rope_append(dev(qkv), q_rot, pool_a, kv_start, slot_t, table_d, dev(inv_freq), heads, kv_heads, d, rot_dim=rot, interleaved=inter)
        want = ops.decode_attention(q_rot, pool_a, torch.empty_like(q_rot), q_start, kv_start, slot_t, table_d, n, heads, kv_heads, d,
                                    scale, max(contexts), num_splits=splits, chunk=0, kernel="tma")
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        got = ops.decode_attention_rope(dev(qkv), pool_b, torch.full_like(q_rot, float("nan")), q_start, kv_start, slot_t, table_d, n,
                                        heads, kv_heads, d, scale, max(contexts), dev(inv_freq), rot_dim=rot, interleaved=inter,
                                        num_splits=splits, error_word=err)
        torch.cuda.synchronize()
        assert int(err) == 0 and torch.isfinite(got).all()
        assert torch.equal(got, want), (splits, (got.float() - want.float()).abs().max())
        a, b = pool_a.cpu(), pool_b.cpu()
        assert torch.equal(torch.isnan(a), torch.isnan(b)) and torch.equal(torch.nan_to_num(a), torch.nan_to_num(b))
    bad = table.clone()
    bad[slots[6], 699 // page] = pool.shape[0] + 3                    # a page id outside the pool is reported, not written
    ops.decode_attention_rope(dev(qkv), dev(pool), torch.empty_like(q_rot), q_start, kv_start, slot_t, dev(bad), n, heads, kv_heads, d,
                              scale, max(contexts), dev(inv_freq), rot_dim=rot, interleaved=inter, error_word=err)
    assert int(err) != 0


def test_tma_decode_attention_refuses_other_shapes():
    need_gpu()
    from torchinferno_b200.kernels import ops
    assert not ops.decode_attention_tma_supports(96, 4, 16) and not ops.decode_attention_tma_supports(128, 32, 16)
    assert not ops.decode_attention_tma_supports(128, 4, 5) and not ops.decode_attention_tma_supports(128, 4, 128)
    with pytest.raises(ops.KernelError, match="does not take this shape"):
        attention_case(torch.bfloat16, 4, 2, 64, 4, [(10, 1)], kernel="tma")


@pytest.mark.parametrize("window", [1, 5, 64, 65, 200])
@pytest.mark.parametrize("kernel", ["mma", "mma_prefill"])
def test_tensor_core_attention_window_edges(window, kernel):
    need_gpu()
    entries = [(0, 190), (300, 1), (95, 70), (63, 1)]
    out, ref = attention_case(torch.bfloat16, 4, 2, 64, 16, entries, window=window, seed=3, kernel=kernel)
    assert torch.allclose(out.double(), ref, **BF16_ATTN), (out.double() - ref).abs().max()


@pytest.mark.parametrize("standout", [0, 3, 511, 512, 700])
def test_tensor_core_attention_finds_one_far_key_among_hundreds(standout):
    need_gpu()
    entries = [(900, 1), (640, 70)]
    out, ref = attention_case(torch.bfloat16, 8, 2, 64, 16, entries, seed=5, standout=standout, kernel="mma")
    assert ref.abs().max() > 3
    assert torch.allclose(out.double(), ref, atol=6e-2, rtol=2e-2)


def test_attention_refuses_what_it_cannot_do():
    need_gpu()
    from torchinferno_b200.kernels import ops
    i32 = lambda xs: dev(torch.tensor(xs, dtype=torch.int32))

    def call(heads, kv_heads, d):
        q = torch.zeros(4, heads * d, device="cuda")
        pool = torch.zeros(2, 2, kv_heads, 16, d, device="cuda")
        ops.paged_attention_simt(q, pool, torch.empty_like(q), i32([0, 4]), i32([0]), i32([0]), i32([[0, 1]]), 1, 4,
                                 heads, kv_heads, d, 1.0)

    call(4, 2, 256)
    with pytest.raises(ops.KernelError, match="size"):
        call(4, 2, 272)                                             # head size above 256
    with pytest.raises(ops.KernelError, match="size"):
        call(5, 2, 32)                                              # heads not a multiple of kv heads
    with pytest.raises(ops.KernelError, match="CUDA tensor"):
        ops.swiglu(torch.zeros(2, 4), torch.zeros(2, 2))            # no CPU path
    assert ops.attention_mma_supports(128, 4) and ops.attention_mma_supports(48, 4)
    assert not ops.attention_mma_supports(40, 4) and not ops.attention_mma_supports(144, 4)
    q = torch.zeros(4, 4 * 144, device="cuda", dtype=torch.bfloat16)
    pool = torch.zeros(2, 2, 2, 16, 144, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ops.KernelError, match="size"):              # the tensor-core kernels take steps of 16 up to 128
        ops.prefill_attention(q, pool, torch.empty_like(q), i32([0, 4]), i32([0]), i32([0]), i32([[0, 1]]), 1, 4, 4, 2, 144, 1.0)


# --------------------------------------------------------------- sampling
def test_greedy_takes_the_lowest_index_among_maxima_and_nan_wins():
    need_gpu()
    from torchinferno_b200.kernels import ops
    logits = rnd(5, 3001)
    logits[0, 77] = logits[0, 2900] = 9.0
    logits[1, 3000] = 50.0
    logits[2, 1500] = float("nan")
    logits[3] = -float("inf")
    out = ops.sample(dev(logits), torch.empty(5, dtype=torch.int32, device="cuda")).cpu()
    assert out.tolist()[:4] == [77, 3000, 1500, 0] and out[4] == int(torch.argmax(logits[4]))


@pytest.mark.parametrize("vocab", [17, 1000, 128256])
def test_temperature_sampling_is_the_seeded_gumbel_max(vocab):
    need_gpu()
    from torchinferno_b200.kernels import ops
    logits = rnd(4, vocab, scale=2)
    temps, seeds, pos = [0.8, 1.5, 0.0, 0.3], [1, 2 ** 40 + 5, 3, -9], [0, 17, 5, 100000]
    i64 = torch.tensor(seeds, dtype=torch.int64)
    out = ops.sample(dev(logits), torch.empty(4, dtype=torch.int32, device="cuda"), dev(torch.tensor(temps)),
                     dev(i64), dev(torch.tensor(pos, dtype=torch.int32))).cpu().tolist()
    for r in range(4):
        if temps[r] == 0:
            assert out[r] == int(torch.argmax(logits[r]))
            continue
        scores = plain_llama.gumbel_scores(logits[r].numpy(), temps[r], seeds[r], pos[r])
        assert scores[out[r]] >= scores.max() - 1e-4        # the argmax, up to float rounding of near-ties
    # what else is in the batch does not matter
    alone = ops.sample(dev(logits[1:2].contiguous()), torch.empty(1, dtype=torch.int32, device="cuda"),
                       dev(torch.tensor(temps[1:2])), dev(i64[1:2].contiguous()), dev(torch.tensor(pos[1:2], dtype=torch.int32))).cpu()
    assert int(alone) == out[1]


def test_temperature_sampling_draws_from_the_softmax():
    need_gpu()
    from torchinferno_b200.kernels import ops
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]]).repeat(20000, 1)
    temp = 0.7
    out = ops.sample(dev(logits), torch.empty(20000, dtype=torch.int32, device="cuda"), dev(torch.full((20000,), temp)),
                     dev(torch.arange(20000, dtype=torch.int64)), dev(torch.zeros(20000, dtype=torch.int32))).cpu()
    freq = torch.bincount(out.long(), minlength=5).double() / 20000
    want = torch.softmax(logits[0].double() / temp, dim=0)
    assert (freq - want).abs().max() < 0.012


def test_the_library_plans_attention_and_products_for_both_ways_of_running_a_block():
    """`tib_plan_attention` and `tib_plan_product` are where the kernels of a step are chosen, for the parts and for
    the native block call: their answers on the shapes the engine meets."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    every = ops.ALLOW_PREFILL_TCGEN05 | ops.ALLOW_DECODE_ROTATES | ops.ALLOW_DECODE_TMA
    plan = ops.plan_attention
    # heads of 128 in groups of 4, pages of 16 back to back
    assert plan(128, 4, 16, True, 8, 8, 0, every) == (ops.ATTENTION_NONE, ops.ATTENTION_DECODE_TMA_ROTATES)
    assert plan(128, 4, 16, True, 9, 9, 0, every) == (ops.ATTENTION_NONE, ops.ATTENTION_DECODE_TMA)           # many requests
    assert plan(128, 4, 16, True, 8, 7, 1, every) == (ops.ATTENTION_PREFILL_TCGEN05, ops.ATTENTION_DECODE_TMA)  # a portion among them
    assert plan(128, 4, 16, True, 8, 8, 0, every & ~ops.ALLOW_DECODE_ROTATES)[1] == ops.ATTENTION_DECODE_TMA
    assert plan(128, 4, 16, False, 8, 7, 1, every) == (ops.ATTENTION_PREFILL_MMA, ops.ATTENTION_DECODE_CP_ASYNC)  # pages not back to back
    assert plan(128, 4, 16, True, 2, 0, 2, every & ~ops.ALLOW_PREFILL_TCGEN05) == (ops.ATTENTION_PREFILL_MMA, ops.ATTENTION_NONE)
    assert plan(128, 4, 3, True, 2, 1, 1, every) == (ops.ATTENTION_PREFILL_MMA, ops.ATTENTION_DECODE_CP_ASYNC)   # pages of 3 tokens
    assert plan(80, 4, 16, True, 2, 1, 1, every) == (ops.ATTENTION_PREFILL_MMA, ops.ATTENTION_DECODE_CP_ASYNC)   # heads of 80
    assert plan(72, 4, 16, True, 2, 1, 1, every) == (ops.ATTENTION_SIMT, ops.ATTENTION_SIMT)                     # heads of 72
    product = ops.plan_product
    assert product(8, 4096, 4096, True, 64, 128, 4, False, True) == ops.PRODUCT_DECODE
    assert product(8, 4096, 4096, True, 4, 128, 4, False, True) == ops.PRODUCT_LIBRARY      # more rows than the weight's bound
    assert product(8, 4096, 4096, True, 64, 128, 4, False, False) == ops.PRODUCT_LIBRARY    # operands not aligned
    assert product(8, 4096, 4096, True, 64, 128, 0, False, True) == ops.PRODUCT_SWAPAB      # no K split chosen: the older kernel
    assert product(8, 4096, 4096, False, 64, 128, 4, False, True) == ops.PRODUCT_SWAPAB     # [out, in] weights
    assert product(8, 28672, 4096, True, 64, 256, 1, True, True) == ops.PRODUCT_DECODE
    assert product(8, 28672, 4096, True, 64, 128, 2, True, True) != ops.PRODUCT_DECODE      # the activation only unsplit
    assert product(0, 4096, 4096, True, 64, 128, 4, False, True) == ops.PRODUCT_LIBRARY


def test_attention_kernels_on_random_shapes_and_batches():
    """Eighty draws of a random search over the attention kernels: head sizes, numbers of heads and groups, page
    sizes, windows, forced splits and ragged batches that no list in this file names, each against the float64
    plain attention; a shape a kernel does not take is passed over."""
    need_gpu()
    import random
    from torchinferno_b200.kernels import ops
    ran = {}
    for draw in range(80):
        rng = random.Random(77000 + draw)
        kernel = rng.choice(["simt32", "simt16", "mma", "mma_prefill", "tcgen05_prefill", "tma"])
        kv = rng.randint(1, 4)
        if kernel.startswith("simt"):
            d, group, page = rng.choice([8, 16, 24, 40, 64, 72, 96, 128, 160, 256]), rng.randint(1, 9), rng.choice([1, 2, 3, 4, 5, 8, 16, 32, 64])
        elif kernel in ("mma", "mma_prefill"):
            d, group = rng.choice([16, 32, 48, 64, 80, 96, 112, 128]), rng.choice([1, 2, 3, 4, 5, 7, 8, 12, 16, 20, 33, 64])
            page = rng.choice([1, 2, 3, 4, 5, 8, 16, 32, 64])
            if not ops.attention_mma_supports(d, group):
                continue
        else:
            d, group = rng.choice([64, 128]), rng.choice([1, 2, 3, 4, 5, 7, 8, 12, 16])
            page = rng.choice([8, 16, 32, 64, 128] if kernel == "tcgen05_prefill" else [8, 16, 32, 64])
            takes = ops.prefill_attention_tcgen05_supports if kernel == "tcgen05_prefill" else ops.decode_attention_tma_supports
            if not takes(d, group, page):
                continue
        heads = kv * group
        if heads * d > 8192:
            continue
        entries = []
        for _ in range(rng.randint(1, 6)):
            r = rng.random()
            entries.append((rng.randint(0, 900), 1) if r < 0.35 else (0, rng.randint(1, 300)) if r < 0.5 else
                           (rng.randint(0, 500), rng.randint(2, 200)))
        window = rng.choice([0, 0, 0, 1, 7, 64, 65, 130, 400])
        splits = (rng.choice([1, 2, 3, 5, 8, 16, 32]), 0) if kernel in ("mma", "tma") and rng.random() < 0.5 else None
        dtype = torch.float32 if kernel == "simt32" else torch.bfloat16
        out, ref = attention_case(dtype, heads, kv, d, page, entries, window=window, seed=draw,
                                  kernel="simt" if kernel.startswith("simt") else kernel, splits=splits)
        what = (draw, kernel, heads, kv, d, page, window, splits, entries)
        assert torch.isfinite(out).all(), what
        assert torch.allclose(out.double(), ref, **(dict(atol=3e-6, rtol=1e-5) if dtype == torch.float32 else BF16_ATTN)), what
        ran[kernel] = ran.get(kernel, 0) + 1
    assert len(ran) == 6 and min(ran.values()) >= 5, ran


def test_product_kernels_on_random_shapes():
    """Two hundred draws of a random search over the product kernels (the two tcgen05 kernels for many rows, the two
    for few rows with either weight layout, tile width, K split, ring depth and the SwiGLU epilogue, the library in
    both layouts, the 32-bit kernel), each against float64; NaN in the output beforehand shows what was not written."""
    need_gpu()
    import random
    from torchinferno_b200.kernels import ops
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    ran = {}
    for draw in range(200):
        rng = random.Random(31000 + draw)
        kind = rng.choice(["tcgen05", "2cta", "swapab", "swapab_kn", "decode", "decode_swiglu", "library", "library_kn", "f32"])
        g = torch.Generator().manual_seed(draw)
        few = kind in ("swapab", "swapab_kn", "decode", "decode_swiglu")
        m = rng.randint(1, 64) if few else rng.choice([1, 2, 7, 64, 100, 129, 256, 300, 513, 1000])
        n = rng.choice([8, 16, 24, 64, 72, 128, 136, 200, 256, 264, 512, 1000, 1024, 3072, 4104])
        k = rng.choice([64, 128, 192, 256, 320, 1024, 2048, 4096])
        out_dtype = rng.choice([torch.bfloat16, torch.float32])
        blank = lambda width, dtype: torch.full((m, width), float("nan"), dtype=dtype, device="cuda")
        if kind == "f32":
            n, k = rng.choice([1, 3, 64, 67, 129, 500]), rng.choice([1, 7, 64, 100, 257, 1000])
            x, w = torch.randn(m, k, generator=g).cuda(), torch.randn(n, k, generator=g).cuda()
            out, want, rel = ops.gemm_f32(x, w, blank(n, torch.float32)), as_ref(x) @ as_ref(w).T, 1e-5
        else:
            x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
            kn = kind in ("swapab_kn", "decode", "decode_swiglu", "library_kn")
            w = (torch.randn((k, n) if kn else (n, k), generator=g) * 0.05).to(torch.bfloat16).cuda()
            want = as_ref(x) @ (as_ref(w) if kn else as_ref(w).T)
            if kind in ("decode", "decode_swiglu"):
                features = rng.choice([128, 256])
                splits = rng.randint(1, 8) if features == 128 and kind == "decode" else 1
                epilogue = ops.DG_SWIGLU if kind == "decode_swiglu" else ops.DG_PLAIN
                if not ops.gemm_decode_supports(m, n, k, features, splits, epilogue):
                    continue
                if epilogue == ops.DG_SWIGLU:
                    want, out_dtype = want[:, 0::2] / (1 + torch.exp(-want[:, 0::2])) * want[:, 1::2], torch.bfloat16
                out = ops.gemm_decode(x, w, blank(want.shape[1], out_dtype), features=features, splits=splits, epilogue=epilogue,
                                      stages=rng.choice([0, 0, 1, 2, 3, 5, 9, 16]), error_word=err)
            elif kind in ("swapab", "swapab_kn"):
                if not ops.gemm_tcgen05_swapab_supports(m, n, k):
                    continue
                out = ops.gemm_tcgen05_swapab(x, w, blank(n, out_dtype), err, w_kn=kn)
            elif kind in ("library", "library_kn"):
                out = ops.library_gemm(x, w, blank(n, out_dtype), w_kn=kn)
            elif kind == "tcgen05":
                if not ops.gemm_tcgen05_supports(m, n, k):
                    continue
                out = ops.gemm_tcgen05(x, w, blank(n, out_dtype), err)
            else:
                if not ops.gemm_tcgen05_2cta_supports(m, n, k):
                    continue
                out = ops.gemm_tcgen05_2cta(x, w, blank(n, out_dtype), err)
            rel = 1.2e-2 if out.dtype == torch.bfloat16 else 2e-4
        what = (draw, kind, m, n, k, out.dtype)
        assert torch.isfinite(out).all(), what
        assert (as_ref(out) - want).abs().max() <= rel * want.abs().max() + 1e-6, what
        assert int(err) == 0, what
        ran[kind] = ran.get(kind, 0) + 1
    assert len(ran) == 9 and min(ran.values()) >= 5, ran
