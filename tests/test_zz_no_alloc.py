"""The decode-attention entry point that allocates nothing, called through its exported C symbol.

Some callers of the library cannot allocate device memory when they need attention (they run under
another framework's fixed memory plan, in a loop that may not enter the allocator, or as a plug-in
whose host forbids allocation after start-up).  For them ``tib_decode_attention_noalloc`` keeps the
split partials in an array inside the library.  It must give what the ordinary entry point gives,
call after call, although the array keeps the previous call's contents.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_longlong, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from torchinferno_b200.kernels.library import load_library
    lib = load_library()
    fn = lib.tib_decode_attention_noalloc
    fn.restype = c_int
    fn.argtypes = [c_void_p] * 7 + [c_int] * 6 + [c_int64, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p]
    lib.tib_decode_attention_noalloc_need.restype = c_longlong
    lib.tib_decode_attention_noalloc_need.argtypes = [c_int] * 4
    lib.tib_decode_attention_noalloc_capacity.restype = c_longlong
    return lib, fn


def _case(n, heads, kv_heads, d, page, contexts, seed):
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-c // page) for c in contexts]
    total = sum(pages_per) + 2
    pool = (torch.randn(total, 2, kv_heads, page, d, generator=g) * 0.7).to(torch.bfloat16).cuda()
    order = torch.randperm(total, generator=g).tolist()
    table = torch.full((n, max(pages_per)), -1, dtype=torch.int32)
    for r in range(n):
        for p in range(pages_per[r]):
            table[r, p] = order.pop()
    q = torch.randn(n, heads * d, generator=g).to(torch.bfloat16).cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    return q, pool, table.cuda(), i32(list(range(n + 1))), i32([c - 1 for c in contexts]), i32(list(range(n)))


def _call_noalloc(fn, q, pool, table, q_start, kv_start, slots, n, heads, kv_heads, d, splits, chunk):
    out = torch.full_like(q, float("nan"))
    longest = int(kv_start.max().item()) + 1
    torch.cuda.synchronize()
    allocations = torch.cuda.memory_stats()["allocation.all.allocated"]
    rc = _raw_call(fn, q, pool, out, table, q_start, kv_start, slots, n, heads, kv_heads, d, splits, chunk, longest)
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocations     # torch's allocator was not entered
    return rc, out


def _raw_call(fn, q, pool, out, table, q_start, kv_start, slots, n, heads, kv_heads, d, splits, chunk, longest=None):
    longest = int(kv_start.max().item()) + 1 if longest is None else longest
    return fn(q.data_ptr(), pool.data_ptr(), out.data_ptr(), q_start.data_ptr(), kv_start.data_ptr(), slots.data_ptr(),
            table.data_ptr(), table.stride(0), n, heads, kv_heads, d, pool.shape[3], pool.stride(0), pool.shape[0], 0,
            1.0 / math.sqrt(d), splits, chunk, longest, torch.cuda.current_stream().cuda_stream)


def test_noalloc_decode_attention_matches_the_ordinary_entry_point_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from torchinferno_b200.kernels import ops
    lib, fn = _symbol()
    cases = [  # two different calls in a row: the second finds the first one's partials in the array
        dict(n=5, heads=8, kv_heads=2, d=128, page=16, contexts=[900, 1, 64, 65, 517], splits=(4, 256), seed=1),
        dict(n=3, heads=4, kv_heads=2, d=64, page=4, contexts=[300, 129, 700], splits=(6, 128), seed=2),
        dict(n=5, heads=8, kv_heads=2, d=128, page=16, contexts=[900, 1, 64, 65, 517], splits=(4, 256), seed=1),
        dict(n=2, heads=8, kv_heads=8, d=64, page=16, contexts=[50, 64], splits=(1, 64), seed=3),
    ]
    for case in cases:
        n, heads, kv_heads, d = case["n"], case["heads"], case["kv_heads"], case["d"]
        q, pool, table, q_start, kv_start, slots = _case(n, heads, kv_heads, d, case["page"], case["contexts"], case["seed"])
        splits, chunk = case["splits"]
        want = ops.decode_attention(q, pool, torch.empty_like(q), q_start, kv_start, slots, table, n, heads, kv_heads, d,
                                    1.0 / math.sqrt(d), max(case["contexts"]), num_splits=splits, chunk=chunk)
        rc, got = _call_noalloc(fn, q, pool, table, q_start, kv_start, slots, n, heads, kv_heads, d, splits, chunk)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.isfinite(got).all()
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(got, want)                                         # the same kernels, the same order


def test_noalloc_decode_attention_refuses_what_does_not_fit():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    lib, fn = _symbol()
    capacity = lib.tib_decode_attention_noalloc_capacity()
    assert capacity == 4 * 1024 * 1024
    n, heads, kv_heads, d = 64, 32, 8, 128
    splits = 17
    assert lib.tib_decode_attention_noalloc_need(n, heads, d, splits) > capacity
    q, pool, table, q_start, kv_start, slots = _case(n, heads, kv_heads, d, 16, [70] * n, 4)
    rc, out = _call_noalloc(fn, q, pool, table, q_start, kv_start, slots, n, heads, kv_heads, d, splits, 64)
    torch.cuda.synchronize()
    assert rc == -7 and torch.isnan(out).all()            # refused, nothing was launched
    rc, _ = _call_noalloc(fn, q, pool, table, q_start, kv_start, slots, n, heads, kv_heads, 144, 1, 128)
    assert rc == -2                                        # a head size the kernel is not built for (steps of 16 up to 128)
    # parts that do not cover the longest context (70 keys in one part of 64) are refused, not run with keys left out
    rc, out = _call_noalloc(fn, q, pool, table, q_start, kv_start, slots, n, heads, kv_heads, d, 1, 64)
    assert rc == -2 and torch.isnan(out).all()
    out = torch.full_like(q, float("nan"))
    assert _raw_call(fn, q, pool, out, table, q_start, kv_start, slots, -1, heads, kv_heads, d, 2, 64) == -5
