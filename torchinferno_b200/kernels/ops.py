"""Python faces of the CUDA kernels.

Each function checks device, dtype, contiguity and shapes, then calls the C
entry point on torch's current stream.  A refusal by a kernel (a size it does
not take) raises :class:`KernelError`; nothing falls back to another path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from torchinferno_b200.kernels.library import load_library

F32, BF16 = 0, 1

_ERRORS = {
    -1: "unknown dtype code",
    -2: "a size this kernel does not take",
    -3: "a pointer or stride that is not aligned as required",
    -4: "needs more shared memory than an SM offers",
    -5: "null pointer or inconsistent arguments",
    -6: "the device-side wait limit was reached (kernel gave up)",
    -7: "needs more scratch than the library's built-in array holds",
}


class KernelError(RuntimeError):
    pass


_counter = {"launches": 0}


def set_dependent_launch(on: bool) -> bool:
    """Programmatic dependent launch of the library's small kernels (on by default): a kernel may be placed on
    the SMs while the one before it drains and waits there for its data.  Returns the setting before.  A
    captured graph keeps what was set when it was captured."""
    return bool(lib().tib_set_dependent_launch(c_int(1 if on else 0)))


KERNEL_CLASSES = ("norm", "qkv", "rope_append", "attention_prefill", "attention_decode", "o", "gate_up", "swiglu", "down")


def set_kernel_timers(on: bool) -> bool:
    """CUDA-event timers around every launch of a natively issued block, by kernel class (off by default; a step
    captured in a graph records nothing).  Returns the setting before."""
    return bool(lib().tib_kernel_timers(c_int(1 if on else 0)))


def read_kernel_timers(reset: bool = False) -> dict[str, dict[str, float]]:
    """{class: {"ms": total, "launches": n}} of what the timers have recorded; waits for the recorded events."""
    n = len(KERNEL_CLASSES)
    ms, counts = (ctypes.c_double * n)(), (ctypes.c_longlong * n)()
    lib().tib_kernel_timers_read(ms, counts, c_int(n), c_int(1 if reset else 0))
    return {name: {"ms": float(ms[i]), "launches": int(counts[i])} for i, name in enumerate(KERNEL_CLASSES)}


def count_launches(n: int) -> None:
    """Launches made by a native call that issues several kernels."""
    _counter["launches"] += n


def launch_count() -> int:
    """How many kernels of this library were launched by this process so far."""
    return _counter["launches"]


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"dtype {dtype} is not supported by the kernels (float32 or bfloat16)")


def _check(name: str, status: int) -> None:
    _counter["launches"] += 1
    if status == 0:
        return
    if status < 0:
        raise KernelError(f"{name}: refused: {_ERRORS.get(status, status)}")
    raise KernelError(f"{name}: CUDA error {status} at launch")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def _stream() -> c_void_p:
    # (the raw handle of the current stream of the current device: a fraction of the cost of
    # torch.cuda.current_stream(), which is asked for at every launch)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


_signatures_set = False


def lib() -> ctypes.CDLL:
    global _signatures_set
    library = load_library()
    if not _signatures_set:
        for fn in ("tib_embedding", "tib_add_rmsnorm", "tib_rmsnorm", "tib_swiglu", "tib_cast",
                   "tib_scatter_i32", "tib_decode_inputs", "tib_sample_records", "tib_rope_append", "tib_paged_attention_simt", "tib_gemm_f32", "tib_sample",
                   "tib_attention_mma_supports", "tib_prefill_attention", "tib_decode_attention",
                   "tib_prefill_attention_tcgen05", "tib_prefill_attention_tcgen05_supports",
                   "tib_decode_attention_tma", "tib_decode_attention_tma_rope", "tib_decode_attention_tma_supports", "tib_set_dependent_launch",
                   "tib_kernel_timers", "tib_kernel_timers_read",
                   "tib_blas_init", "tib_blas_gemm", "tib_gemm_tcgen05_2cta", "tib_gemm_tcgen05_2cta_supports",
                   "tib_gemm_tcgen05", "tib_gemm_tcgen05_supports",
                   "tib_gemm_tcgen05_swapab", "tib_gemm_tcgen05_swapab_supports", "tib_gemm_decode", "tib_gemm_decode_supports",
                   "tib_plan_attention", "tib_plan_product"):
            getattr(library, fn).restype = c_int
        _signatures_set = True
    return library


# ---------------------------------------------------------------------------
def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = float(table[ids[t]]): the residual stream starts in 32-bit."""
    _need(ids, "ids", torch.int32), _need(table, "table"), _need(out, "out", torch.float32)
    n, (vocab, hidden) = ids.numel(), table.shape
    if out.shape != (n, hidden):
        raise KernelError(f"embedding: out is {tuple(out.shape)}, wanted {(n, hidden)}")
    _check("embedding", lib().tib_embedding(_ptr(ids), _ptr(table), _ptr(out), c_int(n), c_int(hidden),
                                            c_int(vocab), c_int(_code(table.dtype)), _stream()))
    return out


def add_rmsnorm(delta: torch.Tensor | None, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
    """residual += delta (fp32, in place, when rows is None); out = rmsnorm(residual) * weight.

    With ``rows`` only those source rows are read, the residual is left as it
    is and ``out`` has one row per index.
    """
    _need(residual, "residual", torch.float32), _need(weight, "weight", torch.float32), _need(out, "out")
    hidden = residual.shape[-1]
    if delta is not None:
        _need(delta, "delta", out.dtype)
        if delta.shape != residual.shape:
            raise KernelError("add_rmsnorm: delta and residual differ in shape")
    if rows is not None:
        _need(rows, "rows", torch.int32)
    n_out = residual.shape[0] if rows is None else rows.numel()
    if out.shape != (n_out, hidden) or weight.numel() != hidden:
        raise KernelError(f"add_rmsnorm: out {tuple(out.shape)} / weight {tuple(weight.shape)} do not fit {(n_out, hidden)}")
    _check("add_rmsnorm", lib().tib_add_rmsnorm(_ptr(delta), _ptr(residual), _ptr(rows), _ptr(weight), _ptr(out),
                                                c_int(n_out), c_int(hidden), c_float(eps),
                                                c_int(_code(out.dtype)), _stream()))
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """RMSNorm over the last dimension of rows held in the activation type."""
    _need(x, "x"), _need(weight, "weight", torch.float32), _need(out, "out", x.dtype)
    hidden = x.shape[-1]
    n_rows = x.numel() // hidden if hidden else 0
    if out.shape != x.shape or weight.numel() != hidden:
        raise KernelError("rmsnorm: shapes do not fit")
    _check("rmsnorm", lib().tib_rmsnorm(_ptr(x), _ptr(weight), _ptr(out), c_int(n_rows), c_int(hidden),
                                        c_float(eps), c_int(_code(x.dtype)), _stream()))
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """out = silu(gate) * up, silu and product in fp32; a row of ``gate_up`` holds the I gates, then the I ups,
    or (``interleaved``) gate i and up i side by side."""
    _need(gate_up, "gate_up"), _need(out, "out", gate_up.dtype)
    n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2):
        raise KernelError("swiglu: shapes do not fit")
    _check("swiglu", lib().tib_swiglu(_ptr(gate_up), _ptr(out), c_int(n), c_int(two_i // 2),
                                      c_int(_code(gate_up.dtype)), c_int(int(interleaved)), _stream()))
    return out


def cast(x: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(x, "x"), _need(out, "out")
    if x.numel() != out.numel():
        raise KernelError("cast: sizes differ")
    _check("cast", lib().tib_cast(_ptr(x), _ptr(out), c_int64(x.numel()), c_int(_code(x.dtype)),
                                  c_int(_code(out.dtype)), _stream()))
    return out


def rope_append(qkv: torch.Tensor, q_out: torch.Tensor, pool: torch.Tensor | None, positions: torch.Tensor,
                token_slot: torch.Tensor | None, block_table: torch.Tensor | None, inv_freq: torch.Tensor,
                heads: int, kv_heads: int, head_dim: int, *, rot_dim: int | None = None,
                interleaved: bool = False, write_kv: bool = True,
                error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate q into ``q_out``; rotate k and copy v into the layer's pages.

    ``qkv``: [tokens, (heads + 2 kv_heads) * head_dim]; ``pool``: the layer's pages
    [pages, 2, kv_heads, page_size, head_dim]; ``block_table``: [slots, max_pages] int32.
    """
    _need(qkv, "qkv"), _need(q_out, "q_out", qkv.dtype), _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    n = qkv.shape[0]
    rot = head_dim if rot_dim is None else rot_dim
    if qkv.shape[1] != (heads + 2 * kv_heads) * head_dim or q_out.numel() != n * heads * head_dim:
        raise KernelError("rope_append: qkv / q_out widths do not fit the head counts")
    if inv_freq.numel() != rot // 2 or positions.numel() != n:
        raise KernelError("rope_append: inv_freq or positions have the wrong length")
    page_size = page_stride = num_pages = table_stride = 0
    if write_kv:
        if pool is None or token_slot is None or block_table is None:
            raise KernelError("rope_append: pool, token_slot and block_table are needed to write the cache")
        _need(pool, "pool", qkv.dtype), _need(token_slot, "token_slot", torch.int32)
        _need(block_table, "block_table", torch.int32)
        if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
            raise KernelError(f"rope_append: pool shape {tuple(pool.shape)} does not fit")
        num_pages, page_size = pool.shape[0], pool.shape[3]
        page_stride = pool.stride(0)
        table_stride = block_table.stride(0)
    _check("rope_append", lib().tib_rope_append(
        _ptr(qkv), _ptr(q_out), _ptr(pool), _ptr(positions), _ptr(token_slot), _ptr(block_table),
        c_int(table_stride), _ptr(inv_freq), c_int(n), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(rot), c_int(int(interleaved)), c_int(page_size), c_int64(page_stride), c_int(num_pages),
        c_int(int(write_kv)), _ptr(error_word), c_int(_code(qkv.dtype)), _stream()))
    return q_out


def paged_attention_simt(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                         kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor,
                         n_entries: int, max_q_len: int, heads: int, kv_heads: int, head_dim: int,
                         scale: float, window: int = 0, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of a ragged batch over the paged cache, on CUDA cores."""
    _need(q, "q"), _need(pool, "pool", q.dtype), _need(out, "out", q.dtype)
    for name, t in (("q_start", q_start), ("kv_start", kv_start), ("slots", slots), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
        raise KernelError(f"paged_attention: pool shape {tuple(pool.shape)} does not fit")
    if q.numel() != out.numel() or q.numel() % (heads * head_dim):
        raise KernelError("paged_attention: q / out do not fit the head counts")
    if q_start.numel() < n_entries + 1 or kv_start.numel() < n_entries or slots.numel() < n_entries:
        raise KernelError("paged_attention: entry arrays are shorter than n_entries")
    _check("paged_attention_simt", lib().tib_paged_attention_simt(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(heads), c_int(kv_heads),
        c_int(head_dim), c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window),
        c_float(scale), _ptr(error_word), c_int(_code(q.dtype)), _stream()))
    return out


def gemm_f32(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] (fp32) = x[M, K] . w[N, K]^T with fp32 FMAs in fixed k order."""
    _need(out, "out", torch.float32)
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.stride(-1) != 1 or t.dim() != 2:
            raise KernelError(f"gemm_f32: {name} must be a 2-D CUDA tensor with unit inner stride")
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_f32: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_f32", lib().tib_gemm_f32(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k),
                                          c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)),
                                          c_int(_code(x.dtype)), c_int(_code(w.dtype)), _stream()))
    return out


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: torch.Tensor | None = None,
           seeds: torch.Tensor | None = None, positions: torch.Tensor | None = None) -> torch.Tensor:
    """Token ids from fp32 logits: greedy where temperature <= 0, else seeded Gumbel-max."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a 2-D fp32 CUDA tensor with unit inner stride")
    _need(out, "out", torch.int32)
    n, vocab = logits.shape
    if temperature is not None:
        _need(temperature, "temperature", torch.float32)
    if seeds is not None:
        _need(seeds, "seeds", torch.int64)
    if positions is not None:
        _need(positions, "positions", torch.int32)
    for t in (temperature, seeds, positions):
        if t is not None and t.numel() < n:
            raise KernelError("sample: a per-row array is shorter than the number of rows")
    if out.numel() < n:
        raise KernelError("sample: out is too short")
    _check("sample", lib().tib_sample(_ptr(logits), c_int64(logits.stride(0)), _ptr(temperature), _ptr(seeds),
                                      _ptr(positions), _ptr(out), c_int(n), c_int(vocab), _stream()))
    return out


def scatter_i32(dst: torch.Tensor, index: torch.Tensor, value: torch.Tensor) -> torch.Tensor:
    """dst.view(-1)[index[i]] = value[i]; applies queued block-table changes."""
    _need(dst, "dst", torch.int32), _need(index, "index", torch.int32), _need(value, "value", torch.int32)
    if index.numel() != value.numel():
        raise KernelError("scatter_i32: index and value differ in length")
    _check("scatter_i32", lib().tib_scatter_i32(_ptr(dst), _ptr(index), _ptr(value), c_int(index.numel()),
                                                c_int64(dst.numel()), _stream()))
    return dst


RECORD_WORDS = 8          # int32 words of a request's record (csrc/common.cuh: TibRequestRecord)
REC_LENGTH, REC_LAST_TOKEN, REC_SEED_LO, REC_SEED_HI, REC_TEMPERATURE, REC_DRAWN = range(6)


def _need_records(records: torch.Tensor) -> None:
    _need(records, "records", torch.int32)
    if records.dim() != 2 or records.shape[1] != RECORD_WORDS:
        raise KernelError(f"records must be [slots, {RECORD_WORDS}] int32")


def sample_records(logits: torch.Tensor, out: torch.Tensor, records: torch.Tensor, record_slots: torch.Tensor,
                   history: torch.Tensor | None = None) -> torch.Tensor:
    """As :func:`sample`, every row's temperature, seed and position taken from the record of its request
    (``record_slots[row]``); the drawn token also goes into that record as the request's next input token."""
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be a 2-D fp32 CUDA tensor with unit inner stride")
    _need(out, "out", torch.int32), _need_records(records), _need(record_slots, "record_slots", torch.int32)
    n, vocab = logits.shape
    if history is not None:
        _need(history, "history", torch.int32)
    if out.numel() < n or record_slots.numel() < n or (history is not None and history.numel() < n):
        raise KernelError("sample: a per-row array is shorter than the number of rows")
    _check("sample", lib().tib_sample_records(_ptr(logits), c_int64(logits.stride(0)), _ptr(records), _ptr(record_slots),
                                              c_int(records.shape[0]), _ptr(out), _ptr(history), c_int(n), c_int(vocab), _stream()))
    return out


def decode_inputs(records: torch.Tensor, slots: torch.Tensor, token_ids: torch.Tensor, positions: torch.Tensor) -> None:
    """token_ids[i], positions[i] = next token and position of the request in slot slots[i]; its record moves on by one."""
    n = slots.numel()
    _need_records(records)
    for name, t in (("slots", slots), ("token_ids", token_ids), ("positions", positions)):
        _need(t, name, torch.int32)
        if t.numel() < n:
            raise KernelError(f"decode_inputs: {name} is shorter than slots")
    _check("decode_inputs", lib().tib_decode_inputs(_ptr(records), _ptr(slots), c_int(records.shape[0]), _ptr(token_ids),
                                                    _ptr(positions), c_int(n), _stream()))


def attention_mma_supports(head_dim: int, group: int) -> bool:
    """Whether the tensor-core attention kernels are built for this head size and group size."""
    return bool(lib().tib_attention_mma_supports(c_int(head_dim), c_int(group)))


def _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim):
    _need(q, "q", torch.bfloat16), _need(pool, "pool", torch.bfloat16), _need(out, "out", torch.bfloat16)
    for name, t in (("q_start", q_start), ("kv_start", kv_start), ("slots", slots), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
        raise KernelError(f"attention: pool shape {tuple(pool.shape)} does not fit")
    if q.numel() != out.numel() or q.numel() % (heads * head_dim):
        raise KernelError("attention: q / out do not fit the head counts")
    if q_start.numel() < n_entries + 1 or kv_start.numel() < n_entries or slots.numel() < n_entries:
        raise KernelError("attention: entry arrays are shorter than n_entries")


def prefill_attention(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                      kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                      max_q_len: int, heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0,
                      skip_single: bool = False) -> torch.Tensor:
    """Causal attention of prompt portions over the paged cache on tensor cores (bf16)."""
    _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim)
    _check("prefill_attention", lib().tib_prefill_attention(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
        c_int(int(skip_single)), _stream()))
    return out


def decode_split(n_entries: int, heads: int, kv_heads: int, max_kv_len: int, target_blocks: int = 148) -> tuple[int, int]:
    """(num_splits, chunk) for a known longest context: about ``target_blocks`` blocks, two tiles a split at least."""
    group = heads // kv_heads
    blocks = max(1, n_entries * kv_heads * ((group + 15) // 16))
    tiles = max(1, -(-max_kv_len // 64))
    splits = max(1, min(-(-tiles // 2), -(-target_blocks // blocks)))
    per = -(-tiles // splits)
    return -(-tiles // per), per * 64


# What tib_plan_attention answers (csrc/block.cu), and what it may be allowed to use.
ATTENTION_NONE, ATTENTION_PREFILL_TCGEN05, ATTENTION_PREFILL_MMA, ATTENTION_DECODE_TMA_ROTATES, ATTENTION_DECODE_TMA, \
    ATTENTION_DECODE_CP_ASYNC, ATTENTION_SIMT = range(7)
ALLOW_PREFILL_TCGEN05, ALLOW_DECODE_ROTATES, ALLOW_DECODE_TMA = 1, 2, 4
PRODUCT_LIBRARY, PRODUCT_DECODE, PRODUCT_SWAPAB = 0, 1, 2


def plan_attention(head_dim: int, group: int, page_size: int, packed: bool, n_entries: int, n_single: int, n_multi: int,
                   allow: int) -> tuple[int, int]:
    """(kernel for the portions of prompts, kernel for the single tokens) of a bfloat16 step, as the CUDA library
    chooses them: the one place where that is decided, for the part-by-part sequence and the native block alike."""
    prefill, decode = c_int(0), c_int(0)
    _check("plan_attention", lib().tib_plan_attention(c_int(head_dim), c_int(group), c_int(page_size), c_int(int(packed)),
                                                      c_int(n_entries), c_int(n_single), c_int(n_multi), c_int(allow),
                                                      ctypes.byref(prefill), ctypes.byref(decode)))
    return prefill.value, decode.value


def plan_product(rows: int, n: int, k: int, kn: bool, few_rows: int, features: int, splits: int, swiglu: bool,
                 aligned: bool) -> int:
    """The kernel a bf16 product of ``rows`` rows goes to (PRODUCT_*), chosen in the same place for both ways of
    running a block."""
    return int(lib().tib_plan_product(c_int(rows), c_int(n), c_int(k), c_int(int(kn)), c_int(few_rows), c_int(features),
                                      c_int(splits), c_int(int(swiglu)), c_int(int(aligned))))


def decode_num_splits(n_entries: int, heads: int, kv_heads: int, max_kv_len: int | None = None,
                      target_blocks: int = 256, slots: int = 296) -> int:
    """How many parts the grid provides for each request's context when the kernel sizes the parts itself.

    Measured on the B200 at 3,072 tokens of context (32 heads, 8 kv heads of 128): the kernel is fastest
    with about 256 blocks in all, just under the two per SM that fit (batch 1: 16 parts, 2: 8 to 16, 4: 8,
    8: 4, 16: 2, 32 and up: 1); more than 16 parts cost more in the merge than they gain, except where the
    context may be long (``max_kv_len`` above 8,192: one request at 32,768 tokens streams at 3.1 TB/s in 16
    parts, 128 blocks), where up to 32 are provided.  The TMA kernel uses only as many of them as the
    request's own context has stretches of 192 keys.

    ``slots``: the blocks that run at once (two on each of 148 SMs).  A batch a little larger than that would run
    one full round and a nearly empty second one; cut in two or three parts its blocks are more and shorter rounds
    (2,100 tokens of context, 38 / 44 / 48 / 52 requests: 95 / 99 / 101 / 103 us in one part, 85 / 91 / 95 / 105 in
    three, 89 / 94 / 95 / 99 in two; from 56 requests on, and past two rounds, one part is fastest again)."""
    group = heads // kv_heads
    blocks = max(1, n_entries * kv_heads * ((group + 15) // 16))
    if slots < blocks < 2 * slots:
        last_round = blocks / slots - 1            # how full the second round would be
        if last_round <= 0.2:
            return 3
        if last_round <= 0.45:
            return 2
    most = 32 if max_kv_len is not None and max_kv_len > 8192 else 16
    return max(1, min(most, target_blocks // blocks))


def decode_attention(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                     kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                     heads: int, kv_heads: int, head_dim: int, scale: float, max_kv_len: int, window: int = 0,
                     scratch: torch.Tensor | None = None, num_splits: int | None = None,
                     chunk: int | None = None, kernel: str = "auto", error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of single tokens over the paged cache, the context split over blocks (bf16).

    ``kernel``: "tma" (keys and values copied by the TMA unit; see ``decode_attention_tma_supports``),
    "cp_async" (every key row fetched by its own address; any page size), or "auto": the first where
    it takes the shape.

    Entries that bring more than one token are skipped.  ``max_kv_len`` bounds the longest context
    (keys 0 .. position) of the batch when ``num_splits`` and ``chunk`` are given (by default the kernel
    cuts each request's own context into equal parts); ``scratch`` (fp32, at least n_entries * heads * num_splits *
    (head_dim + 2) elements) holds the partial results when there is more than one split.
    """
    _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim)
    if num_splits is None or chunk is None:
        # each request's own context is cut into num_splits equal parts by the kernel (chunk 0)
        num_splits, chunk = decode_num_splits(n_entries, heads, kv_heads, max_kv_len), 0
    elif chunk != 0 and num_splits * chunk < max_kv_len:
        raise KernelError("decode_attention: num_splits * chunk does not cover the longest context")
    scratch_o = scratch_ml = None
    if num_splits > 1:
        need = n_entries * heads * num_splits * (head_dim + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError("decode_attention: scratch is too small")
        scratch_o = scratch
        scratch_ml = scratch[n_entries * heads * num_splits * head_dim:]
    if kernel not in ("auto", "tma", "cp_async"):
        raise KernelError(f"decode_attention: no kernel {kernel!r}")
    packed = pool.stride(0) == 2 * kv_heads * pool.shape[3] * head_dim
    tma = plan_attention(head_dim, heads // kv_heads, pool.shape[3], packed, n_entries, n_entries, 0,
                         0 if kernel == "cp_async" else ALLOW_DECODE_TMA)[1] == ATTENTION_DECODE_TMA
    if kernel == "tma" and not tma:
        raise KernelError("decode_attention: the TMA kernel does not take this shape "
                          f"(head_dim {head_dim}, group {heads // kv_heads}, pages of {pool.shape[3]}, packed={packed})")
    if tma:
        _check("decode_attention_tma", lib().tib_decode_attention_tma(
            _ptr(q), _ptr(pool), _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), _ptr(q_start), _ptr(kv_start), _ptr(slots),
            _ptr(block_table), c_int(block_table.stride(0)), c_int(n_entries), c_int(heads), c_int(kv_heads), c_int(head_dim),
            c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
            c_int(num_splits), c_int(chunk), _ptr(_split_counters(q.device, n_entries * kv_heads) if num_splits > 1 else None),
            _ptr(error_word), _stream()))
        return out
    _check("decode_attention", lib().tib_decode_attention(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), _ptr(q_start), _ptr(kv_start), _ptr(slots),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(n_entries), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
        c_int(num_splits), c_int(chunk), _stream()))
    return out


def decode_attention_rope(qkv: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                          kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                          heads: int, kv_heads: int, head_dim: int, scale: float, max_kv_len: int, inv_freq: torch.Tensor,
                          *, rot_dim: int | None = None, interleaved: bool = False, window: int = 0,
                          scratch: torch.Tensor | None = None, num_splits: int | None = None,
                          error_word: torch.Tensor | None = None) -> torch.Tensor:
    """A step of single tokens straight from the rows of the qkv product: the TMA decode kernel rotates the queries,
    rotates each token's key and writes it and the value into the token's page, then attends
    (:func:`rope_append` followed by :func:`decode_attention`, in one kernel and bit for bit).  Every entry must bring
    one token; needs a shape the TMA kernel takes (``decode_attention_tma_supports``)."""
    _need(qkv, "qkv", torch.bfloat16), _need(pool, "pool", torch.bfloat16), _need(out, "out", torch.bfloat16)
    _need(inv_freq, "inv_freq", torch.float32)
    for name, t in (("q_start", q_start), ("kv_start", kv_start), ("slots", slots), ("block_table", block_table)):
        _need(t, name, torch.int32)
    rot = head_dim if rot_dim is None else rot_dim
    if pool.dim() != 5 or pool.shape[1] != 2 or pool.shape[2] != kv_heads or pool.shape[4] != head_dim:
        raise KernelError(f"attention: pool shape {tuple(pool.shape)} does not fit")
    if qkv.dim() != 2 or qkv.shape[1] != (heads + 2 * kv_heads) * head_dim or out.shape != (qkv.shape[0], heads * head_dim):
        raise KernelError("decode_attention_rope: qkv / out do not fit the head counts")
    if inv_freq.numel() != rot // 2:
        raise KernelError("decode_attention_rope: inv_freq has the wrong length")
    if q_start.numel() < n_entries + 1 or kv_start.numel() < n_entries or slots.numel() < n_entries:
        raise KernelError("attention: entry arrays are shorter than n_entries")
    packed = pool.stride(0) == 2 * kv_heads * pool.shape[3] * head_dim
    if not (packed and decode_attention_tma_supports(head_dim, heads // kv_heads, pool.shape[3])):
        raise KernelError("decode_attention_rope: the TMA kernel does not take this shape")
    if num_splits is None:
        num_splits = decode_num_splits(n_entries, heads, kv_heads, max_kv_len)
    scratch_o = scratch_ml = None
    if num_splits > 1:
        need = n_entries * heads * num_splits * (head_dim + 2)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError("decode_attention: scratch is too small")
        scratch_o, scratch_ml = scratch, scratch[n_entries * heads * num_splits * head_dim:]
    _check("decode_attention_tma_rope", lib().tib_decode_attention_tma_rope(
        _ptr(qkv), _ptr(pool), _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), _ptr(q_start), _ptr(kv_start), _ptr(slots),
        _ptr(block_table), c_int(block_table.stride(0)), c_int(n_entries), c_int(heads), c_int(kv_heads), c_int(head_dim),
        c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]), c_int(window), c_float(scale),
        c_int(num_splits), c_int(0), _ptr(_split_counters(qkv.device, n_entries * kv_heads) if num_splits > 1 else None),
        _ptr(error_word), _ptr(inv_freq), c_int(rot), c_int(int(interleaved)), _stream()))
    return out


_counters: dict[torch.device, torch.Tensor] = {}
_COUNTERS = 65536     # allocated once per device, outside any graph capture that may come later


def _split_counters(device: torch.device, n: int) -> torch.Tensor | None:
    """Zeroed ints in which the parts of a split context count themselves in (the kernel leaves them zero).
    One buffer per device: launches on one stream follow one another."""
    if n > _COUNTERS:
        return None            # (the kernel then merges with a second launch)
    have = _counters.get(device)
    if have is None:
        have = _counters[device] = torch.zeros(_COUNTERS, dtype=torch.int32, device=device)
    return have


def decode_attention_tma_supports(head_dim: int, group: int, page_size: int) -> bool:
    return bool(lib().tib_decode_attention_tma_supports(c_int(head_dim), c_int(group), c_int(page_size)))


_blas_workspace: dict[int, torch.Tensor] = {}
BLAS_WORKSPACE_BYTES = 32 << 20


def library_gemm_ready(device: torch.device) -> None:
    """Make the cuBLAS handle of ``device`` and give it its workspace (once)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _blas_workspace:
        buffer = torch.empty(BLAS_WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        with torch.cuda.device(index):
            status = lib().tib_blas_init(_ptr(buffer), ctypes.c_size_t(buffer.numel()))
        if status:
            raise KernelError(f"library_gemm: cuBLAS could not be set up (status {status})")
        _blas_workspace[index] = buffer


def library_gemm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, w_kn: bool) -> torch.Tensor:
    """out[M, N] (bf16 or fp32) = x[M, K] . w^T by cuBLAS, called from the engine's own library: ``w`` is stored
    [N, K], or [K, N] when ``w_kn``.  The library's workspace is a buffer of this module, made at the first call on
    a device (make that call outside a stream capture)."""
    library_gemm_ready(x.device)
    m, k = x.shape
    n = w.shape[1] if w_kn else w.shape[0]
    if (w.shape[0] if w_kn else w.shape[1]) != k or out.shape != (m, n):
        raise KernelError(f"library_gemm: shapes {tuple(x.shape)}, {tuple(w.shape)} (kn={w_kn}), {tuple(out.shape)} do not fit")
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.stride(1) != 1 or w.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("library_gemm: bf16 operands with unit inner stride are needed")
    status = lib().tib_blas_gemm(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)),
                                 c_int64(w.stride(0)), c_int64(out.stride(0)), c_int(1 if w_kn else 0),
                                 c_int(_code(out.dtype)), _stream())
    if status:
        raise KernelError(f"library_gemm: status {status} (20000 + n: cuBLAS status n)")
    return out        # (a library kernel: not counted among this library's launches)


def gemm_tcgen05_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().tib_gemm_tcgen05_supports(c_int(m), c_int(n), c_int(k)))


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] (bf16 or fp32) = x[M, K] . w[N, K]^T on tcgen05 tensor cores (TMA loads, TMEM accumulator)."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tcgen05: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_tcgen05: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_tcgen05", lib().tib_gemm_tcgen05(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k),
                                                  c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)),
                                                  c_int(_code(out.dtype)), _ptr(error_word), _stream()))
    return out


def gemm_tcgen05_2cta_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().tib_gemm_tcgen05_2cta_supports(c_int(m), c_int(n), c_int(k)))


def gemm_tcgen05_2cta(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] (bf16 or fp32) = x[M, K] . w[N, K]^T on pairs of SMs (`tcgen05.mma.cta_group::2`, 256 x 256 tiles)."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tcgen05_2cta: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    (m, k), (n, k2) = x.shape, w.shape
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_tcgen05_2cta: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_tcgen05_2cta", lib().tib_gemm_tcgen05_2cta(_ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k),
                                                            c_int64(x.stride(0)), c_int64(w.stride(0)), c_int64(out.stride(0)),
                                                            c_int(_code(out.dtype)), _ptr(error_word), _stream()))
    return out


def gemm_tcgen05_swapab_supports(m: int, n: int, k: int) -> bool:
    return bool(lib().tib_gemm_tcgen05_swapab_supports(c_int(m), c_int(n), c_int(k)))


def gemm_tcgen05_swapab(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, error_word: torch.Tensor | None = None,
                        splits: int = 0, w_kn: bool = False) -> torch.Tensor:
    """out[M, N] = x[M, K] . w^T for M <= 64 on tcgen05 tensor cores with the operands swapped: w ([N, K], or
    [K, N] with ``w_kn``) is streamed by TMA as the 128-row operand, K is split over a thread-block cluster
    (``splits`` = 0: chosen by the library) and the partial tiles are summed through distributed shared memory."""
    for name, t in (("x", x), ("w", w)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_tcgen05_swapab: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    m, k = x.shape
    k2, n = w.shape if w_kn else (w.shape[1], w.shape[0])
    if k != k2 or out.shape != (m, n):
        raise KernelError(f"gemm_tcgen05_swapab: shapes {tuple(x.shape)} x {tuple(w.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_tcgen05_swapab", lib().tib_gemm_tcgen05_swapab(
        _ptr(x), _ptr(w), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)), c_int64(w.stride(0)),
        c_int64(out.stride(0)), c_int(int(w_kn)), c_int(_code(out.dtype)), c_int(splits), _ptr(error_word), _stream()))
    return out


DG_PLAIN, DG_SWIGLU = 0, 1


def gemm_decode_supports(m: int, n: int, k: int, features: int = 128, splits: int = 1, epilogue: int = DG_PLAIN) -> bool:
    return bool(lib().tib_gemm_decode_supports(c_int(m), c_int(n), c_int(k), c_int(features), c_int(splits), c_int(epilogue)))


def gemm_decode(x: torch.Tensor, w_kn: torch.Tensor, out: torch.Tensor, *, features: int = 128, splits: int = 1,
                epilogue: int = DG_PLAIN, stages: int = 0, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """The product of a decode step, out[M, N] = x[M, K] . w for M <= 64 with ``w_kn`` stored [K, N]: tiles of
    ``features`` (128 or 256) features streamed by TMA through a ring of ``stages`` stages (0: the kernel's default),
    K shared by ``splits`` blocks of a cluster.  With the SwiGLU
    epilogue ``w_kn`` holds gate and up columns interleaved and ``out`` is the activation [M, N / 2]."""
    for name, t in (("x", x), ("w_kn", w_kn)):
        if not t.is_cuda or t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
            raise KernelError(f"gemm_decode: {name} must be a 2-D bf16 CUDA tensor with unit inner stride")
    _need(out, "out")
    (m, k), (k2, n) = x.shape, w_kn.shape
    if k != k2 or out.shape != (m, n // 2 if epilogue == DG_SWIGLU else n):
        raise KernelError(f"gemm_decode: shapes {tuple(x.shape)} x {tuple(w_kn.shape)} -> {tuple(out.shape)} do not fit")
    _check("gemm_decode", lib().tib_gemm_decode(
        _ptr(x), _ptr(w_kn), _ptr(out), c_int(m), c_int(n), c_int(k), c_int64(x.stride(0)), c_int64(w_kn.stride(0)),
        c_int64(out.stride(0)), c_int(_code(out.dtype)), c_int(features), c_int(splits), c_int(epilogue), c_int(stages),
        _ptr(error_word), _stream()))
    return out


def prefill_attention_tcgen05_supports(head_dim: int, group: int, page_size: int) -> bool:
    return bool(lib().tib_prefill_attention_tcgen05_supports(c_int(head_dim), c_int(group), c_int(page_size)))


def prefill_attention_tcgen05(q: torch.Tensor, pool: torch.Tensor, out: torch.Tensor, q_start: torch.Tensor,
                              kv_start: torch.Tensor, slots: torch.Tensor, block_table: torch.Tensor, n_entries: int,
                              max_q_len: int, heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0,
                              skip_single: bool = False, error_word: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of prompt portions over the paged cache on tcgen05 tensor cores (bf16): S and O in
    TMEM, Q / K / V tiles by TMA, softmax in fp32 by one thread per row."""
    _check_attention_args(q, pool, out, q_start, kv_start, slots, block_table, n_entries, heads, kv_heads, head_dim)
    _check("prefill_attention_tcgen05", lib().tib_prefill_attention_tcgen05(
        _ptr(q), _ptr(pool), _ptr(out), _ptr(q_start), _ptr(kv_start), _ptr(slots), _ptr(block_table),
        c_int(block_table.stride(0)), c_int(n_entries), c_int(max_q_len), c_int(q.numel() // (heads * head_dim)),
        c_int(heads), c_int(kv_heads), c_int(head_dim), c_int(pool.shape[3]), c_int64(pool.stride(0)), c_int(pool.shape[0]),
        c_int(window), c_float(scale), c_int(int(skip_single)), _ptr(error_word), _stream()))
    return out
