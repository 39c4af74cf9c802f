"""Choice of the attention kernel for a step.

All kernels here read the ragged batch the same way: entry e owns the token
rows q_start[e] .. q_start[e+1]-1, its first query token stands at position
kv_start[e] of the request, and its pages are row slots[e] of the block table.
A kernel that does not take a shape is passed over: portions of prompts go to the
tcgen05 kernel (head size 64 or 128, pages of 8 .. 128 tokens), else to the
mma.sync kernel (head size 64 or 128, any page size); single tokens to the TMA
decode kernel (groups up to 16, pages of 8 .. 64), else to the cp.async one; and
what none of them takes to the CUDA-core kernel, which takes every shape and is
the only one used in 32-bit.  The choice itself is made by `tib_plan_attention` in
csrc/block.cu, which the native block call asks too.
"""
from __future__ import annotations

import torch

from torchinferno_b200.kernels import ops


# Portions of prompts go to the tcgen05 kernel where it takes the shape (set False to compare with mma.sync).
PREFILL_TCGEN05 = True


def _allow(rotates: bool) -> int:
    return (ops.ALLOW_DECODE_TMA | (ops.ALLOW_PREFILL_TCGEN05 if PREFILL_TCGEN05 else 0)
            | (ops.ALLOW_DECODE_ROTATES if rotates and DECODE_ROTATES else 0))


def _plan(ctx, heads: int, kv_heads: int, head_dim: int, rotates: bool) -> tuple[int, int]:
    batch, kv = ctx.batch, ctx.kv
    packed = kv.pool.dim() == 5 and kv.pool.stride(0) == 2 * kv_heads * kv.page_size * head_dim
    return ops.plan_attention(head_dim, heads // kv_heads, kv.page_size, packed, batch.n_entries, batch.n_single, batch.n_multi,
                              _allow(rotates))


def paged_attention(q: torch.Tensor, out: torch.Tensor, ctx, heads: int, kv_heads: int, head_dim: int,
                    scale: float, window: int | None) -> torch.Tensor:
    batch, kv = ctx.batch, ctx.kv
    win = int(window or 0)
    prefill, decode = _plan(ctx, heads, kv_heads, head_dim, False) if q.dtype == torch.bfloat16 else (ops.ATTENTION_SIMT,) * 2
    if prefill == ops.ATTENTION_SIMT:
        return ops.paged_attention_simt(
            q, kv.pool, out, batch.q_start, batch.kv_start, batch.slots, kv.block_table,
            batch.n_entries, batch.max_q_len, heads, kv_heads, head_dim, scale,
            window=win, error_word=ctx.error_word)
    args = (q, kv.pool, out, batch.q_start, batch.kv_start, batch.slots, kv.block_table, batch.n_entries)
    if prefill == ops.ATTENTION_PREFILL_TCGEN05:      # TMA tiles, S and O in TMEM (pages of 8 .. 128 tokens)
        ops.prefill_attention_tcgen05(*args, batch.max_q_len, heads, kv_heads, head_dim, scale, window=win,
                                      skip_single=batch.n_single > 0, error_word=ctx.error_word)
    elif prefill == ops.ATTENTION_PREFILL_MMA:
        ops.prefill_attention(*args, batch.max_q_len, heads, kv_heads, head_dim, scale, window=win,
                              skip_single=batch.n_single > 0)
    if decode != ops.ATTENTION_NONE:
        ops.decode_attention(*args, heads, kv_heads, head_dim, scale, batch.max_kv_len, window=win,
                             kernel="tma" if decode == ops.ATTENTION_DECODE_TMA else "cp_async", error_word=ctx.error_word)
    return out


# Single tokens go to the decode kernel unrotated where it can rotate and store them itself (set False to compare
# with the rotary kernel followed by the attention kernel); up to how many requests a step, the library says
# (tib_plan_attention in csrc/block.cu, with the measurements behind the number).
DECODE_ROTATES = True


def decode_takes_unrotated(x: torch.Tensor, ctx, heads: int, kv_heads: int, head_dim: int, position) -> bool:
    """Whether this step's attention can run as one kernel from the rows of the qkv product: a step of single tokens
    only, in bfloat16, a shape the TMA decode kernel takes, and a position encoding that is a rotary table."""
    if not (DECODE_ROTATES and x.dtype == torch.bfloat16 and hasattr(position, "rotary_table")) or ctx.batch.n_entries == 0:
        return False
    return _plan(ctx, heads, kv_heads, head_dim, True)[1] == ops.ATTENTION_DECODE_TMA_ROTATES


def decode_attention_unrotated(qkv: torch.Tensor, out: torch.Tensor, ctx, heads: int, kv_heads: int, head_dim: int,
                               scale: float, window: int | None, position) -> torch.Tensor:
    batch, kv = ctx.batch, ctx.kv
    inv_freq, rot_dim, interleaved = position.rotary_table()
    return ops.decode_attention_rope(qkv, kv.pool, out, batch.q_start, batch.kv_start, batch.slots, kv.block_table,
                                     batch.n_entries, heads, kv_heads, head_dim, scale, batch.max_kv_len, inv_freq,
                                     rot_dim=rot_dim, interleaved=interleaved, window=int(window or 0), error_word=ctx.error_word)
