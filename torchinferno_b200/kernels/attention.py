"""Choice of the attention kernel for a step.

All kernels here read the ragged batch the same way: entry e owns the token
rows q_start[e] .. q_start[e+1]-1, its first query token stands at position
kv_start[e] of the request, and its pages are row slots[e] of the block table.
A kernel that does not take a shape is passed over: portions of prompts go to the
tcgen05 kernel (head size 64 or 128, pages of 8 .. 128 tokens), else to the
mma.sync kernel (head size 64 or 128, any page size); single tokens to the TMA
decode kernel (groups up to 16, pages of 8 .. 64), else to the cp.async one; and
what none of them takes to the CUDA-core kernel, which takes every shape and is
the only one used in 32-bit.  (A block of the built-in parts makes the same
choices in csrc/block.cu.)
"""
from __future__ import annotations

import torch

from torchinferno_b200.kernels import ops


# Portions of prompts go to the tcgen05 kernel where it takes the shape (set False to compare with mma.sync).
PREFILL_TCGEN05 = True


def paged_attention(q: torch.Tensor, out: torch.Tensor, ctx, heads: int, kv_heads: int, head_dim: int,
                    scale: float, window: int | None) -> torch.Tensor:
    batch, kv = ctx.batch, ctx.kv
    win = int(window or 0)
    if q.dtype == torch.bfloat16 and ops.attention_mma_supports(head_dim, heads // kv_heads):
        args = (q, kv.pool, out, batch.q_start, batch.kv_start, batch.slots, kv.block_table, batch.n_entries)
        if batch.n_multi:
            if (PREFILL_TCGEN05 and ops.prefill_attention_tcgen05_supports(head_dim, heads // kv_heads, kv.page_size)
                    and kv.pool.stride(0) == 2 * kv_heads * kv.page_size * head_dim):
                # TMA tiles, S and O in TMEM (pages of 8 .. 128 tokens)
                ops.prefill_attention_tcgen05(*args, batch.max_q_len, heads, kv_heads, head_dim, scale, window=win,
                                              skip_single=batch.n_single > 0, error_word=ctx.error_word)
            else:
                ops.prefill_attention(*args, batch.max_q_len, heads, kv_heads, head_dim, scale, window=win,
                                      skip_single=batch.n_single > 0)
        if batch.n_single:
            ops.decode_attention(*args, heads, kv_heads, head_dim, scale, batch.max_kv_len, window=win,
                                 error_word=ctx.error_word)
        return out
    return ops.paged_attention_simt(
        q, kv.pool, out, batch.q_start, batch.kv_start, batch.slots, kv.block_table,
        batch.n_entries, batch.max_q_len, heads, kv_heads, head_dim, scale,
        window=win, error_word=ctx.error_word)


# Single tokens go to the decode kernel unrotated where it can rotate and store them itself (set False to compare
# with the rotary kernel followed by the attention kernel), in steps of up to DECODE_ROTATES_MAX_ENTRIES requests.
# With few requests the step is a chain of short kernels and one link less is a gain (8 requests at 2,100 tokens,
# 8B sizes: 3.54 -> 3.51 ms a step); with many the attention kernel streams long enough that the head start it had
# under the rotary kernel (older keys are fetched while that runs) is worth more than the link (32 requests:
# 4.47 -> 4.52 ms, 64: 5.92 -> 6.01; 4 and 16: no difference).
DECODE_ROTATES = True
DECODE_ROTATES_MAX_ENTRIES = 8


def decode_takes_unrotated(x: torch.Tensor, ctx, heads: int, kv_heads: int, head_dim: int, position) -> bool:
    """Whether this step's attention can run as one kernel from the rows of the qkv product: a step of single tokens
    only, in bfloat16, a shape the TMA decode kernel takes, and a position encoding that is a rotary table."""
    batch, kv = ctx.batch, ctx.kv
    return (DECODE_ROTATES and x.dtype == torch.bfloat16 and batch.n_multi == 0
            and 0 < batch.n_single == batch.n_entries <= DECODE_ROTATES_MAX_ENTRIES
            and hasattr(position, "rotary_table") and kv.pool.dim() == 5
            and kv.pool.stride(0) == 2 * kv_heads * kv.page_size * head_dim
            and ops.decode_attention_tma_supports(head_dim, heads // kv_heads, kv.page_size))


def decode_attention_unrotated(qkv: torch.Tensor, out: torch.Tensor, ctx, heads: int, kv_heads: int, head_dim: int,
                               scale: float, window: int | None, position) -> torch.Tensor:
    batch, kv = ctx.batch, ctx.kv
    inv_freq, rot_dim, interleaved = position.rotary_table()
    return ops.decode_attention_rope(qkv, kv.pool, out, batch.q_start, batch.kv_start, batch.slots, kv.block_table,
                                     batch.n_entries, heads, kv_heads, head_dim, scale, batch.max_kv_len, inv_freq,
                                     rot_dim=rot_dim, interleaved=interleaved, window=int(window or 0), error_word=ctx.error_word)
