"""Rotary position encoding with an optional frequency-scaling law.

inv_freq[i] = theta^(-2i/rot) for i in [0, rot/2)
(src/torchinferno/models/llama3/pipeline.py:532-536); the llama3 law rescales
the table by wavelength bands (pipeline.py:537-552).  Angles, cos and sin are
fp32 and are computed in the kernel from integer positions and this table, so
another scaling law is another table.  Pairing is rotate-half (i, i + rot/2) by
default (pipeline.py:562-568) or interleaved (2i, 2i+1).  K is cached after
rotation, V unrotated (src/torchinferno/models/llama3/tensor_parallel.py:7416-7420).
"""
from __future__ import annotations

import math
from typing import Any, Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.parts.base import LayerContext, PositionEncoding, register_part


def rotary_frequencies(rot_dim: int, theta: float, scaling: Mapping[str, Any] | None = None) -> torch.Tensor:
    """The fp32 frequency table [rot_dim / 2], on the CPU."""
    exponent = torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim
    inv_freq = 1.0 / (theta ** exponent)
    if not scaling:
        return inv_freq
    kind = scaling.get("rope_type")
    if kind != "llama3":
        raise ValueError(f"unknown rotary scaling law {kind!r}")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    low_wavelen, high_wavelen = original / low, original / high
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (original / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * scaled / factor + smooth * scaled
    medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, scaled)


class RotaryEncoding(PositionEncoding):
    def __init__(self, *, head_dim: int, theta: float, scaling: Mapping[str, Any] | None = None,
                 rot_dim: int | None = None, interleaved: bool = False,
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.head_dim = int(head_dim)
        self.rot_dim = self.head_dim if rot_dim is None else int(rot_dim)
        if self.rot_dim % 2 or self.rot_dim > self.head_dim:
            raise ValueError("rot_dim must be even and at most head_dim")
        self.interleaved = bool(interleaved)
        self.inv_freq = rotary_frequencies(self.rot_dim, float(theta), scaling).to(device)

    def rotary_table(self):
        """(inv_freq, rot_dim, interleaved): what a kernel needs to apply this encoding itself."""
        return self.inv_freq, self.rot_dim, self.interleaved

    def encode_and_store(self, qkv, q_out, ctx: LayerContext, heads, kv_heads, head_dim):
        kv = ctx.kv
        write = kv is not None and kv.writes
        return ops.rope_append(
            qkv, q_out, kv.pool if write else None, ctx.batch.positions,
            ctx.batch.token_slot if write else None, kv.block_table if write else None,
            self.inv_freq, heads, kv_heads, head_dim, rot_dim=self.rot_dim,
            interleaved=self.interleaved, write_kv=write, error_word=ctx.error_word)


class NoPositionEncoding(PositionEncoding):
    """No encoding: q passes through, k and v are stored as they are."""

    def __init__(self, *, head_dim: int, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.inv_freq = torch.zeros(0, dtype=torch.float32, device=device)

    def rotary_table(self):
        return self.inv_freq, 0, False

    def encode_and_store(self, qkv, q_out, ctx: LayerContext, heads, kv_heads, head_dim):
        kv = ctx.kv
        write = kv is not None and kv.writes
        return ops.rope_append(
            qkv, q_out, kv.pool if write else None, ctx.batch.positions,
            ctx.batch.token_slot if write else None, kv.block_table if write else None,
            self.inv_freq, heads, kv_heads, head_dim, rot_dim=0, write_kv=write,
            error_word=ctx.error_word)


register_part("position", "rotary", RotaryEncoding)
register_part("position", "none", NoPositionEncoding)
