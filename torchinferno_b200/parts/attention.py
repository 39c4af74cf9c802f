"""Grouped-query attention over the paged cache.

q = x Wq^T, k = x Wk^T, v = x Wv^T run as one product on cat(Wq, Wk, Wv) split at
(h d, k d, k d) (src/torchinferno/models/llama3/tensor_parallel.py:4385-4388,
3832-3855); position encoding of q and k; k, v go to the cache; query head j
reads kv head j // (h / k) (src/torchinferno/models/llama3/raw_ops.py:38-41);
scores scaled by ``scale`` (1 / sqrt(head_dim) for Llama, raw_ops.py:45), causal
mask, fp32 softmax, p . v; then the output projection
(src/torchinferno/models/llama3/pipeline.py:206-245).  No bias anywhere.

A layer call whose cache binding does not write (``ctx.kv.writes`` False)
projects only q and reads keys and values another layer call stored.
"""
from __future__ import annotations

import math
from typing import Mapping

import torch

from torchinferno_b200.kernels import attention as attention_kernels
from torchinferno_b200.kernels.gemm import LinearWeight, linear
from torchinferno_b200.parts.base import (CacheSpec, LayerContext, Mixer, PartSpec, WeightSpec,
                                          build_part, register_part)


class GQAAttention(Mixer):
    def __init__(self, *, hidden_size: int, heads: int, kv_heads: int, head_dim: int,
                 position: PartSpec | Mapping, scale: float | None = None, window: int | None = None,
                 q_name: str = "q_proj.weight", k_name: str = "k_proj.weight",
                 v_name: str = "v_proj.weight", o_name: str = "o_proj.weight",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        self.hidden_size, self.heads, self.kv_heads, self.head_dim = hidden_size, heads, kv_heads, head_dim
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
        self.window = window
        self.names = (q_name, k_name, v_name, o_name)
        if not isinstance(position, PartSpec):
            position = PartSpec(**position)
        self.position = build_part("position", position, dtype=dtype, device=device)
        self.qkv_weight: LinearWeight | None = None
        self.o_weight: LinearWeight | None = None

    def weight_specs(self) -> list[WeightSpec]:
        q, k, v, o = self.names
        qw, kw = self.heads * self.head_dim, self.kv_heads * self.head_dim
        return [WeightSpec(q, (qw, self.hidden_size)), WeightSpec(k, (kw, self.hidden_size)),
                WeightSpec(v, (kw, self.hidden_size)), WeightSpec(o, (self.hidden_size, qw))]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        q, k, v, o = self.names
        self.qkv_weight = LinearWeight(torch.cat([weights[q], weights[k], weights[v]], dim=0), few_rows_tcgen05=None)
        # (which kernel takes the products of few rows is measured per shape once the whole model is bound)
        self.o_weight = LinearWeight(weights[o], few_rows_tcgen05=None)

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(self.kv_heads, self.head_dim, self.window)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        if ctx.kv is None:
            raise RuntimeError("attention needs a cache binding")
        h, k, d = self.heads, self.kv_heads, self.head_dim
        n = x.shape[0]
        window = self.window if self.window is not None else ctx.kv.window
        if ctx.kv.writes and attention_kernels.decode_takes_unrotated(x, ctx, h, k, d, self.position):
            # a step of single tokens: the decode kernel rotates and stores the newest token itself
            qkv = linear(x, self.qkv_weight)
            out = torch.empty((n, h * d), dtype=x.dtype, device=x.device)
            attention_kernels.decode_attention_unrotated(qkv, out, ctx, h, k, d, self.scale, window, self.position)
            return linear(out, self.o_weight)
        q = torch.empty((n, h * d), dtype=x.dtype, device=x.device)
        if ctx.kv.writes:
            qkv = linear(x, self.qkv_weight)
            self.position.encode_and_store(qkv, q, ctx, h, k, d)
        else:
            q_only = linear(x, self.qkv_weight.rows(0, h * d))
            self.position.encode_and_store(q_only, q, ctx, h, 0, d)
        out = torch.empty_like(q)
        attention_kernels.paged_attention(q, out, ctx, h, k, d, self.scale, window)
        return linear(out, self.o_weight)


register_part("mixer", "gqa_attention", GQAAttention)
