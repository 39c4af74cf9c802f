"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)).

gate and up run as one product (src/torchinferno/models/llama3/tensor_parallel.py:4398, 3170 concatenates
them, gate first); here their rows are interleaved instead (row 2i = gate i, row 2i + 1 = up i), so that one
tile of the product holds both and the few-rows kernel of a decode step can apply the activation in its
epilogue;
silu(g) = g / (1 + exp(-g)) with g in fp32
(src/torchinferno/kernels/triton_ops.py:29-32); no bias
(src/torchinferno/models/llama3/pipeline.py:247-250).
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear, linear_swiglu
from torchinferno_b200.parts.base import FeedForward, LayerContext, WeightSpec, register_part


class SwiGLUFeedForward(FeedForward):
    def __init__(self, *, hidden_size: int, intermediate_size: int, gate_name: str = "gate_proj.weight",
                 up_name: str = "up_proj.weight", down_name: str = "down_proj.weight",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.names = (gate_name, up_name, down_name)
        self.gate_up_weight: LinearWeight | None = None
        self.down_weight: LinearWeight | None = None

    def weight_specs(self) -> list[WeightSpec]:
        g, u, d = self.names
        return [WeightSpec(g, (self.intermediate_size, self.hidden_size)),
                WeightSpec(u, (self.intermediate_size, self.hidden_size)),
                WeightSpec(d, (self.hidden_size, self.intermediate_size))]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        g, u, d = self.names
        pairs = torch.stack([weights[g], weights[u]], dim=1).reshape(2 * self.intermediate_size, self.hidden_size)
        self.gate_up_weight = LinearWeight(pairs, few_rows_tcgen05=None, epilogue="swiglu")
        self.down_weight = LinearWeight(weights[d], few_rows_tcgen05=None)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        return linear(linear_swiglu(x, self.gate_up_weight), self.down_weight)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
