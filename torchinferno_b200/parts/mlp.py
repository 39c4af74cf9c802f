"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)).

gate and up run as one product on cat(Wg, Wu) split at (I, I), gate first
(src/torchinferno/models/llama3/tensor_parallel.py:4398, 3170);
silu(g) = g / (1 + exp(-g)) with g in fp32
(src/torchinferno/kernels/triton_ops.py:29-32); no bias
(src/torchinferno/models/llama3/pipeline.py:247-250).
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.kernels.gemm import LinearWeight, linear
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
        self.gate_up_weight = LinearWeight(torch.cat([weights[g], weights[u]], dim=0), few_rows_tcgen05=None)
        self.down_weight = LinearWeight(weights[d], few_rows_tcgen05=None)

    def forward(self, x: torch.Tensor, ctx: LayerContext) -> torch.Tensor:
        gate_up = linear(x, self.gate_up_weight)
        act = torch.empty((x.shape[0], self.intermediate_size), dtype=gate_up.dtype, device=x.device)
        ops.swiglu(gate_up, act)
        return linear(act, self.down_weight)


register_part("feed_forward", "swiglu", SwiGLUFeedForward)
