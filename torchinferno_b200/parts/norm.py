"""RMSNorm, plain and fused with the residual add.

y = x * rsqrt(mean(x^2) + eps) * w with the statistics, the product and the
residual sum in fp32 (src/torchinferno/models/llama3/raw_ops.py:9-11,
src/torchinferno/kernels/triton_ops.py:2044-2048, 2088-2096).  The weight
multiplies after normalisation; there is no bias and no ``1 + w`` form.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import ops
from torchinferno_b200.parts.base import Norm, WeightSpec, register_part


class RMSNorm(Norm):
    def __init__(self, *, width: int, eps: float, weight_name: str = "weight",
                 dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.width, self.eps, self.weight_name = int(width), float(eps), weight_name
        self.weight: torch.Tensor | None = None

    def weight_specs(self) -> list[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), init="ones", role="vector")]

    def bind(self, weights: Mapping[str, torch.Tensor]) -> None:
        self.weight = weights[self.weight_name].to(torch.float32).contiguous()

    def forward(self, residual, out, rows=None):
        return ops.add_rmsnorm(None, residual, self.weight, self.eps, out, rows)

    def add_forward(self, delta, residual, out, rows=None):
        return ops.add_rmsnorm(delta, residual, self.weight, self.eps, out, rows)

    def forward_rows(self, x: torch.Tensor) -> torch.Tensor:
        """Norm rows held in the activation type (not the residual stream)."""
        return ops.rmsnorm(x, self.weight, self.eps, torch.empty_like(x))


register_part("norm", "rmsnorm", RMSNorm)
