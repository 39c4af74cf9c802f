"""Matrix products of the projections: out = x . w^T with w stored [out, in].

32-bit operands go to the engine's own CUDA-core kernel (true fp32, fixed k
order).  bfloat16 operands go to the hand-written tensor-core kernels where one
takes the shape and otherwise to cuBLAS, which is where the reference sends
every projection (``F.linear``: src/torchinferno/models/llama3/pipeline.py:206-208,
src/torchinferno/models/llama3/tensor_parallel.py:11176-11198).
"""
from __future__ import annotations

import torch

from torchinferno_b200.kernels import ops


def linear(x: torch.Tensor, weight: torch.Tensor, *, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """``x``: [tokens, in]; ``weight``: [out, in]; returns [tokens, out] in ``out_dtype``."""
    if x.dim() != 2 or weight.dim() != 2 or x.shape[1] != weight.shape[1]:
        raise ops.KernelError(f"linear: shapes {tuple(x.shape)} and {tuple(weight.shape)} do not fit")
    if not x.is_cuda or not weight.is_cuda:
        raise ops.KernelError("linear: operands must be CUDA tensors (there is no CPU path)")
    out_dtype = out_dtype or x.dtype
    m, n = x.shape[0], weight.shape[0]
    if x.dtype == torch.float32 or weight.dtype == torch.float32:
        target = out if (out is not None and out.dtype == torch.float32) else \
            torch.empty((m, n), dtype=torch.float32, device=x.device)
        ops.gemm_f32(x, weight, target)
        if out_dtype == torch.float32:
            return target
        result = out if out is not None else torch.empty((m, n), dtype=out_dtype, device=x.device)
        return ops.cast(target, result)
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise ops.KernelError(f"linear: unsupported dtypes {x.dtype} / {weight.dtype}")
    return _linear_bf16(x, weight, out_dtype, out)


def _linear_bf16(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                 out: torch.Tensor | None) -> torch.Tensor:
    m, n = x.shape[0], weight.shape[0]
    if out_dtype == torch.bfloat16:
        if out is None:
            out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
        torch.mm(x, weight.t(), out=out)
        return out
    if out_dtype == torch.float32:
        result = torch.mm(x, weight.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(result)
            return out
        return result
    raise ops.KernelError(f"linear: unsupported output dtype {out_dtype}")
