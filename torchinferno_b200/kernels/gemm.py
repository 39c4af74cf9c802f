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

# Which kernel multiplies bf16 operands:
#   "auto"     whichever measured faster inside the engine's steps on the B200.  Today that is cuBLAS
#              for every shape of the model (the swap-AB kernel ties it in isolation at up to 16 rows
#              but costs about 10 us more per layer inside a captured decode step), so SWAPAB_AUTO_ROWS
#              is 0; the hand-written kernels are chosen with "tcgen05"
#   "tcgen05"  the hand-written kernels wherever they take the shape (swap-AB up to 64 rows, the
#              128 x 256-tile kernel above)
#   "library"  cuBLAS everywhere
_backend = "auto"
_error_word: torch.Tensor | None = None
SWAPAB_AUTO_ROWS = 0


def set_backend(name: str) -> None:
    global _backend
    if name not in ("auto", "tcgen05", "library"):
        raise ValueError(f"unknown GEMM backend {name!r}: auto, tcgen05 or library")
    _backend = name


def get_backend() -> str:
    return _backend


def set_error_word(word: torch.Tensor | None) -> None:
    """The device word in which the tcgen05 kernels report a bounded wait that ran out."""
    global _error_word
    _error_word = word


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
    k = x.shape[1]
    if _backend != "library" and out_dtype in (torch.bfloat16, torch.float32):
        rows = SWAPAB_AUTO_ROWS if _backend == "auto" else 64
        aligned = x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
        if aligned and m <= rows and ops.gemm_tcgen05_swapab_supports(m, n, k):
            if out is None or out.dtype != out_dtype:
                out = torch.empty((m, n), dtype=out_dtype, device=x.device)
            return ops.gemm_tcgen05_swapab(x, weight, out, _error_word)
        if aligned and _backend == "tcgen05" and ops.gemm_tcgen05_supports(m, n, k):
            if out is None or out.dtype != out_dtype:
                out = torch.empty((m, n), dtype=out_dtype, device=x.device)
            return ops.gemm_tcgen05(x, weight, out, _error_word)
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
