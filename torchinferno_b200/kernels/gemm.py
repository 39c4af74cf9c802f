"""Matrix products of the projections: out = x . w^T with w stored [out, in].

32-bit operands go to the engine's own CUDA-core kernel (true fp32, fixed k
order).  bfloat16 operands go to the hand-written tensor-core kernels where they
were measured faster (or everywhere, on request) and otherwise to cuBLAS, called
from the engine's library (csrc/library_gemm.cu), which is where the reference
sends every projection (``F.linear``: src/torchinferno/models/llama3/pipeline.py:206-208,
src/torchinferno/models/llama3/tensor_parallel.py:11176-11198).
"""
from __future__ import annotations

import torch

from torchinferno_b200.kernels import ops

# Which kernel multiplies bf16 operands:
#   "auto"     whichever measured faster inside the engine's steps on the B200.  Inside a captured decode
#              step of the 8B sizes at 8 rows (us, hand-written swap-AB / cuBLAS, time after the kernel
#              before has ended): qkv 12.5 / 9.9, o 9.2 / 12.1, gate_up 40.7 / 36.3, down 23.3 / 21.9.
#              So a weight may say that it wants the swap-AB kernel for few rows
#              (LinearWeight(few_rows_tcgen05=True): the attention output projection does); everything
#              else goes to cuBLAS (SWAPAB_AUTO_ROWS = 0).  All hand-written kernels: "tcgen05"
#   "tcgen05"  the hand-written kernels wherever they take the shape (swap-AB up to 64 rows, the
#              128 x 256-tile kernel above, and from 256 rows the two-SM kernel on 256 x 256 tiles)
#   "library"  cuBLAS everywhere
_backend = "auto"
_error_word: torch.Tensor | None = None
SWAPAB_AUTO_ROWS = 0
TWO_CTA_ROWS = 256
TWO_CTA_MAX_N = 65536


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


class LinearWeight:
    """A projection matrix as the chosen kernels want it laid out.

    Checkpoints store [out, in].  The hand-written kernels read that layout (K-major rows).  cuBLAS is
    measurably faster on few rows when the matrix is stored [in, out] (at 8 rows of the 8B sizes: qkv
    14.8 -> 12.5 us, gate/up 42.4 -> 37.8 us, down 26.8 -> 25.3 us; no difference at 2,048 rows), which is
    what the reference's optional pre-transposed copies for M <= 64 are for
    (src/torchinferno/models/llama3/tensor_parallel.py:11201-11239).  Only one layout is kept.
    """

    FEW_ROWS = 16      # up to this many rows a weight with few_rows_tcgen05 goes to the swap-AB kernel under "auto"

    def __init__(self, weight: torch.Tensor, *, allow_transpose: bool = True, few_rows_tcgen05: bool = False) -> None:
        self.out_features, self.in_features = weight.shape
        self.few_rows_tcgen05 = bool(few_rows_tcgen05 and weight.dtype == torch.bfloat16 and weight.is_cuda)
        self.transposed = bool(allow_transpose and not self.few_rows_tcgen05 and weight.dtype == torch.bfloat16
                               and weight.is_cuda and _backend != "tcgen05")
        self.tensor = weight.t().contiguous() if self.transposed else weight.contiguous()

    @property
    def dtype(self) -> torch.dtype:
        return self.tensor.dtype

    def rows(self, start: int, stop: int) -> "LinearWeight":
        """The projection onto output features start .. stop-1 (a view, nothing is copied)."""
        view = object.__new__(LinearWeight)
        view.out_features, view.in_features, view.transposed = stop - start, self.in_features, self.transposed
        view.few_rows_tcgen05 = self.few_rows_tcgen05
        view.tensor = self.tensor[:, start:stop] if self.transposed else self.tensor[start:stop]
        return view

    def nbytes(self) -> int:
        return self.tensor.numel() * self.tensor.element_size()


def linear(x: torch.Tensor, weight: "torch.Tensor | LinearWeight", *, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None) -> torch.Tensor:
    """``x``: [tokens, in]; ``weight``: [out, in] (or a :class:`LinearWeight`); returns [tokens, out] in ``out_dtype``."""
    few_rows = 0
    if isinstance(weight, LinearWeight):
        if weight.transposed:
            return _linear_library_kn(x, weight.tensor, out_dtype or x.dtype, out)
        few_rows = LinearWeight.FEW_ROWS if weight.few_rows_tcgen05 else 0
        weight = weight.tensor
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
    return _linear_bf16(x, weight, out_dtype, out, few_rows)


def _linear_library_kn(x: torch.Tensor, weight_kn: torch.Tensor, out_dtype: torch.dtype,
                       out: torch.Tensor | None) -> torch.Tensor:
    """cuBLAS on a matrix stored [in, out]."""
    if x.dim() != 2 or x.shape[1] != weight_kn.shape[0]:
        raise ops.KernelError(f"linear: shapes {tuple(x.shape)} and [in, out] = {tuple(weight_kn.shape)} do not fit")
    if _backend == "tcgen05":
        raise ops.KernelError("linear: these weights were laid out for the library; bind the model after "
                              "choosing the tcgen05 backend")
    if out is None or out.dtype != out_dtype:
        out = torch.empty((x.shape[0], weight_kn.shape[1]), dtype=out_dtype, device=x.device)
    return ops.library_gemm(x, weight_kn, out, w_kn=True)


def _linear_bf16(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                 out: torch.Tensor | None, few_rows: int = 0) -> torch.Tensor:
    m, n = x.shape[0], weight.shape[0]
    k = x.shape[1]
    if _backend != "library" and out_dtype in (torch.bfloat16, torch.float32):
        rows = max(SWAPAB_AUTO_ROWS, few_rows) if _backend == "auto" else 64
        aligned = x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0 and x.stride(1) == 1 and weight.stride(1) == 1
        if aligned and m <= rows and ops.gemm_tcgen05_swapab_supports(m, n, k):
            if out is None or out.dtype != out_dtype:
                out = torch.empty((m, n), dtype=out_dtype, device=x.device)
            return ops.gemm_tcgen05_swapab(x, weight, out, _error_word)
        if aligned and _backend == "tcgen05" and ops.gemm_tcgen05_supports(m, n, k):
            if out is None or out.dtype != out_dtype:
                out = torch.empty((m, n), dtype=out_dtype, device=x.device)
            # from 256 rows on, pairs of SMs on 256 x 256 tiles (7 to 14 % ahead of one block per 128 x 256 tile on
            # the layers' shapes at 2,048 rows; the one-block kernel keeps the widest shape, the head)
            if m >= TWO_CTA_ROWS and n <= TWO_CTA_MAX_N and ops.gemm_tcgen05_2cta_supports(m, n, k):
                return ops.gemm_tcgen05_2cta(x, weight, out, _error_word)
            return ops.gemm_tcgen05(x, weight, out, _error_word)
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ops.KernelError(f"linear: unsupported output dtype {out_dtype}")
    if out is None or out.dtype != out_dtype:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    return ops.library_gemm(x, weight, out, w_kn=False)
