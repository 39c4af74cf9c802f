"""Matrix products of the projections: out = x . w^T with w stored [out, in].

32-bit operands go to the engine's own CUDA-core kernel (true fp32, fixed k
order).  bfloat16 operands go to the hand-written tensor-core kernels where they
were measured faster (or everywhere, on request) and otherwise to cuBLAS, called
from the engine's library (csrc/library_gemm.cu), which is where the reference
sends every projection (``F.linear``: src/torchinferno/models/llama3/pipeline.py:206-208,
src/torchinferno/models/llama3/tensor_parallel.py:11176-11198).
"""
from __future__ import annotations

import weakref

import torch

from torchinferno_b200.kernels import ops

# Which kernel multiplies bf16 operands:
#   "auto"     whichever is faster on this GPU.  Many rows go to cuBLAS.  At few rows (decode steps) neither the
#              hand-written swap-AB kernel nor cuBLAS wins everywhere: inside a captured decode step of the 8B
#              sizes at 8 rows (us, swap-AB / cuBLAS, time after the kernel before has ended) qkv 12.5 / 9.9,
#              o 9.2 / 12.1, gate_up 40.7 / 36.3, down 23.3 / 21.9, while at the 1B and 3B sizes cuBLAS takes
#              13 and 18 us for down projections that stream in 5 and 8.  So a weight is given to the swap-AB
#              kernel for few rows if it says so (few_rows_tcgen05=True) or, left open (None), if that
#              measured faster for its shape when the model was bound (tune_few_rows)
#   "tcgen05"  the hand-written kernels wherever they take the shape (swap-AB up to 64 rows, the
#              128 x 256-tile kernel above, and from 256 rows the two-SM kernel on 256 x 256 tiles)
#   "library"  cuBLAS everywhere
_backend = "auto"
_error_word: torch.Tensor | None = None
TWO_CTA_ROWS = 256
TWO_CTA_MAX_N = 65536
# Under "auto", how a weight left open (few_rows_tcgen05=None) gets its few-rows kernel:
#   "measured"  by timing, once per (GPU model, shape): the outcome is written beside the built library and read
#               back by later processes, so the same checkpoint runs the same kernels from one process to the next
#   "swapab"    always the hand-written kernel (up to FEW_ROWS rows), "library" never: nothing is timed
_few_rows_choice = "measured"
_generation = 0       # rises whenever a weight is bound or a choice changes: holders of raw pointers compare it


def generation() -> int:
    return _generation


def _changed() -> None:
    global _generation
    _generation += 1


def set_backend(name: str) -> None:
    global _backend
    if name not in ("auto", "tcgen05", "library"):
        raise ValueError(f"unknown GEMM backend {name!r}: auto, tcgen05 or library")
    if name != _backend:
        _changed()
    _backend = name


def set_few_rows_choice(mode: str) -> None:
    global _few_rows_choice
    if mode not in ("measured", "swapab", "library"):
        raise ValueError(f"unknown few-rows choice {mode!r}: measured, swapab or library")
    _few_rows_choice = mode


def get_few_rows_choice() -> str:
    return _few_rows_choice


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
    (src/torchinferno/models/llama3/tensor_parallel.py:11201-11239).  Only one layout is kept: [in, out] under
    "auto" (the swap-AB kernel reads both), [out, in] for the other hand-written kernels.

    ``few_rows_tcgen05``: True gives products of up to FEW_ROWS rows to the swap-AB kernel under "auto", False
    never does, None leaves it to :func:`tune_few_rows` (the library until that has run).
    """

    FEW_ROWS = 64      # up to this many rows a weight may go to the swap-AB kernel under "auto" (the most it takes)

    def __init__(self, weight: torch.Tensor, *, allow_transpose: bool = True, few_rows_tcgen05: bool | None = False) -> None:
        self.out_features, self.in_features = weight.shape
        on_gpu = weight.dtype == torch.bfloat16 and weight.is_cuda
        self.few_rows = LinearWeight.FEW_ROWS if few_rows_tcgen05 and on_gpu else 0
        self.transposed = bool(allow_transpose and on_gpu and _backend != "tcgen05")
        self.tensor = weight.t().contiguous() if self.transposed else weight.contiguous()
        if few_rows_tcgen05 is None and on_gpu and _backend == "auto":
            _undecided.add(self)
        _changed()

    @property
    def dtype(self) -> torch.dtype:
        return self.tensor.dtype

    def rows(self, start: int, stop: int) -> "LinearWeight":
        """The projection onto output features start .. stop-1 (a view, nothing is copied)."""
        view = object.__new__(LinearWeight)
        view.out_features, view.in_features, view.transposed = stop - start, self.in_features, self.transposed
        view.few_rows = self.few_rows
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
            return _linear_kn(x, weight.tensor, out_dtype or x.dtype, out, weight.few_rows)
        few_rows = weight.few_rows
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


def _swapab_takes_kn(x: torch.Tensor, weight_kn: torch.Tensor) -> bool:
    k, n = weight_kn.shape
    return (x.stride(1) == 1 and weight_kn.stride(1) == 1 and x.stride(0) % 8 == 0 and weight_kn.stride(0) % 8 == 0
            and weight_kn.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0 and ops.gemm_tcgen05_swapab_supports(x.shape[0], n, k))


def _linear_kn(x: torch.Tensor, weight_kn: torch.Tensor, out_dtype: torch.dtype, out: torch.Tensor | None,
               few_rows: int = 0) -> torch.Tensor:
    """A matrix stored [in, out]: the swap-AB kernel up to ``few_rows`` rows, else cuBLAS."""
    if x.dim() != 2 or x.shape[1] != weight_kn.shape[0]:
        raise ops.KernelError(f"linear: shapes {tuple(x.shape)} and [in, out] = {tuple(weight_kn.shape)} do not fit")
    if _backend == "tcgen05":
        raise ops.KernelError("linear: these weights were laid out for the library; bind the model after "
                              "choosing the tcgen05 backend")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ops.KernelError(f"linear: unsupported output dtype {out_dtype}")
    if out is None or out.dtype != out_dtype:
        out = torch.empty((x.shape[0], weight_kn.shape[1]), dtype=out_dtype, device=x.device)
    if _backend == "auto" and 0 < x.shape[0] <= few_rows and _swapab_takes_kn(x, weight_kn):
        return ops.gemm_tcgen05_swapab(x, weight_kn, out, _error_word, w_kn=True)
    return ops.library_gemm(x, weight_kn, out, w_kn=True)


# ---------------------------------------------------------------------------
# Which kernel takes a weight's few-row products, by measurement.
_undecided: "weakref.WeakSet[LinearWeight]" = weakref.WeakSet()
_tuned: dict[tuple, int] = {}           # (out, in, device) -> rows up to which the swap-AB kernel measured faster
tuning_times: dict[tuple, dict[str, float]] = {}   # (out, in, device, rows) -> milliseconds of the timed walk with either kernel
# cuBLAS changes kernels with the row count (at the 8B sizes its output projection takes 16.2 us at 8 rows and
# 10.8 at 16, the swap-AB kernel 12.4 and 12.9; its down projection is 9 % behind the swap-AB kernel at 1 row
# and 4 % at 8), so several row counts are measured, each standing for the counts up to it: a shape may go to
# the swap-AB kernel up to 4 rows, up to 8, 16, 32 or 64, or not at all.
TUNE_ROWS = ((1, 4), (8, 8), (16, 16), (32, 32), (64, 64))      # (rows measured, rows it stands for)
# The swap-AB kernel must take under this share of the library's time.  The measurement repeats within about half
# a per cent; the line leaves a dead band of several per cent below parity, so a shape near parity stays with the
# library whatever the noise of one run, and what is decided is kept (see _stored_choices): the kernels a
# checkpoint runs on a GPU model do not change from one process to the next.
TUNE_MARGIN = 0.93
TUNE_MEMBERS = 32
_flush: dict[torch.device, torch.Tensor] = {}     # larger than the L2; made once per tuning pass


def _choice_file():
    """The file of decisions beside the built library (which a changed kernel source replaces: its stamp is part of
    every key), or None when that folder cannot be written."""
    from pathlib import Path
    from torchinferno_b200.kernels.library import library_path
    path = library_path()
    return None if path is None else Path(path).parent / "gemm_choice.json"


def _choice_key(n: int, k: int, device: torch.device, members: int) -> str:
    """What a stored decision holds for: the GPU model, the build of the kernels, the line, the shape, and whether
    the measured weights together exceed the L2 (a model of two layers is timed out of the L2, one of thirty-two
    out of memory, and the two may well decide differently)."""
    from pathlib import Path
    from torchinferno_b200.kernels.library import library_path
    stamp = Path(library_path()).parent / "stamp.txt"
    mark = stamp.read_text().strip()[:16] if stamp.is_file() else "?"
    measured = min(members, TUNE_MEMBERS)
    where = "from memory" if measured * n * k * 2 > (256 << 20) else f"{measured} weights"
    return f"{torch.cuda.get_device_name(device)}|{mark}|margin {TUNE_MARGIN}|{n}x{k}|{where}"


def _stored_choices() -> dict[str, int]:
    import json
    path = _choice_file()
    try:
        return {str(k): int(v) for k, v in json.loads(path.read_text()).items()} if path and path.is_file() else {}
    except (OSError, ValueError):
        return {}


def _store_choice(key: str, rows: int) -> None:
    import json
    import os
    path = _choice_file()
    if path is None:
        return
    choices = _stored_choices()
    choices[key] = rows
    try:
        tmp = path.with_suffix(f".tmp{os.getpid()}")
        tmp.write_text(json.dumps(choices, indent=0, sort_keys=True))
        os.replace(tmp, path)
    except OSError:
        pass          # (a read-only folder: the choice is measured again by the next process)


def decisions() -> dict[tuple, int]:
    """(out, in, device) -> rows up to which the swap-AB kernel takes that shape's products, as decided so far."""
    return dict(_tuned)


def tune_few_rows() -> dict[tuple, int]:
    """Decide, for every weight bound with ``few_rows_tcgen05=None`` since the last call, up to how many rows the
    swap-AB kernel takes its products (0, 4, 8, 16, 32 or 64), and return the decisions made so far by (out, in, device).

    Under the "measured" choice, weights of one shape are measured together, once per shape and GPU model, the way
    a decode step runs them: a CUDA graph walks over them (different weights one after the other, so nothing
    comes from L2), each product behind a small kernel, as in a layer (under programmatic dependent launch the
    swap-AB kernel fetches its first weights while that kernel runs, and a measurement of the product alone
    would not show it).  The graph is timed with either kernel; the swap-AB kernel gets the shape if it takes
    less than TUNE_MARGIN of the library's time.  The outcome is stored and later processes read it."""
    groups: dict[tuple, list[LinearWeight]] = {}
    for w in list(_undecided):
        groups.setdefault((w.out_features, w.in_features, w.tensor.device), []).append(w)
    _undecided.clear()
    if groups:
        ops.lib()                 # (loads, and at the first call builds, the library the decisions are kept beside)
    try:
        for key, group in groups.items():
            if key not in _tuned:
                n, k, device = key
                if _few_rows_choice != "measured":
                    takes = _few_rows_choice == "swapab" and group[0].transposed and ops.gemm_tcgen05_swapab_supports(1, n, k)
                    _tuned[key] = LinearWeight.FEW_ROWS if takes else 0
                else:
                    name, stored = _choice_key(n, k, device, len(group)), _stored_choices()
                    if name in stored:
                        _tuned[key] = stored[name]
                    else:
                        rows_taken = 0
                        for rows, stands_for in TUNE_ROWS:      # (rising: the first row count at which the library wins ends it)
                            if not _swapab_is_faster(group[:TUNE_MEMBERS], rows):
                                break
                            rows_taken = stands_for
                        _tuned[key] = min(rows_taken, LinearWeight.FEW_ROWS)
                        _store_choice(name, _tuned[key])
            for w in group:
                w.few_rows = _tuned[key]
    finally:
        _flush.clear()
    if groups:
        _changed()
    return dict(_tuned)


def _swapab_is_faster(group: "list[LinearWeight]", rows: int) -> bool:
    first = group[0]
    n, k, device = first.out_features, first.in_features, first.tensor.device
    if not first.transposed or not ops.gemm_tcgen05_swapab_supports(rows, n, k):
        return False
    ops.library_gemm_ready(device)
    with torch.cuda.device(device):
        x = torch.zeros((rows, k), dtype=torch.bfloat16, device=device)
        if not all(_swapab_takes_kn(x, w.tensor) for w in group):
            return False
        # the small kernel before each product: a norm of as many rows of a usual width (a few microseconds)
        width = min(k, 4096)
        delta = torch.zeros((rows, width), dtype=torch.bfloat16, device=device)
        residual, normed = torch.randn((rows, width), dtype=torch.float32, device=device), torch.empty_like(delta)
        norm_weight = torch.ones(width, dtype=torch.float32, device=device)
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
        flush = _flush.get(device)
        if flush is None:
            flush = _flush[device] = torch.empty(256 << 20, dtype=torch.uint8, device=device)      # larger than the L2
        products = {"library": lambda w: ops.library_gemm(x, w.tensor, out, w_kn=True),
                    "swapab": lambda w: ops.gemm_tcgen05_swapab(x, w.tensor, out, None, w_kn=True)}
        graphs = {}
        for name, product in products.items():
            def walk() -> None:
                for w in group:
                    ops.add_rmsnorm(delta, residual, norm_weight, 1e-5, normed)
                    product(w)
            walk()                                                            # (first launches: attributes, handles)
            torch.cuda.synchronize(device)
            graphs[name] = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graphs[name]):
                walk()
        # the two graphs take turns, and the fastest replay of each counts: what slows a replay down (clocks on
        # their way up, another process's traffic) only ever adds time
        times = {name: float("inf") for name in graphs}
        for i in range(8):
            for name, graph in graphs.items():
                flush.zero_()
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                graph.replay()
                end.record()
                end.synchronize()
                if i >= 2:
                    times[name] = min(times[name], begin.elapsed_time(end))
        del graphs
    tuning_times[(n, k, device, rows)] = times
    return times["swapab"] < TUNE_MARGIN * times["library"]


def _linear_bf16(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                 out: torch.Tensor | None, few_rows: int = 0) -> torch.Tensor:
    m, n = x.shape[0], weight.shape[0]
    k = x.shape[1]
    if _backend != "library" and out_dtype in (torch.bfloat16, torch.float32):
        rows = few_rows if _backend == "auto" else 64
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
