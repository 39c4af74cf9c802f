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

    ``few_rows_tcgen05``: True gives products of up to FEW_ROWS rows to the hand-written few-rows kernel under
    "auto", False never does, None leaves it to :func:`tune_few_rows` (the library until that has run).

    ``epilogue="swiglu"``: the rows of ``weight`` are (gate i, up i) pairs, and what is wanted of the product is
    silu(gate) * up (:func:`linear_swiglu`); the few-rows kernel then writes that directly.

    ``features`` / ``splits``: the few-rows kernel's tile width (128 or 256 features) and the number of blocks
    that share K (0: the older swap-AB kernel with its own choice), set with the choice of the kernel.
    """

    FEW_ROWS = 64      # up to this many rows a weight may go to the few-rows kernel under "auto" (the most it takes)

    def __init__(self, weight: torch.Tensor, *, allow_transpose: bool = True, few_rows_tcgen05: bool | None = False,
                 epilogue: str = "none") -> None:
        if epilogue not in ("none", "swiglu"):
            raise ValueError(f"unknown epilogue {epilogue!r}")
        self.out_features, self.in_features = weight.shape
        on_gpu = weight.dtype == torch.bfloat16 and weight.is_cuda
        self.few_rows = LinearWeight.FEW_ROWS if few_rows_tcgen05 and on_gpu else 0
        self.transposed = bool(allow_transpose and on_gpu and _backend != "tcgen05")
        self.tensor = weight.t().contiguous() if self.transposed else weight.contiguous()
        self.epilogue = epilogue
        self.features, self.splits, self.stages = 128, 0, 0
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
        view.few_rows, view.epilogue, view.features, view.splits, view.stages = self.few_rows, "none", 128, 0, 0
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
            return _linear_kn(x, weight.tensor, out_dtype or x.dtype, out, weight.few_rows, weight.features, weight.splits, weight.stages)
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


def linear_swiglu(x: torch.Tensor, weight: LinearWeight) -> torch.Tensor:
    """silu(gate) * up of the product with a weight whose rows are (gate i, up i) pairs: [tokens, out / 2].
    At few rows the few-rows kernel applies it in its epilogue; else the product is followed by the SwiGLU kernel."""
    if weight.epilogue != "swiglu":
        raise ops.KernelError("linear_swiglu: the weight was not bound with epilogue='swiglu'")
    m, inter = x.shape[0], weight.out_features // 2
    w = weight.tensor
    if (weight.transposed and _backend == "auto" and x.dtype == torch.bfloat16
            and ops.plan_product(m, weight.out_features, weight.in_features, True, weight.few_rows, weight.features, weight.splits,
                                 True, _aligned(x, w)) == ops.PRODUCT_DECODE):
        act = torch.empty((m, inter), dtype=x.dtype, device=x.device)
        return ops.gemm_decode(x, w, act, features=weight.features, splits=1, epilogue=ops.DG_SWIGLU, stages=weight.stages,
                               error_word=_error_word)
    gate_up = linear(x, weight)
    act = torch.empty((m, inter), dtype=gate_up.dtype, device=x.device)
    return ops.swiglu(gate_up, act, interleaved=True)


def _aligned(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """What the TMA copies of the few-rows kernels ask of their operands."""
    return (x.stride(1) == 1 and weight.stride(1) == 1 and x.stride(0) % 8 == 0 and weight.stride(0) % 8 == 0
            and weight.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0)


def _linear_kn(x: torch.Tensor, weight_kn: torch.Tensor, out_dtype: torch.dtype, out: torch.Tensor | None,
               few_rows: int = 0, features: int = 128, splits: int = 0, stages: int = 0) -> torch.Tensor:
    """A matrix stored [in, out]: a few-rows kernel up to ``few_rows`` rows, else cuBLAS."""
    if x.dim() != 2 or x.shape[1] != weight_kn.shape[0]:
        raise ops.KernelError(f"linear: shapes {tuple(x.shape)} and [in, out] = {tuple(weight_kn.shape)} do not fit")
    if _backend == "tcgen05":
        raise ops.KernelError("linear: these weights were laid out for the library; bind the model after "
                              "choosing the tcgen05 backend")
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise ops.KernelError(f"linear: unsupported output dtype {out_dtype}")
    if out is None or out.dtype != out_dtype:
        out = torch.empty((x.shape[0], weight_kn.shape[1]), dtype=out_dtype, device=x.device)
    if _backend == "auto":      # (which kernel: decided where the native block call decides it too)
        k, n = weight_kn.shape
        kernel = ops.plan_product(x.shape[0], n, k, True, few_rows, features, splits, False, _aligned(x, weight_kn))
        if kernel == ops.PRODUCT_DECODE:
            return ops.gemm_decode(x, weight_kn, out, features=features, splits=splits, stages=stages, error_word=_error_word)
        if kernel == ops.PRODUCT_SWAPAB:
            return ops.gemm_tcgen05_swapab(x, weight_kn, out, _error_word, w_kn=True)
    return ops.library_gemm(x, weight_kn, out, w_kn=True)


# ---------------------------------------------------------------------------
# Which kernel takes a weight's few-row products, by measurement.
_undecided: "weakref.WeakSet[LinearWeight]" = weakref.WeakSet()
# (out, in, device, epilogue) -> (rows up to which the few-rows kernel takes the shape, its tile width, its K split)
_tuned: dict[tuple, tuple[int, int, int]] = {}
tuning_times: dict[tuple, dict[str, float]] = {}   # (out, in, device, epilogue, rows) -> microseconds per product with either kernel
# cuBLAS changes kernels with the row count (at the 8B sizes its output projection takes 14.5 us at 8 rows and
# 10.8 at 16, the few-rows kernel 12.0 and 12.4), so several row counts are measured, each standing for the
# counts up to it: a shape may go to the few-rows kernel up to 4 rows, up to 8, 16, 32 or 64, or not at all.
TUNE_ROWS = ((1, 4), (8, 8), (16, 16), (32, 32), (64, 64))      # (rows measured, rows it stands for)
# The few-rows kernel gets a shape unless it takes more than this share of the library's time in the walk.  The
# walk understates what the kernel is worth inside a layer: there its neighbours are kernels of this library too, each
# placed while the one before drains, and a library kernel in the chain breaks it.  Measured in a captured decode
# step of the 8B sizes (8 requests at 2,100 to 2,300 tokens, ms a step): every product on the library 3.78; the
# attention output projection here (0.81 of the library's time in the walk) 3.64; the down projection too (0.98 in
# the walk) 3.58; gate/up with the activation in its epilogue too (1.01) 3.54; the qkv projection too (1.17) 3.62.
# So parity in the walk is a gain in the layer, and the line is drawn a little above it; what is decided is kept
# (see _stored_choices): the kernels a checkpoint runs on a GPU model do not change from one process to the next.
TUNE_MARGIN = 1.04
TUNE_MEMBERS = 32
_flush: dict[torch.device, torch.Tensor] = {}     # larger than the L2; made once per tuning pass


def _choice_file():
    """The file of decisions beside the built library (which a changed kernel source replaces: its stamp is part of
    every key), or None when that folder cannot be written."""
    from pathlib import Path
    from torchinferno_b200.kernels.library import library_path
    path = library_path()
    return None if path is None else Path(path).parent / "gemm_choice.json"


def _choice_key(n: int, k: int, device: torch.device, members: int, epilogue: str) -> str:
    """What a stored decision holds for: the GPU model, the build of the kernels, the line, the shape, and whether
    the measured weights together exceed the L2 (a model of two layers is timed out of the L2, one of thirty-two
    out of memory, and the two may well decide differently)."""
    from pathlib import Path
    from torchinferno_b200.kernels.library import library_path
    stamp = Path(library_path()).parent / "stamp.txt"
    mark = stamp.read_text().strip()[:16] if stamp.is_file() else "?"
    measured = min(members, TUNE_MEMBERS)
    where = "from memory" if measured * n * k * 2 > (256 << 20) else f"{measured} weights"
    return f"{torch.cuda.get_device_name(device)}|{mark}|margin {TUNE_MARGIN}|{n}x{k}|{epilogue}|{where}"


def _stored_choices() -> dict[str, list[int]]:
    import json
    path = _choice_file()
    try:
        return {str(k): [int(x) for x in v] for k, v in json.loads(path.read_text()).items()} if path and path.is_file() else {}
    except (OSError, ValueError, TypeError):
        return {}


def _store_choice(key: str, choice: tuple[int, int, int]) -> None:
    import json
    import os
    path = _choice_file()
    if path is None:
        return
    choices = _stored_choices()
    choices[key] = list(choice)
    try:
        tmp = path.with_suffix(f".tmp{os.getpid()}")
        tmp.write_text(json.dumps(choices, indent=0, sort_keys=True))
        os.replace(tmp, path)
    except OSError:
        pass          # (a read-only folder: the choice is measured again by the next process)


def decisions() -> dict[tuple, tuple[int, int, int]]:
    """(out, in, device, epilogue) -> (rows up to which the few-rows kernel takes that shape's products, tile width,
    K split), as decided so far."""
    return dict(_tuned)


def _candidates(n: int, k: int, epilogue: str) -> list[tuple[int, int]]:
    """(tile width, K split) worth timing for a [k, n] weight: 256 features a tile only where that still gives about
    a hundred blocks, splits that leave every block a few k slices and the grid neither tiny nor many rounds deep."""
    out = []
    if n >= 256 * 96 and ops.gemm_decode_supports(8, n, k, 256, 1, ops.DG_SWIGLU if epilogue == "swiglu" else ops.DG_PLAIN):
        out.append((256, 1))
    tiles = -(-n // 128)
    for splits in range(1, 9):
        if epilogue == "swiglu" and splits > 1:
            break
        if not ops.gemm_decode_supports(8, n, k, 128, splits, ops.DG_PLAIN) or k // 64 < 4 * splits:
            continue
        if splits > 1 and (tiles * splits < 64 or tiles * splits > 4 * 148):
            continue
        out.append((128, splits))
    return out


def tune_few_rows() -> dict[tuple, tuple[int, int, int]]:
    """Decide, for every weight bound with ``few_rows_tcgen05=None`` since the last call, whether and up to how many
    rows the hand-written few-rows kernel takes its products (0, 4, 8, 16, 32 or 64) and with which tiles, and return
    the decisions made so far by (out, in, device, epilogue).

    Under the "measured" choice, weights of one shape are measured together, once per shape and GPU model, the way
    a decode step runs them: a CUDA graph walks over them (different weights one after the other, so nothing
    comes from L2), each product behind a small kernel, as in a layer (under programmatic dependent launch the
    few-rows kernel fetches its first weights while that kernel runs, and a measurement of the product alone
    would not show it).  First the kernel's own configurations are timed at 8 rows and the fastest is kept; then
    the graph is timed with either kernel at rising row counts, and the few-rows kernel gets the shape up to
    the last count at which it takes less than TUNE_MARGIN of the library's time.  The outcome is stored and later
    processes read it."""
    groups: dict[tuple, list[LinearWeight]] = {}
    for w in list(_undecided):
        groups.setdefault((w.out_features, w.in_features, w.tensor.device, w.epilogue), []).append(w)
    _undecided.clear()
    if groups:
        ops.lib()                 # (loads, and at the first call builds, the library the decisions are kept beside)
    try:
        for key, group in groups.items():
            if key not in _tuned:
                n, k, device, epilogue = key
                configs = _candidates(n, k, epilogue) if group[0].transposed else []
                if _few_rows_choice != "measured" or not configs:
                    takes = _few_rows_choice == "swapab" and bool(configs)
                    _tuned[key] = (LinearWeight.FEW_ROWS, *configs[0]) if takes else (0, 128, 0)
                else:
                    name, stored = _choice_key(n, k, device, len(group), epilogue), _stored_choices()
                    if name in stored and len(stored[name]) == 3:
                        _tuned[key] = tuple(stored[name])
                    else:
                        members = group[:TUNE_MEMBERS]
                        timed = {c: _walk_time(members, 8, c, epilogue) for c in configs}
                        best = min(timed, key=timed.get)
                        rows_taken = 0
                        for rows, stands_for in TUNE_ROWS:      # (rising: the first row count at which the library wins ends it)
                            times = {"few_rows": _walk_time(members, rows, best, epilogue), "library": _walk_time(members, rows, None, epilogue)}
                            tuning_times[(n, k, device, epilogue, rows)] = times
                            if not times["few_rows"] <= TUNE_MARGIN * times["library"]:
                                break
                            rows_taken = stands_for
                        _tuned[key] = (min(rows_taken, LinearWeight.FEW_ROWS), *best)
                        _store_choice(name, _tuned[key])
            for w in group:
                w.few_rows, w.features, w.splits = _tuned[key]
    finally:
        _flush.clear()
    if groups:
        _changed()
    return dict(_tuned)


def _walk_time(group: "list[LinearWeight]", rows: int, config: tuple[int, int] | None, epilogue: str) -> float:
    """Microseconds per (small kernel + product) of a captured walk over ``group``'s weights with the few-rows
    kernel in ``config`` (tile width, K split), or with the library (None); with the SwiGLU epilogue the library's
    product is followed by the SwiGLU kernel, as it is in a layer."""
    first = group[0]
    n, k, device = first.out_features, first.in_features, first.tensor.device
    ops.library_gemm_ready(device)
    with torch.cuda.device(device):
        x = torch.zeros((rows, k), dtype=torch.bfloat16, device=device)
        # the small kernel before each product: a norm of as many rows of a usual width (a few microseconds)
        width = min(k, 4096)
        delta = torch.zeros((rows, width), dtype=torch.bfloat16, device=device)
        residual, normed = torch.randn((rows, width), dtype=torch.float32, device=device), torch.empty_like(delta)
        norm_weight = torch.ones(width, dtype=torch.float32, device=device)
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=device)
        act = torch.empty((rows, n // 2), dtype=torch.bfloat16, device=device)
        flush = _flush.get(device)
        if flush is None:
            flush = _flush[device] = torch.empty(256 << 20, dtype=torch.uint8, device=device)      # larger than the L2

        def product(w: LinearWeight) -> None:
            if config is None:
                ops.library_gemm(x, w.tensor, out, w_kn=True)
                if epilogue == "swiglu":
                    ops.swiglu(out, act, interleaved=True)
            elif epilogue == "swiglu":
                ops.gemm_decode(x, w.tensor, act, features=config[0], splits=config[1], epilogue=ops.DG_SWIGLU)
            else:
                ops.gemm_decode(x, w.tensor, out, features=config[0], splits=config[1])

        def walk() -> None:
            for w in group:
                ops.add_rmsnorm(delta, residual, norm_weight, 1e-5, normed)
                product(w)
        walk()                                                            # (first launches: attributes, handles)
        torch.cuda.synchronize(device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            walk()
        # the fastest replay counts: what slows a replay down (clocks on their way up, another process's traffic)
        # only ever adds time
        best = float("inf")
        for i in range(7):
            flush.zero_()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            graph.replay()
            end.record()
            end.synchronize()
            if i >= 2:
                best = min(best, begin.elapsed_time(end))
        del graph
    return best * 1e3 / len(group)


def _linear_bf16(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype,
                 out: torch.Tensor | None, few_rows: int = 0) -> torch.Tensor:
    m, n = x.shape[0], weight.shape[0]
    k = x.shape[1]
    if _backend != "library" and out_dtype in (torch.bfloat16, torch.float32):
        rows = few_rows if _backend == "auto" else 64
        aligned = _aligned(x, weight)
        if ops.plan_product(m, n, k, False, rows, 128, 0, False, aligned) == ops.PRODUCT_SWAPAB:
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
