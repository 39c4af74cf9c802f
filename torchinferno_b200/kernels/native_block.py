"""A pre-norm block of the built-in parts issued as one call into the CUDA library.

The parts stay what they are (each with its weights and its own forward); when a block is made only of
the built-in kinds (RMSNorm, grouped-query attention with rotary or no position encoding, SwiGLU) in
bfloat16, `PreNormBlock` hands the whole sequence of launches to ``tib_prenorm_gqa_glu_block``, which issues the
same kernels with the same choices without returning to the interpreter between them: an eager step of
32 layers costs the host about a third of what the part-by-part sequence does.  Any other composition,
the float32 path and the ``tcgen05`` GEMM backend keep the part-by-part sequence.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_int64, c_void_p

import torch

from torchinferno_b200.kernels import gemm, ops
from torchinferno_b200.kernels.gemm import LinearWeight


class BlockWeights(Structure):
    _fields_ = [(name, c_int) for name in ("hidden", "heads", "kv_heads", "head_dim", "intermediate", "rot_dim", "interleaved",
                                           "qkv_kn", "o_kn", "gate_up_kn", "down_kn",
                                           "qkv_few_rows", "o_few_rows", "gate_up_few_rows", "down_few_rows",
                                           "qkv_features", "o_features", "gate_up_features", "down_features",
                                           "qkv_splits", "o_splits", "gate_up_splits", "down_splits",
                                           "qkv_stages", "o_stages", "gate_up_stages", "down_stages")] + \
               [(name, c_float) for name in ("eps_mixer", "eps_feed_forward", "scale")] + \
               [(name, c_void_p) for name in ("norm_mixer", "norm_feed_forward", "inv_freq", "qkv", "o", "gate_up", "down")]


class BlockStep(Structure):
    _fields_ = [(name, c_int) for name in ("n_tokens", "n_entries", "max_q_len", "n_single", "n_multi", "decode_splits", "decode_rotates", "own_launches")] + \
               [(name, c_void_p) for name in ("positions", "token_slot", "q_start", "kv_start", "slots", "residual", "normed",
                                              "qkv", "q", "attn", "o_out", "gate_up", "act", "out", "split_scratch",
                                              "split_counters", "error_word")]


_configured = False


def _function():
    global _configured
    fn = ops.lib().tib_prenorm_gqa_glu_block
    if not _configured:
        fn.restype = c_int
        fn.argtypes = [POINTER(BlockWeights), POINTER(BlockStep), c_void_p, c_void_p, c_void_p, c_int, c_int, c_int64, c_int,
                       c_int, c_void_p]
        _configured = True
    return fn


def _matrix(weight: LinearWeight) -> tuple[int, int]:
    return weight.tensor.data_ptr(), 1 if weight.transposed else 0


def block_weights(block) -> BlockWeights | None:
    """The description of ``block`` for the native call, or None when it is not made of the built-in parts."""
    from torchinferno_b200.parts.attention import GQAAttention
    from torchinferno_b200.parts.mlp import SwiGLUFeedForward
    from torchinferno_b200.parts.norm import RMSNorm
    from torchinferno_b200.parts.rope import NoPositionEncoding, RotaryEncoding
    mixer, ffn, n1, n2 = block.mixer, block.feed_forward, block.mixer_norm, block.feed_forward_norm
    if block.dtype != torch.bfloat16 or block.device.type != "cuda" or gemm.get_backend() == "tcgen05":
        return None
    if type(mixer) is not GQAAttention or type(ffn) is not SwiGLUFeedForward or type(n1) is not RMSNorm or type(n2) is not RMSNorm:
        return None
    position = mixer.position
    if type(position) not in (RotaryEncoding, NoPositionEncoding):
        return None
    if not ops.attention_mma_supports(mixer.head_dim, mixer.heads // mixer.kv_heads):
        return None
    matrices = (mixer.qkv_weight, mixer.o_weight, ffn.gate_up_weight, ffn.down_weight)
    if any(m is None or m.dtype != torch.bfloat16 for m in matrices) or n1.weight is None or n2.weight is None:
        return None
    w = BlockWeights()
    w.hidden, w.heads, w.kv_heads, w.head_dim = mixer.hidden_size, mixer.heads, mixer.kv_heads, mixer.head_dim
    w.intermediate = ffn.intermediate_size
    rotary = type(position) is RotaryEncoding
    w.rot_dim, w.interleaved = (position.rot_dim, int(position.interleaved)) if rotary else (0, 0)
    w.inv_freq = position.inv_freq.data_ptr() if rotary else None
    (w.qkv, w.qkv_kn), (w.o, w.o_kn) = _matrix(mixer.qkv_weight), _matrix(mixer.o_weight)
    (w.gate_up, w.gate_up_kn), (w.down, w.down_kn) = _matrix(ffn.gate_up_weight), _matrix(ffn.down_weight)
    auto = gemm.get_backend() == "auto"
    w.qkv_few_rows, w.o_few_rows = (m.few_rows if auto else 0 for m in (mixer.qkv_weight, mixer.o_weight))
    w.gate_up_few_rows, w.down_few_rows = (m.few_rows if auto else 0 for m in (ffn.gate_up_weight, ffn.down_weight))
    for name, m in (("qkv", mixer.qkv_weight), ("o", mixer.o_weight), ("gate_up", ffn.gate_up_weight), ("down", ffn.down_weight)):
        setattr(w, name + "_features", m.features)
        setattr(w, name + "_splits", m.splits)
        setattr(w, name + "_stages", m.stages)
    if ffn.gate_up_weight.epilogue != "swiglu":
        return None
    w.eps_mixer, w.eps_feed_forward, w.scale = n1.eps, n2.eps, mixer.scale
    w.norm_mixer, w.norm_feed_forward = n1.weight.data_ptr(), n2.weight.data_ptr()
    return w


class StepWorkspace:
    """The buffers one step's blocks work in (shared by all layers: they run one after another), and the
    step's side of the native call.  Kept on the batch, so a captured step keeps its buffers."""

    def __init__(self, batch, residual: torch.Tensor, w: BlockWeights, error_word: torch.Tensor | None) -> None:
        n, dev, bf16 = batch.n_tokens, residual.device, torch.bfloat16
        q_width, kv_width = w.heads * w.head_dim, w.kv_heads * w.head_dim
        self.key = (w.hidden, w.heads, w.kv_heads, w.head_dim, w.intermediate)
        sizes = {"normed": w.hidden, "qkv": q_width + 2 * kv_width, "q": q_width, "attn": q_width, "o_out": w.hidden,
                 "gate_up": 2 * w.intermediate, "act": w.intermediate, "out": w.hidden}
        self.buffers = {name: torch.empty((n, width), dtype=bf16, device=dev) for name, width in sizes.items()}
        splits = ops.decode_num_splits(batch.n_entries, w.heads, w.kv_heads, batch.max_kv_len) if batch.n_single else 1
        self.scratch = torch.empty(batch.n_entries * w.heads * splits * (w.head_dim + 2), dtype=torch.float32, device=dev) \
            if splits > 1 else None
        counters = ops._split_counters(dev, batch.n_entries * w.kv_heads) if splits > 1 else None
        ops.library_gemm_ready(dev)
        s = self.step = BlockStep()
        s.n_tokens, s.n_entries, s.max_q_len, s.n_single, s.n_multi = n, batch.n_entries, batch.max_q_len, batch.n_single, batch.n_multi
        s.decode_splits = splits
        from torchinferno_b200.kernels import attention
        s.decode_rotates = int(attention.DECODE_ROTATES)
        for name in ("positions", "token_slot", "q_start", "kv_start", "slots"):
            setattr(s, name, getattr(batch, name).data_ptr())
        s.residual = residual.data_ptr()
        for name, tensor in self.buffers.items():
            setattr(s, name, tensor.data_ptr())
        s.split_scratch = None if self.scratch is None else self.scratch.data_ptr()
        s.split_counters = None if counters is None else counters.data_ptr()
        s.error_word = None if error_word is None else error_word.data_ptr()
        self.residual = residual


def run_block(w: BlockWeights, stream_state, ctx, window: int | None) -> None:
    """The block on ``stream_state`` (a ResidualStream): its result is left pending there."""
    batch, kv = ctx.batch, ctx.kv
    ws = getattr(batch, "native_workspace", None)
    key = (w.hidden, w.heads, w.kv_heads, w.head_dim, w.intermediate)
    if ws is None or ws.key != key or ws.residual is not stream_state.residual:
        ws = batch.native_workspace = StepWorkspace(batch, stream_state.residual, w, ctx.error_word)
    pending = stream_state.pending
    if pending is not None and (pending.dtype != torch.bfloat16 or not pending.is_contiguous()):
        raise ops.KernelError("native block: the pending delta must be contiguous bfloat16")
    status = _function()(ctypes.byref(w), ctypes.byref(ws.step), None if pending is None else pending.data_ptr(),
                         kv.pool.data_ptr(), kv.block_table.data_ptr(), kv.block_table.stride(0), kv.page_size,
                         kv.pool.stride(0), kv.pool.shape[0], int(window or 0),
                         torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))
    if status:
        raise ops.KernelError(f"native block: status {status} (negative: refused arguments; 20000 + n: cuBLAS status n; "
                              f"else a CUDA error at launch)")
    ops.count_launches(ws.step.own_launches)      # this library's own kernels among them (the library products are not counted)
    stream_state.pending = ws.buffers["out"]
