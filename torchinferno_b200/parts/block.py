"""The arrangement of parts in one layer.

Pre-norm block (src/torchinferno/models/llama3/pipeline.py:190-198):
    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))
The adds are left pending on the residual stream so the next norm (of this
block, of the next block or the final one) does them in its own pass
(src/torchinferno/models/llama3/tensor_parallel.py:7430-7435).
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import gemm, native_block
from torchinferno_b200.parts.base import (Block, LayerContext, Part, PartSpec, ResidualStream,
                                          build_part, register_part)


NATIVE_BLOCKS = True          # False: always the part-by-part sequence
_UNKNOWN = object()


def _spec(value: PartSpec | Mapping) -> PartSpec:
    return value if isinstance(value, PartSpec) else PartSpec(**value)


class PreNormBlock(Block):
    def __init__(self, *, mixer: PartSpec, feed_forward: PartSpec, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec, dtype: torch.dtype, device: torch.device) -> None:
        super().__init__(dtype=dtype, device=device)
        self.specs = {"mixer": _spec(mixer), "feed_forward": _spec(feed_forward),
                      "mixer_norm": _spec(mixer_norm), "feed_forward_norm": _spec(feed_forward_norm)}
        self.mixer = build_part("mixer", self.specs["mixer"], dtype=dtype, device=device)
        self.feed_forward = build_part("feed_forward", self.specs["feed_forward"], dtype=dtype, device=device)
        self.mixer_norm = build_part("norm", self.specs["mixer_norm"], dtype=dtype, device=device)
        self.feed_forward_norm = build_part("norm", self.specs["feed_forward_norm"], dtype=dtype, device=device)
        self._native = _UNKNOWN
        self._native_generation = -1

    def named_parts(self) -> list[tuple[str, Part]]:
        return [(self.specs["mixer_norm"].prefix, self.mixer_norm),
                (self.specs["mixer"].prefix, self.mixer),
                (self.specs["feed_forward_norm"].prefix, self.feed_forward_norm),
                (self.specs["feed_forward"].prefix, self.feed_forward)]

    def forward(self, stream: ResidualStream, ctx: LayerContext) -> None:
        if self._native is _UNKNOWN or self._native_generation != gemm.generation():
            # (decided at the first use, when the weights are bound, and again whenever a weight was bound or a
            # kernel choice changed since: a block of the built-in parts in bfloat16 is issued as one call into
            # the CUDA library, the same kernels in the same order)
            self._native = native_block.block_weights(self) if NATIVE_BLOCKS else None
            self._native_generation = gemm.generation()
        if self._native is not None and ctx.kv is not None and ctx.kv.writes and ctx.batch is not None:
            window = self.mixer.window if self.mixer.window is not None else ctx.kv.window
            native_block.run_block(self._native, stream, ctx, window)
            return
        stream.add(self.mixer.forward(stream.normed(self.mixer_norm), ctx))
        stream.add(self.feed_forward.forward(stream.normed(self.feed_forward_norm), ctx))


register_part("block", "prenorm", PreNormBlock)
