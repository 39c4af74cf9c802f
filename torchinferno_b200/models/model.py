"""The runnable model: parts built from a :class:`ModelSpec`, weights bound by name.

One forward pass serves every kind of step: it embeds the tokens of a ragged
batch, runs the schedule of layer calls against the cache, norms only the rows
whose logits are wanted and projects them to the vocabulary
(src/torchinferno/models/llama3/tensor_parallel.py:7088-7090 gathers before the
head likewise).  Logits are fp32.
"""
from __future__ import annotations

from typing import Mapping

import torch

from torchinferno_b200.kernels import gemm, ops
from torchinferno_b200.kernels.gemm import linear
from torchinferno_b200.models.spec import ModelSpec
from torchinferno_b200.parts.base import (Block, CacheSpec, KVBinding, LayerContext, ResidualStream,
                                          StateSpec, WeightSpec, build_part)


class CausalLM:
    def __init__(self, spec: ModelSpec, *, dtype: torch.dtype, device: torch.device | str) -> None:
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"compute dtype must be float32 or bfloat16, got {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.blocks: list[Block] = [
            build_part("block", layer.block, dtype=dtype, device=self.device) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, dtype=dtype, device=self.device)
        self.after_embedding = None if spec.after_embedding is None else \
            build_part("stream_stage", spec.after_embedding, dtype=dtype, device=self.device)
        self.embedding: torch.Tensor | None = None
        self.head: torch.Tensor | None = None

    # ------------------------------------------------------------ weights
    def expected_tensors(self) -> dict[str, WeightSpec]:
        """Every tensor the model reads, by full checkpoint name."""
        spec = self.spec
        expected: dict[str, WeightSpec] = {
            spec.embedding_name: WeightSpec(spec.embedding_name, (spec.vocab_size, spec.hidden_size))}
        for layer, block in zip(spec.layers, self.blocks):
            for prefix, part in block.named_parts():
                for ws in part.weight_specs():
                    name = layer.prefix + prefix + ws.name
                    expected[name] = WeightSpec(name, ws.shape, ws.init, ws.std, ws.role, ws.optional)
        for part, part_spec in ((self.final_norm, spec.final_norm), (self.after_embedding, spec.after_embedding)):
            for ws in (part.weight_specs() if part is not None else ()):
                name = part_spec.prefix + ws.name
                expected[name] = WeightSpec(name, ws.shape, ws.init, ws.std, ws.role, ws.optional)
        if spec.head_name is not None:
            expected[spec.head_name] = WeightSpec(
                spec.head_name, (spec.vocab_size, spec.hidden_size), optional=spec.tie_head_to_embedding)
        return expected

    def unused_optional_tensors(self) -> list[str]:
        """Optional tensors that are not read even when the file has them (a head tied to the embedding)."""
        spec = self.spec
        return [spec.head_name] if spec.tie_head_to_embedding and spec.head_name is not None else []

    def bind(self, tensors: Mapping[str, torch.Tensor], consume: bool = False) -> None:
        """Give every part its tensors.  ``consume``: ``tensors`` is a dict of the caller's that is emptied part
        by part, so that a part which repacks its weights (fused projections) does not leave the sources alive
        beside the packed copy until the whole model is bound."""
        spec = self.spec
        take = tensors.pop if consume else tensors.__getitem__
        self.embedding = take(spec.embedding_name)
        if spec.tie_head_to_embedding or spec.head_name is None:
            self.head = self.embedding
        elif spec.head_name in tensors:
            self.head = take(spec.head_name)
        else:
            # An untied model whose file has no head is refused on purpose: guessing that the embedding
            # doubles as the head would turn a truncated checkpoint into silently wrong logits.
            raise KeyError(f"{spec.head_name}: the model does not tie its head to the embedding, and no head was given")
        for layer, block in zip(spec.layers, self.blocks):
            for prefix, part in block.named_parts():
                full = layer.prefix + prefix
                part.bind({ws.name: take(full + ws.name) for ws in part.weight_specs()
                           if full + ws.name in tensors})
        self.final_norm.bind({ws.name: take(spec.final_norm.prefix + ws.name)
                              for ws in self.final_norm.weight_specs()})
        if self.after_embedding is not None:
            self.after_embedding.bind({ws.name: take(spec.after_embedding.prefix + ws.name)
                                       for ws in self.after_embedding.weight_specs()
                                       if spec.after_embedding.prefix + ws.name in tensors})
        if self.device.type == "cuda":
            gemm.tune_few_rows()      # weights that left the choice of their few-rows kernel open get it now

    def weight_bytes(self) -> int:
        """Bytes of distinct weight storage one step reads (a tied head counts once)."""
        seen: dict[int, int] = {}

        def note(t: torch.Tensor | None) -> None:
            if isinstance(t, torch.Tensor):
                seen[t.data_ptr()] = t.numel() * t.element_size()

        note(self.head)
        parts = [part for block in self.blocks for _, part in block.named_parts()] + [self.final_norm]
        for part in parts:
            for key, value in vars(part).items():
                if key.endswith("weight"):
                    note(getattr(value, "tensor", value) if not isinstance(value, torch.Tensor) else value)
        return sum(seen.values())

    # -------------------------------------------------------------- needs
    def cache_requirements(self) -> list[CacheSpec]:
        """CacheSpec of every cache layer, in cache-layer order."""
        needs: dict[int, CacheSpec] = {}
        for call in self.spec.schedule:
            if call.cache is None:
                continue
            cs = self.blocks[call.layer].mixer.cache_spec()
            if cs is None:
                raise ValueError(f"layer {call.layer} is given cache layer {call.cache} but its mixer keeps no keys")
            if call.cache in needs and needs[call.cache] != cs:
                raise ValueError(f"cache layer {call.cache} is shared by mixers of different shapes")
            needs.setdefault(call.cache, cs)
        return [needs[i] for i in range(self.spec.cache_layers)]

    def capturable(self) -> bool:
        """Whether a decode step of this model may be captured in a CUDA graph (see ``Mixer.capturable``)."""
        parts = [block.mixer for block in self.blocks] + ([self.after_embedding] if self.after_embedding is not None else [])
        return all(getattr(part, "capturable", getattr(part, "state_spec", lambda: None)() is None) for part in parts)

    def state_requirements(self) -> list[StateSpec | None]:
        """StateSpec of every layer call of the schedule (None where the mixer has none)."""
        return [self.blocks[call.layer].mixer.state_spec() for call in self.spec.schedule]

    # ------------------------------------------------------------ forward
    def forward(self, batch, cache) -> torch.Tensor:
        """Run the tokens of ``batch``; return fp32 logits [len(batch.logit_rows), vocab]."""
        n = batch.n_tokens
        residual = torch.empty((n, self.spec.hidden_size), dtype=torch.float32, device=self.device)
        ops.embedding(batch.token_ids, self.embedding, residual)
        stream = ResidualStream(residual, self.dtype)
        if self.after_embedding is not None:
            self.after_embedding.forward(stream, LayerContext(batch=batch, error_word=cache.error_word, layer_index=-1))
        for index, call in enumerate(self.spec.schedule):
            kv = None
            if call.cache is not None:
                kv = cache.kv_binding(call.cache)
                kv = KVBinding(kv.pool, kv.block_table, kv.page_size, kv.window, call.writes_cache, kv.keys, kv.values)
            ctx = LayerContext(batch=batch, kv=kv, state=cache.state(index),
                               error_word=cache.error_word, layer_index=index)
            self.blocks[call.layer].forward(stream, ctx)
        if batch.n_logits == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=self.device)
        rows = stream.normed(self.final_norm, batch.logit_rows)
        return linear(rows, self.head, out_dtype=torch.float32)
