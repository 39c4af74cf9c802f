"""Llama 3 as a description made of parts.

Layer recipe and tensor names: src/torchinferno/models/llama3/pipeline.py:173-250,
306-326.  Every layer is a pre-norm block of grouped-query attention with
rotary positions (llama3 scaling when the configuration asks for it) and a
SwiGLU feed-forward; layer i uses cache layer i.
"""
from __future__ import annotations

from torchinferno_b200.config.model_config import LlamaConfig
from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture
from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
from torchinferno_b200.parts.base import PartSpec


def build_llama(config: LlamaConfig) -> ModelSpec:
    scaling = None if config.rope_scaling is None else config.rope_scaling.to_dict()
    position = PartSpec("rotary", {"head_dim": config.head_dim, "theta": config.rope_theta, "scaling": scaling})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": config.hidden_size, "heads": config.num_attention_heads,
        "kv_heads": config.num_key_value_heads, "head_dim": config.head_dim, "position": position,
    }, prefix="self_attn.")
    feed_forward = PartSpec("swiglu", {
        "hidden_size": config.hidden_size, "intermediate_size": config.intermediate_size}, prefix="mlp.")
    norm = {"width": config.hidden_size, "eps": config.rms_norm_eps}
    block = PartSpec("prenorm", {
        "mixer": mixer, "feed_forward": feed_forward,
        "mixer_norm": PartSpec("rmsnorm", norm, prefix="input_layernorm."),
        "feed_forward_norm": PartSpec("rmsnorm", norm, prefix="post_attention_layernorm."),
    })
    layers = tuple(BlockSpec(block, f"model.layers.{i}.") for i in range(config.num_hidden_layers))
    schedule = tuple(LayerCall(layer=i, cache=i) for i in range(config.num_hidden_layers))
    return ModelSpec(
        architecture="LlamaForCausalLM", hidden_size=config.hidden_size, vocab_size=config.vocab_size,
        max_positions=config.max_position_embeddings, embedding_name="model.embed_tokens.weight",
        layers=layers, schedule=schedule, final_norm=PartSpec("rmsnorm", norm, prefix="model.norm."),
        head_name="lm_head.weight", tie_head_to_embedding=config.tie_word_embeddings,
        config=config.to_dict())


LLAMA = register_architecture(ArchitectureEntry(
    name="LlamaForCausalLM", aliases=("Llama3ForCausalLM",), model_types=("llama", "llama3"),
    config_class=LlamaConfig, build=build_llama))
