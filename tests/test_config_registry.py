"""Configuration parsing, its errors, and the architecture registry (CPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from torchinferno_b200.config.model_config import ConfigError, LlamaConfig, RopeScaling, read_config_json
from torchinferno_b200.config.registry import (ArchitectureEntry, register_architecture, registered_architectures,
                                               resolve_architecture, unregister_architecture)


def test_reads_every_key_and_derives_head_dim():
    a = LlamaConfig.from_dict(TINY_A)
    assert (a.vocab_size, a.hidden_size, a.intermediate_size, a.num_hidden_layers) == (256, 64, 128, 2)
    assert (a.num_attention_heads, a.num_key_value_heads, a.head_dim, a.group_size) == (4, 2, 16, 2)
    assert a.rope_theta == 10000.0 and a.rope_scaling is None and a.rms_norm_eps == 1e-5 and not a.tie_word_embeddings
    b = LlamaConfig.from_dict(TINY_B)
    assert b.head_dim == 32 and b.tie_word_embeddings and b.rms_norm_eps == 1e-6
    assert b.rope_scaling == RopeScaling("llama3", 8.0, 1.0, 4.0, 64)
    c = LlamaConfig.from_dict(TINY_C)
    assert c.head_dim == 48 and c.hidden_size != c.head_dim * c.num_attention_heads


def test_aliases_and_round_trip():
    cfg = dict(TINY_A)
    cfg["n_layers"] = cfg.pop("num_hidden_layers")
    cfg["num_kv_heads"] = cfg.pop("num_key_value_heads")
    cfg["max_seq_len"] = cfg.pop("max_position_embeddings")
    a = LlamaConfig.from_dict(cfg)
    assert a.num_hidden_layers == 2 and a.num_key_value_heads == 2 and a.max_position_embeddings == 128
    assert LlamaConfig.from_dict(a.to_dict()) == a
    assert LlamaConfig.from_dict(LlamaConfig.from_dict(TINY_B).to_dict()) == LlamaConfig.from_dict(TINY_B)


def test_parameter_count_of_the_8b_sizes():
    cfg = LlamaConfig.from_dict({
        "vocab_size": 128256, "hidden_size": 4096, "intermediate_size": 14336, "num_hidden_layers": 32,
        "num_attention_heads": 32, "num_key_value_heads": 8, "max_position_embeddings": 131072,
        "rope_theta": 500000.0, "rms_norm_eps": 1e-5})
    assert cfg.parameter_count() == 8_030_261_248


def test_missing_keys_are_listed_together():
    cfg = {k: v for k, v in TINY_A.items() if k not in ("vocab_size", "rope_theta", "rms_norm_eps")}
    with pytest.raises(ConfigError) as err:
        LlamaConfig.from_dict(cfg)
    for key in ("vocab_size", "rope_theta", "rms_norm_eps"):
        assert key in str(err.value)


@pytest.mark.parametrize("patch, word", [
    ({"num_key_value_heads": 3}, "divisible"),
    ({"hidden_size": 66}, "divisible"),
    ({"head_dim": 15}, "even"),
    ({"vocab_size": 0}, "positive"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"mlp_bias": True}, "mlp_bias"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 2.0}}, "yarn"),
    ({"rope_scaling": {"rope_type": "llama3", "factor": 8.0}}, "lacks keys"),
    ({"rope_scaling": {"factor": 8.0}}, "rope_type"),
    ({"num_hidden_layers": 2.5}, "integer"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps"),
])
def test_bad_values_are_refused(patch, word):
    with pytest.raises(ConfigError) as err:
        LlamaConfig.from_dict({**TINY_A, **patch})
    assert word in str(err.value)


def test_rope_scaling_type_synonym_and_default():
    block = dict(TINY_B["rope_scaling"])
    block["type"] = block.pop("rope_type")
    assert LlamaConfig.from_dict({**TINY_B, "rope_scaling": block}).rope_scaling.rope_type == "llama3"
    assert LlamaConfig.from_dict({**TINY_B, "rope_scaling": {"rope_type": "default"}}).rope_scaling is None


def test_read_config_json(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert read_config_json(tmp_path)["hidden_size"] == 64
    with pytest.raises(FileNotFoundError):
        read_config_json(tmp_path / "nowhere")
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        read_config_json(tmp_path)


def test_registry_resolves_by_architecture_and_model_type():
    assert resolve_architecture(TINY_A).name == "LlamaForCausalLM"
    assert resolve_architecture({"model_type": "llama3"}).name == "LlamaForCausalLM"
    assert resolve_architecture({"architectures": ["llamaforcausallm"]}).name == "LlamaForCausalLM"
    assert "LlamaForCausalLM" in registered_architectures()
    with pytest.raises(ValueError, match="unsupported model identity"):
        resolve_architecture({"model_type": "gpt2", "architectures": ["GPT2LMHeadModel"]})


def test_registry_rejects_conflicts_and_duplicates():
    other = ArchitectureEntry("ToyForCausalLM", LlamaConfig, lambda c: None, model_types=("toy",))
    register_architecture(other)
    try:
        with pytest.raises(ValueError, match="conflicting model identity"):
            resolve_architecture({"model_type": "toy", "architectures": ["LlamaForCausalLM"]})
        with pytest.raises(ValueError, match="conflicting model architectures"):
            resolve_architecture({"architectures": ["LlamaForCausalLM", "ToyForCausalLM"]})
        with pytest.raises(ValueError, match="already registered"):
            register_architecture(ArchitectureEntry("ToyForCausalLM", LlamaConfig, lambda c: None))
    finally:
        unregister_architecture("ToyForCausalLM")
    with pytest.raises(ValueError):
        resolve_architecture({"model_type": "toy"})


def test_model_spec_is_data_and_checks_its_schedule():
    from torchinferno_b200.models.llama import build_llama
    from torchinferno_b200.models.spec import LayerCall
    import dataclasses
    spec = build_llama(LlamaConfig.from_dict(TINY_B))
    assert len(spec.layers) == 3 and [c.cache for c in spec.schedule] == [0, 1, 2] and spec.cache_layers == 3
    assert spec.tie_head_to_embedding
    # a layer may run twice and a call may read another call's cache
    twice = dataclasses.replace(spec, schedule=(LayerCall(0, 0), LayerCall(1, 1), LayerCall(0, 2), LayerCall(2, 1, writes_cache=False)))
    assert twice.cache_layers == 3
    with pytest.raises(ValueError, match="read before"):
        dataclasses.replace(spec, schedule=(LayerCall(0, 0, writes_cache=False),))
    with pytest.raises(ValueError, match="written by two"):
        dataclasses.replace(spec, schedule=(LayerCall(0, 0), LayerCall(1, 0)))
    with pytest.raises(ValueError, match="names layer"):
        dataclasses.replace(spec, schedule=(LayerCall(7, 0),))


def test_engine_config_keeps_the_reference_names_and_checks_its_values():
    """Names and defaults of src/torchinferno/engine/config.py:40-61 where the reference has them."""
    from torchinferno_b200.config.engine_config import EngineConfig
    c = EngineConfig(model="m")
    assert (c.model_kind, c.dtype, c.cache_backend, c.page_size, c.max_batch_size) == ("auto", "auto", "paged", 16, 64)
    assert c.async_scheduling and c.use_cuda_graphs and c.gemm_backend == "auto" and c.cache_memory_fraction == 0.9
    for bad in (dict(cache_backend="dense"), dict(page_size=0), dict(max_batch_size=0), dict(max_num_batched_tokens=0),
                dict(cache_memory_fraction=0.0), dict(cache_memory_fraction=1.5)):
        with pytest.raises(ValueError):
            EngineConfig(model="m", **bad)
