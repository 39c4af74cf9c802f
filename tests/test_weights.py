"""Weight loading: names, shapes, storage rule, errors; random mode (CPU)."""
import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY_A, TINY_B
from torchinferno_b200.weights.loader import WeightError, checkpoint_files, load_weights, place
from torchinferno_b200.weights.random_init import build_model, write_random_model


def _model(cfg, dtype=torch.bfloat16):
    return build_model(cfg, dtype=dtype, device="cpu")


def test_random_folder_has_every_tensor_and_loads(tmp_path):
    write_random_model(TINY_A, tmp_path, seed=0)
    cfg = json.loads((tmp_path / "config.json").read_text())
    assert cfg["torch_dtype"] == "bfloat16" and cfg["hidden_size"] == 64
    tensors = load_file(str(tmp_path / "model.safetensors"))
    model = _model(TINY_A)
    assert set(tensors) == set(model.expected_tensors())
    assert all(t.dtype == torch.bfloat16 for t in tensors.values())
    assert torch.all(tensors["model.norm.weight"] == 1)
    w = tensors["model.layers.1.mlp.down_proj.weight"].float()
    assert w.shape == (64, 128) and abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    report = load_weights(model, tmp_path)
    assert report["tensors"] == len(tensors) and report["stored_dtypes"] == ["bfloat16"]
    block = model.blocks[0]
    assert block.mixer.qkv_weight.tensor.shape == ((4 + 2 * 2) * 16, 64) and block.mixer.qkv_weight.dtype == torch.bfloat16
    assert torch.equal(block.mixer.qkv_weight.tensor[:64], tensors["model.layers.0.self_attn.q_proj.weight"])
    assert torch.equal(block.mixer.qkv_weight.tensor[64:96], tensors["model.layers.0.self_attn.k_proj.weight"])
    # (gate and up rows are interleaved: row 2i = gate i, row 2i + 1 = up i)
    assert torch.equal(block.feed_forward.gate_up_weight.tensor[1::2], tensors["model.layers.0.mlp.up_proj.weight"])
    assert torch.equal(block.feed_forward.gate_up_weight.tensor[0::2], tensors["model.layers.0.mlp.gate_proj.weight"])
    assert block.mixer_norm.weight.dtype == torch.float32          # vectors are widened
    assert model.head is not model.embedding


def test_seed_and_name_decide_the_values(tmp_path):
    write_random_model(TINY_A, tmp_path / "a", seed=3)
    write_random_model(TINY_A, tmp_path / "b", seed=3)
    write_random_model(TINY_A, tmp_path / "c", seed=4)
    a, b, c = (load_file(str(tmp_path / n / "model.safetensors")) for n in "abc")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    assert not torch.equal(a["model.layers.0.mlp.gate_proj.weight"], a["model.layers.0.mlp.up_proj.weight"])
    fewer = {**TINY_A, "num_hidden_layers": 1}
    write_random_model(fewer, tmp_path / "d", seed=3)
    d = load_file(str(tmp_path / "d" / "model.safetensors"))
    assert all(torch.equal(a[k], d[k]) for k in d)               # independent of which other tensors exist


def test_tied_head_is_not_stored_and_is_shared(tmp_path):
    write_random_model(TINY_B, tmp_path, seed=1)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    assert "lm_head.weight" not in tensors
    model = _model(TINY_B)
    load_weights(model, tmp_path)
    assert model.head is model.embedding
    # a tied checkpoint that also stores the head is accepted (the head is optional when tied)
    tensors["lm_head.weight"] = tensors["model.embed_tokens.weight"].clone()
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(16)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    model = _model(TINY_B)
    report = load_weights(model, tmp_path)
    assert model.head is model.embedding and report["not_read"] == ["lm_head.weight"]
    assert report["ignored"] == ["model.layers.0.self_attn.rotary_emb.inv_freq"]


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    write_random_model(TINY_A, tmp_path, seed=0)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    del tensors["model.layers.0.self_attn.k_proj.weight"]
    del tensors["model.norm.weight"]
    tensors["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(8)      # a known harmless buffer: ignored
    tensors["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(8)
    tensors["model.layers.1.mlp.up_proj.weight"] = torch.zeros(64, 128, dtype=torch.bfloat16)
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as err:
        load_weights(_model(TINY_A), tmp_path)
    text = str(err.value)
    assert "missing (2)" in text and "model.layers.0.self_attn.k_proj.weight" in text and "model.norm.weight" in text
    assert "unexpected (1)" in text and "q_norm.weight" in text and "inv_freq" not in text
    assert "wrong shape (1)" in text and "model.layers.1.mlp.up_proj.weight: file [64, 128] vs model [128, 64]" in text


def test_untied_model_needs_its_head(tmp_path):
    write_random_model(TINY_A, tmp_path, seed=0)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    del tensors["lm_head.weight"]
    save_file(tensors, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError, match="lm_head.weight"):
        load_weights(_model(TINY_A), tmp_path)


def test_storage_rule():
    bf, f32, f16 = torch.ones(2, 2, dtype=torch.bfloat16), torch.ones(2, 2), torch.ones(2, 2, dtype=torch.float16)
    cpu = torch.device("cpu")
    assert place(bf, "matrix", torch.bfloat16, cpu).dtype == torch.bfloat16
    assert place(f32, "matrix", torch.bfloat16, cpu).dtype == torch.float32      # stored in 32-bit stays so
    assert place(f16, "matrix", torch.bfloat16, cpu).dtype == torch.bfloat16
    assert place(bf, "vector", torch.bfloat16, cpu).dtype == torch.float32
    assert place(bf, "matrix", torch.float32, cpu).dtype == torch.float32        # the 32-bit path widens all
    assert place(torch.ones(3, dtype=torch.int64), "int_table", torch.bfloat16, cpu).dtype == torch.int32


def test_sharded_checkpoint_with_index(tmp_path):
    write_random_model(TINY_A, tmp_path, seed=0)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    (tmp_path / "model.safetensors").unlink()
    names = sorted(tensors)
    shards = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    weight_map = {}
    for shard, members in shards.items():
        save_file({n: tensors[n] for n in members}, str(tmp_path / shard))
        weight_map.update({n: shard for n in members})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    assert len(checkpoint_files(tmp_path)) == len(names)
    model = _model(TINY_A)
    load_weights(model, tmp_path)
    assert torch.equal(model.embedding, tensors["model.embed_tokens.weight"])
    weight_map[names[0]] = "../outside.safetensors"
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps({"weight_map": weight_map}))
    with pytest.raises(WeightError, match="inside the folder"):
        checkpoint_files(tmp_path)


def test_no_checkpoint_at_all(tmp_path):
    with pytest.raises(FileNotFoundError):
        checkpoint_files(tmp_path)
