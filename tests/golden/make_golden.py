"""Compare tests/plain_llama.py with the reference project's own Llama 3 code, once, on the CPU.

Run from the repository root with the reference's sources on the path:

    PYTHONPATH=<reference>/src:. HF_HUB_OFFLINE=1 python tests/golden/make_golden.py

It writes a tiny random model (seeded) to a temporary folder in the form the
reference's loader wants (HF tensor names, an index file, ``lm_head.weight``
stored even when tied: src/torchinferno/models/llama3/pipeline.py:83-87, 308),
runs ``Llama3PipelineForCausalLM`` in float32 on the CPU and stores, in
``tests/golden/llama_tiny.json``: the configuration, the seed, the token ids and
the reference's logits of the last four positions plus its greedy continuation.
``tests/test_plain_reference.py`` regenerates the same weights from the seed and
checks the plain implementation against these numbers.
"""
from __future__ import annotations

import json
import sys
import tempfile
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))

CONFIGS = {
    "plain_rope": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 96, "hidden_size": 48,
        "intermediate_size": 80, "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2,
        "max_position_embeddings": 128, "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
        "tie_word_embeddings": False,
    },
    "llama3_rope": {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 120, "hidden_size": 96,
        "intermediate_size": 176, "num_hidden_layers": 3, "num_attention_heads": 6, "num_key_value_heads": 3,
        "max_position_embeddings": 256, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    },
}


def golden_weights(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Seeded fp32 weights, N(0, 0.02) matrices (norm vectors near 1 so that they matter)."""
    g = torch.Generator().manual_seed(seed)
    h, i, v = config["hidden_size"], config["intermediate_size"], config["vocab_size"]
    heads, kv = config["num_attention_heads"], config["num_key_value_heads"]
    d = h // heads

    def mat(*shape):
        return torch.randn(*shape, generator=g) * 0.02 * 4  # larger than 0.02 so logits are not all alike

    def vec(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g)

    w = {"model.embed_tokens.weight": mat(v, h), "model.norm.weight": vec(h)}
    for layer in range(config["num_hidden_layers"]):
        p = f"model.layers.{layer}."
        w[p + "input_layernorm.weight"] = vec(h)
        w[p + "post_attention_layernorm.weight"] = vec(h)
        w[p + "self_attn.q_proj.weight"] = mat(heads * d, h)
        w[p + "self_attn.k_proj.weight"] = mat(kv * d, h)
        w[p + "self_attn.v_proj.weight"] = mat(kv * d, h)
        w[p + "self_attn.o_proj.weight"] = mat(h, heads * d)
        w[p + "mlp.gate_proj.weight"] = mat(i, h)
        w[p + "mlp.up_proj.weight"] = mat(i, h)
        w[p + "mlp.down_proj.weight"] = mat(h, i)
    w["lm_head.weight"] = w["model.embed_tokens.weight"].clone() if config["tie_word_embeddings"] else mat(v, h)
    return w


def golden_tokens(config: dict, seed: int, length: int) -> list[int]:
    g = torch.Generator().manual_seed(seed + 1000)
    return torch.randint(0, config["vocab_size"], (length,), generator=g).tolist()


def main() -> None:
    from safetensors.torch import save_file
    from torchinferno.models.llama3.pipeline import Llama3PipelineForCausalLM

    out = {}
    for seed, (name, config) in enumerate(CONFIGS.items()):
        weights = golden_weights(config, seed)
        tokens = golden_tokens(config, seed, 90)
        with tempfile.TemporaryDirectory() as tmp:
            folder = Path(tmp)
            (folder / "config.json").write_text(json.dumps(config))
            save_file({k: t.contiguous() for k, t in weights.items()}, str(folder / "model.safetensors"))
            (folder / "model.safetensors.index.json").write_text(json.dumps(
                {"metadata": {}, "weight_map": {k: "model.safetensors" for k in weights}}))
            model = Llama3PipelineForCausalLM.from_pretrained(str(folder), devices=["cpu"], dtype=torch.float32)
            logits, _ = model.forward(torch.tensor([tokens]), use_cache=False)
            generated = model.generate(torch.tensor([tokens[:20]]), max_new_tokens=6, temperature=0.0)
        out[name] = {
            "config": config, "seed": seed, "tokens": tokens,
            "last_logits": logits[0, -4:].double().tolist(),
            "greedy_prompt_len": 20, "greedy_tokens": generated[0, 20:].tolist(),
        }
    (HERE / "llama_tiny.json").write_text(json.dumps(out))
    print("wrote", HERE / "llama_tiny.json")


if __name__ == "__main__":
    main()
