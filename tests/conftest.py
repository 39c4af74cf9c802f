"""Shared fixtures: pytest markers, tiny configurations, temporary model folders."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for path in (str(ROOT), str(ROOT / "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


# Two tiny configurations that differ in every size and option.
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 128,
    "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 384, "hidden_size": 192, "intermediate_size": 512, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 3, "max_position_embeddings": 512,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
}
# A third one with sizes that are no power of two, head_dim given explicitly
# (not hidden / heads), one kv head, and a vocabulary that is odd.
TINY_C = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 331, "hidden_size": 120, "intermediate_size": 200, "num_hidden_layers": 2,
    "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 48, "max_position_embeddings": 640,
    "rope_theta": 250000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 2.0,
                     "original_max_position_embeddings": 128},
    "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
}
# Head sizes the tensor-core attention kernels are built for (64 with groups of 2, 128 with groups of 4).
TINY_D = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 300, "hidden_size": 256, "intermediate_size": 320, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "max_position_embeddings": 1024,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 256},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
TINY_E = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "vocab_size": 270, "hidden_size": 160, "intermediate_size": 224, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128, "max_position_embeddings": 1024,
    "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
}
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 2), "D": (TINY_D, 3), "E": (TINY_E, 4)}


@pytest.fixture(autouse=True)
def same_random_data_every_run():
    """Data drawn from torch's global generator is the same for a test whatever ran before it."""
    import torch
    torch.manual_seed(20240607)


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> folder with config.json + model.safetensors (bf16 storage, seeded)."""
    from torchinferno_b200.weights.random_init import write_random_model
    folders = {}
    for name, (config, seed) in TINY.items():
        folder = tmp_path_factory.mktemp(f"tiny{name}")
        write_random_model(config, folder, seed)
        folders[name] = folder
    return folders


def pytest_terminal_summary(terminalreporter):
    """The largest error each comparison with the plain implementation saw, as a share of its tolerance."""
    try:
        from gpu_common import WORST
    except Exception:
        return
    if not WORST:
        return
    terminalreporter.section("largest error / tolerance")
    by_dtype: dict[str, float] = {}
    for what, share in sorted(WORST.items(), key=lambda kv: -kv[1])[:12]:
        terminalreporter.write_line(f"{share:6.3f}  {what}")
    for what, share in WORST.items():
        kind = "bfloat16" if "bfloat16" in what else "float32"
        by_dtype[kind] = max(by_dtype.get(kind, 0.0), share)
    terminalreporter.write_line("worst by dtype: " + ", ".join(f"{k} {v:.3f}" for k, v in sorted(by_dtype.items())))
