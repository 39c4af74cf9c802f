"""Random weights: every matrix N(0, std) and every norm vector 1, from a seed.

Each tensor has a generator of its own, keyed by (seed, tensor name), so a
tensor's values do not depend on which other tensors exist or on their order.
The reference has no such mode; its tests build an eager model under
``torch.manual_seed`` and write it out to load it back
(tests/test_model_variants.py:319-354 in the reference project).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any, Mapping

import torch

from torchinferno_b200.config.registry import resolve_architecture
from torchinferno_b200.weights.loader import SINGLE_FILE, place


def _tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def random_tensor(spec, seed: int, *, device: torch.device | str = "cpu",
                  dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if spec.init == "ones":
        return torch.ones(spec.shape, dtype=dtype, device=device)
    if spec.init == "zeros":
        return torch.zeros(spec.shape, dtype=dtype, device=device)
    if spec.init != "normal":
        raise ValueError(f"unknown init {spec.init!r} for {spec.name}")
    generator = torch.Generator(device=device)
    generator.manual_seed(_tensor_seed(seed, spec.name))
    out = torch.empty(spec.shape, dtype=torch.float32, device=device)
    out.normal_(0.0, spec.std, generator=generator)
    return out.to(dtype)


def build_model(config: Mapping[str, Any], *, dtype: torch.dtype, device: torch.device | str):
    """The model that ``config`` (a config.json as a dict) names, without weights."""
    from torchinferno_b200.models.model import CausalLM
    entry = resolve_architecture(config)
    typed = entry.config_class.from_dict(config)
    return CausalLM(entry.build(typed), dtype=dtype, device=device)


def write_random_model(config: Mapping[str, Any], folder: str | Path, seed: int,
                       dtype: torch.dtype = torch.bfloat16) -> Path:
    """Write ``config.json`` and ``model.safetensors`` with seeded random weights."""
    from safetensors.torch import save_file
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    config = dict(config)
    config["torch_dtype"] = str(dtype).replace("torch.", "")
    model = build_model(config, dtype=torch.float32, device="cpu")
    tensors = {}
    for name, spec in model.expected_tensors().items():
        if spec.optional:
            continue  # e.g. a head tied to the embedding is not stored
        tensors[name] = random_tensor(spec, seed, dtype=dtype).contiguous()
    (folder / "config.json").write_text(json.dumps(config, indent=1) + "\n")
    save_file(tensors, str(folder / SINGLE_FILE), metadata={"format": "pt", "seed": str(seed)})
    return folder


def init_random_weights(model, seed: int, storage_dtype: torch.dtype = torch.bfloat16) -> None:
    """Bind seeded random weights generated on the model's device (nothing touches the disk)."""
    tensors = {}
    for name, spec in model.expected_tensors().items():
        if spec.optional:
            continue
        raw = random_tensor(spec, seed, device=model.device, dtype=storage_dtype)
        tensors[name] = place(raw, spec.role, model.dtype, model.device)
    model.bind(tensors, consume=True)
