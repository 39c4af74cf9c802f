"""Weights from safetensors, bound by tensor name and checked against the model.

The reference reads tensors lazily by name through ``model.safetensors.index.json``
(src/torchinferno/models/llama3/pipeline.py:80-135) or from a lone
``model.safetensors`` (src/torchinferno/models/checkpoint_io.py:22-48), refuses
shard names that leave the folder (checkpoint_io.py:74-87) and does not compare
shapes with the configuration.  Here every name and shape is compared before
anything is copied, and one error lists all that is missing, unexpected or of
the wrong shape.

Storage rule: a tensor stored in bfloat16 stays bfloat16 and one stored in
32-bit stays 32-bit when the engine computes in bfloat16; norm vectors are
widened to fp32 (lossless); integer tables become int32.  When the engine
computes in float32 every floating tensor is widened to fp32.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Iterable

import torch

SINGLE_FILE = "model.safetensors"
INDEX_FILE = "model.safetensors.index.json"


class WeightError(ValueError):
    """The checkpoint does not hold what the model needs."""


# Buffers some exporters store beside the weights; they are recomputed from the configuration and never read.
# Anything else the model does not expect is an error.
IGNORED_SUFFIXES = ("rotary_emb.inv_freq", "self_attn.rotary_emb.inv_freq", "attn.masked_bias", "attn.bias")


_DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "F64": torch.float64,
           "I32": torch.int32, "I64": torch.int64, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool}


def _safe_open(path: Path):
    from safetensors import safe_open
    return safe_open(str(path), framework="pt", device="cpu")


def checkpoint_files(folder: str | Path) -> dict[str, Path]:
    """Tensor name -> file that holds it."""
    folder = Path(folder)
    index = folder / INDEX_FILE
    single = folder / SINGLE_FILE
    if index.is_file():
        data = json.loads(index.read_text())
        weight_map = data.get("weight_map")
        if not isinstance(weight_map, dict):
            raise WeightError(f"{index} has no weight_map")
        root = folder.resolve()
        files: dict[str, Path] = {}
        for name, shard in weight_map.items():
            shard_path = (folder / str(shard)).resolve()
            if root not in shard_path.parents or not str(shard).endswith(".safetensors"):
                raise WeightError(f"{index}: shard {shard!r} of {name!r} is not a safetensors file inside the folder")
            if not shard_path.is_file():
                raise WeightError(f"{index}: shard {shard!r} of {name!r} does not exist")
            files[str(name)] = shard_path
        return files
    if single.is_file():
        with _safe_open(single) as handle:
            return {name: single for name in handle.keys()}
    raise FileNotFoundError(f"no {SINGLE_FILE} or {INDEX_FILE} in {folder}")


def _describe(names: Iterable[str], limit: int = 12) -> str:
    names = sorted(names)
    shown = ", ".join(names[:limit])
    return shown + (f", ... (+{len(names) - limit} more)" if len(names) > limit else "")


def load_weights(model, folder: str | Path) -> dict[str, object]:
    """Check the checkpoint against ``model.expected_tensors()``, copy it to the device and bind it."""
    files = checkpoint_files(folder)
    expected = model.expected_tensors()
    handles: dict[Path, object] = {}

    def handle_of(path: Path):
        if path not in handles:
            handles[path] = _safe_open(path).__enter__()
        return handles[path]

    try:
        missing = [n for n, ws in expected.items() if n not in files and not ws.optional]
        ignored = sorted(n for n in files if n not in expected and n.endswith(IGNORED_SUFFIXES))
        unexpected = [n for n in files if n not in expected and n not in ignored]
        # a head that the model ties to its embedding is not read even if the file stores a copy
        unused = set(model.unused_optional_tensors()) if hasattr(model, "unused_optional_tensors") else set()
        wrong: list[str] = []
        for name, ws in expected.items():
            if name not in files:
                continue
            view = handle_of(files[name]).get_slice(name)
            shape = tuple(view.get_shape())
            if shape != tuple(ws.shape):
                wrong.append(f"{name}: file {list(shape)} vs model {list(ws.shape)}")
        if missing or unexpected or wrong:
            parts = [f"checkpoint {folder} does not fit the model ({model.spec.architecture}):"]
            if missing:
                parts.append(f"  missing ({len(missing)}): {_describe(missing)}")
            if unexpected:
                parts.append(f"  unexpected ({len(unexpected)}): {_describe(unexpected)}")
            if wrong:
                parts.append(f"  wrong shape ({len(wrong)}): " + "; ".join(sorted(wrong)[:12])
                             + (f"; ... (+{len(wrong) - 12} more)" if len(wrong) > 12 else ""))
            raise WeightError("\n".join(parts))
        tensors: dict[str, torch.Tensor] = {}
        stored: dict[str, str] = {}
        for name, ws in expected.items():
            if name not in files or name in unused:
                continue
            tensor = handle_of(files[name]).get_tensor(name)
            stored[name] = str(tensor.dtype).replace("torch.", "")
            tensors[name] = place(tensor, ws.role, model.dtype, model.device)
    finally:
        for handle in handles.values():
            handle.__exit__(None, None, None)
    count = len(tensors)
    model.bind(tensors, consume=True)      # (each part's source tensors are dropped as it binds them)
    return {"tensors": count, "stored_dtypes": sorted(set(stored.values())), "ignored": ignored,
            "not_read": sorted(unused & set(files))}


def place(tensor: torch.Tensor, role: str, compute_dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    """Apply the storage rule to one tensor and move it to the device."""
    if role == "int_table" or not tensor.is_floating_point():
        return tensor.to(torch.int32).contiguous().to(device)
    if role == "vector" or compute_dtype == torch.float32:
        return tensor.to(torch.float32).contiguous().to(device)
    if tensor.dtype in (torch.bfloat16, torch.float32):
        return tensor.contiguous().to(device)
    return tensor.to(torch.bfloat16).contiguous().to(device)
