"""From a model folder to a model, a cache and a step function."""
from __future__ import annotations

from pathlib import Path
from typing import Any, Mapping

import torch

from torchinferno_b200.cache.manager import CacheManager
from torchinferno_b200.config.model_config import read_config_json
from torchinferno_b200.engine.runner import ModelRunner
from torchinferno_b200.weights.loader import load_weights
from torchinferno_b200.weights.random_init import build_model, init_random_weights


def parse_dtype(name: str | torch.dtype | None, config: Mapping[str, Any] | None = None) -> torch.dtype:
    """Names as the reference takes them (src/torchinferno/models/llama3/pipeline.py:508-521);
    only bfloat16 and float32 have kernels here."""
    if isinstance(name, torch.dtype):
        dtype = name
    else:
        text = str(name or "auto").lower().replace("torch.", "")
        if text == "auto":
            text = str((config or {}).get("torch_dtype", "bfloat16")).lower().replace("torch.", "")
        table = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32,
                 "fp16": torch.float16, "float16": torch.float16, "half": torch.float16}
        if text not in table:
            raise ValueError(f"unsupported dtype: {name}")
        dtype = table[text]
    if dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"dtype {dtype} has no kernels in this engine (bfloat16 or float32)")
    return dtype


def require_cuda(device: str | torch.device = "cuda:0") -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("this engine runs on a CUDA device only (sm_100a kernels; there is no CPU path)")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise RuntimeError(f"the kernels are built for sm_100a; device {device} is sm_{major}{minor}")
    return device


def load_model(folder: str | Path, *, dtype: str | torch.dtype = "auto", device: str | torch.device = "cuda:0"):
    """Build the model ``config.json`` names and bind the folder's weights."""
    config = read_config_json(folder)
    device = require_cuda(device)
    model = build_model(config, dtype=parse_dtype(dtype, config), device=device)
    load_weights(model, folder)
    return model


def random_model(config: Mapping[str, Any], seed: int, *, dtype: str | torch.dtype = "bfloat16",
                 device: str | torch.device = "cuda:0"):
    """Build the model ``config`` names with seeded random weights made on the device."""
    device = require_cuda(device)
    model = build_model(config, dtype=parse_dtype(dtype, config), device=device)
    init_random_weights(model, seed)
    return model


def make_runner(model, *, page_size: int = 16, max_tokens: int | None = None, num_pages: int | None = None,
                max_requests: int = 64, max_request_tokens: int | None = None,
                check_errors: bool = True) -> ModelRunner:
    """A cache sized for ``max_tokens`` tokens (or ``num_pages`` pages) and the step function over it."""
    if num_pages is None:
        if max_tokens is None:
            raise ValueError("give max_tokens or num_pages")
        num_pages = -(-max_tokens // page_size)
    limit = model.spec.max_positions if max_request_tokens is None else min(max_request_tokens, model.spec.max_positions)
    limit = min(limit, num_pages * page_size)
    cache = CacheManager(model.cache_requirements(), model.state_requirements(), page_size=page_size,
                         num_pages=num_pages, max_requests=max_requests, max_request_tokens=limit,
                         dtype=model.dtype, device=model.device)
    return ModelRunner(model, cache, check_errors=check_errors)
