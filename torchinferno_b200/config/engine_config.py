"""Engine options.

Names and defaults the reference has are kept as they are
(src/torchinferno/engine/config.py:40-61): ``model``, ``model_kind="auto"``,
``tokenizer``, ``device``, ``dtype="auto"``, ``max_model_len``, ``page_size=16``,
``max_batch_size=64``, ``cache_backend`` (only "paged" exists here).  Options
for several GPUs, disaggregation and servers are not carried.  Added: the
per-step token budget, the prompt portion size, the size of the page pool and
the default sampling seed, ``async_scheduling``, and which kernels multiply
(``gemm_backend``, ``few_rows_choice``).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class EngineConfig:
    model: str                              # folder with config.json and model.safetensors
    model_kind: str = "auto"                # "auto": whatever config.json names
    tokenizer: str | None = None
    device: str | None = None               # default cuda:0
    dtype: str = "auto"                     # auto | bfloat16 | float32
    max_model_len: int | None = None        # most tokens one request may hold
    cache_backend: str = "paged"
    page_size: int = 16
    max_batch_size: int = 64                # most requests running at once
    max_num_batched_tokens: int = 8192      # token budget of one step
    prefill_chunk_size: int | None = 2048   # longest prompt portion in one step
    num_pages: int | None = None            # pages per cache group; default from kv_cache_tokens
    kv_cache_tokens: int | None = None      # pool size in tokens; default max_batch_size * max_model_len, capped by memory
    cache_memory_fraction: float = 0.9      # of the free device memory, the most the default pool may take
    seed: int = 0
    use_cuda_graphs: bool = True
    async_scheduling: bool = True           # launch the next decode step before the host has read this one's tokens
    gemm_backend: str = "auto"              # auto | tcgen05 | library (bf16 projections)
    few_rows_choice: str = "measured"       # under "auto", which kernel multiplies few rows (decode steps): measured
                                            # once per GPU model and shape and kept on disk | swapab | library

    profile_kernels: bool = False           # CUDA-event timers per kernel class around the layers' launches
                                            # (InferenceEngine.kernel_times()); steps then run uncaptured

    def __post_init__(self) -> None:
        if self.cache_backend != "paged":
            raise ValueError(f"cache_backend={self.cache_backend!r}: only 'paged' exists in this engine")
        if not 0.0 < self.cache_memory_fraction <= 1.0:
            raise ValueError("cache_memory_fraction must lie in (0, 1]")
        if self.page_size < 1 or self.max_batch_size < 1 or self.max_num_batched_tokens < 1:
            raise ValueError("page_size, max_batch_size and max_num_batched_tokens must be positive")
