"""Shared by the GPU tests: tolerances (set once), plain-reference logits, request sets."""
from __future__ import annotations


import numpy as np
import pytest
import torch

import plain_llama

# The 32-bit path against the float64 plain implementation.
F32_ATOL, F32_RTOL = 2e-5, 1e-4
# bfloat16 against the same: largest error relative to the largest logit of the sequence
# (the measure of scripts/cmp_paged_dense_logits.py in the reference project, which expects
# about 1 % in bf16 on a deep model).  Seen on the B200 with the tiny configurations: at most 0.0064 (twice
# that is the bound); at the 8B layer sizes (two layers, width 4096, vocabulary 128256: the largest of far
# more logits, each summed over far more terms): 0.0133 to 0.0143 for short prompts and for a 2,048-token
# prompt followed by 64 decoded tokens alike, moving by a few per cent of itself with the kernels the measured
# choice picks on a box (they sum in different orders); the bound there is 1.4 times the worst seen.
BF16_REL = 0.0125
BF16_REL_LARGE = 0.02


# The largest error a test saw, as a share of its bound (printed at the end of the run, so that it shows how much
# room a tolerance leaves).
WORST: dict[str, float] = {}


def note_worst(what: str, share: float) -> None:
    WORST[what] = max(WORST.get(what, 0.0), float(share))


def need_gpu():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")


def requests_for(config, seed, lengths):
    g = torch.Generator().manual_seed(1234 + seed)
    return {f"r{i}": torch.randint(0, config["vocab_size"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


_plain_cache: dict = {}


def plain_logits(folder, tokens):
    key = (str(folder), tuple(tokens))
    if key not in _plain_cache:
        if str(folder) not in _plain_cache:
            _plain_cache[str(folder)] = plain_llama.read_model_folder(folder)
        config, weights = _plain_cache[str(folder)]
        _plain_cache[key] = plain_llama.forward(config, weights, tokens).numpy()
    return _plain_cache[key]


def check_rows(rows, folder, requests, dtype, what: str | None = None):
    """Every (request, position) row against the plain implementation.  Returns, and notes under ``what`` (by
    default the running test's name), the largest error as a share of its bound."""
    import os
    assert rows, "nothing was compared"
    what = what or os.environ.get("PYTEST_CURRENT_TEST", "?").split("::")[-1].split(" (")[0]
    worst = 0.0
    for (name, pos), got_list in rows.items():
        ref = plain_logits(folder, requests[name])
        for got in got_list:
            got = np.asarray(got, dtype=np.float64)
            assert np.isfinite(got).all(), f"{name}@{pos}: non-finite logits"
            err = np.abs(got - ref[pos]).max()
            if dtype == "float32":
                bound = F32_ATOL + F32_RTOL * np.abs(ref[pos]).max()
            else:
                bound = BF16_REL * np.abs(ref).max()
            worst = max(worst, err / bound)
            assert err <= bound, f"{name}@{pos} ({dtype}): max error {err:.3e} exceeds {bound:.3e}"
    note_worst(f"{what} [{dtype}]", worst)
    return worst
