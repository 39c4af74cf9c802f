"""The plain implementation against numbers taken from the reference project's own model code.

``tests/golden/llama_tiny.json`` was written by ``tests/golden/make_golden.py``, which ran the
reference's ``Llama3PipelineForCausalLM`` (float32, CPU) on tiny seeded models.
"""
import json
from pathlib import Path

import pytest
import torch

import plain_llama
from golden.make_golden import golden_tokens, golden_weights

GOLDEN = json.loads((Path(__file__).parent / "golden" / "llama_tiny.json").read_text())


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_plain_matches_reference_logits(name):
    case = GOLDEN[name]
    weights = {k: v.double() for k, v in golden_weights(case["config"], case["seed"]).items()}
    assert golden_tokens(case["config"], case["seed"], 90) == case["tokens"]
    logits = plain_llama.forward(case["config"], weights, case["tokens"])
    want = torch.tensor(case["last_logits"], dtype=torch.float64)
    assert torch.allclose(logits[-4:], want, atol=2e-5, rtol=1e-4), (logits[-4:] - want).abs().max()


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_plain_matches_reference_greedy(name):
    case = GOLDEN[name]
    weights = {k: v.double() for k, v in golden_weights(case["config"], case["seed"]).items()}
    prompt = case["tokens"][: case["greedy_prompt_len"]]
    assert plain_llama.generate_greedy(case["config"], weights, prompt, 6) == case["greedy_tokens"]


def test_llama3_scaling_has_three_bands():
    case = GOLDEN["llama3_rope"]["config"]
    scaled = plain_llama.inverse_frequencies(case)
    plain = plain_llama.inverse_frequencies({**case, "rope_scaling": None})
    ratio = (plain / scaled)
    assert torch.isclose(ratio.max(), torch.tensor(8.0)) and torch.isclose(ratio.min(), torch.tensor(1.0))
    assert ((ratio > 1.001) & (ratio < 7.999)).any()  # the smoothed middle band is exercised


def test_causal_attention_window_and_groups():
    torch.manual_seed(0)
    q, k, v = torch.randn(4, 9, 8, dtype=torch.float64), torch.randn(2, 9, 8, dtype=torch.float64), torch.randn(2, 9, 8, dtype=torch.float64)
    full = plain_llama.causal_attention(q, k, v, 2)
    # position 0 sees only key 0
    assert torch.allclose(full[:, 0], v.repeat_interleave(2, 0)[:, 0])
    windowed = plain_llama.causal_attention(q, k, v, 2, window=3)
    assert torch.allclose(windowed[:, :3], full[:, :3]) and not torch.allclose(windowed[:, 5], full[:, 5])


def test_gumbel_scores_are_seeded_and_uniform():
    import numpy as np
    logits = np.zeros(4096)
    a = plain_llama.gumbel_scores(logits, 1.0, seed=7, position=3)
    b = plain_llama.gumbel_scores(logits, 1.0, seed=7, position=3)
    c = plain_llama.gumbel_scores(logits, 1.0, seed=7, position=4)
    assert (a == b).all() and (a != c).any()
    u = np.exp(-np.exp(-a))            # back to the uniforms
    assert 0.45 < u.mean() < 0.55 and u.min() > 0 and u.max() < 1
