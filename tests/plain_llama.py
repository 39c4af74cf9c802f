"""A plain, slow Llama 3 forward pass for the tests: whole sequences, no cache.

It rests on the formulas of the reference project, one function per part, each
citing where the formula stands there (paths within bobrenjc93/TorchInferno).
It shares no code with ``torchinferno_b200``: it reads config.json and
model.safetensors itself, and computes on the CPU in float64 by default so that
its own rounding does not count against the engine.  ``tests/golden/`` holds a
comparison of this file with the reference's own model code on a tiny random
model (made by ``tests/golden/make_golden.py``).
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch


# ------------------------------------------------------------------ loading
def read_model_folder(folder, dtype=torch.float64):
    """config.json as a dict and every tensor of model.safetensors, widened to ``dtype``."""
    from safetensors import safe_open
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            weights[name] = handle.get_tensor(name).to(dtype)
    return config, weights


# -------------------------------------------------------------------- parts
def rms_norm(x, weight, eps):
    """y = x * rsqrt(mean(x^2) + eps) * w  (src/torchinferno/models/llama3/raw_ops.py:9-11)."""
    variance = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(variance + eps) * weight


def inverse_frequencies(config):
    """theta^(-2i/d) and the llama3 scaling law (src/torchinferno/models/llama3/pipeline.py:532-552).

    Computed in float32 as there, because the table is an fp32 constant of the model.
    """
    heads = config["num_attention_heads"]
    d = config.get("head_dim") or config["hidden_size"] // heads
    theta = float(config["rope_theta"])
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    scaling = config.get("rope_scaling") or {}
    if scaling.get("rope_type", scaling.get("type")) != "llama3":
        return inv_freq
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    old_len = float(scaling["original_max_position_embeddings"])
    low_wavelen = old_len / low
    high_wavelen = old_len / high
    wavelen = 2 * math.pi / inv_freq
    inv_llama = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (old_len / wavelen - low) / (high - low)
    smoothed = (1 - smooth) * inv_llama / factor + smooth * inv_llama
    medium = ~(wavelen < high_wavelen) & ~(wavelen > low_wavelen)
    return torch.where(medium, smoothed, inv_llama)


def rotary(x, positions, inv_freq):
    """Rotate-half RoPE on x [heads, T, d] (src/torchinferno/models/llama3/pipeline.py:555-568).

    The angle is the fp32 product position * inv_freq, as there; cos and sin are then
    taken in the working precision.
    """
    angles = torch.outer(positions.to(torch.float32), inv_freq.to(torch.float32)).to(x.dtype)
    emb = torch.cat((angles, angles), dim=-1)
    cos, sin = emb.cos()[None], emb.sin()[None]
    half = x.shape[-1] // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return x * cos + rotated * sin


def causal_attention(q, k, v, group, window=None, rows=None):
    """softmax(q k^T / sqrt(d) + causal mask) v with grouped heads.

    q [h, T, d], k, v [kv, T, d]; query head j reads kv head j // group
    (src/torchinferno/models/llama3/raw_ops.py:38-51).  ``rows`` (positions): q holds only the queries at
    these positions of the sequence, [h, len(rows), d]; the keys are still all T (long sequences of which
    a few rows are compared).
    """
    k = k.repeat_interleave(group, dim=0)
    v = v.repeat_interleave(group, dim=0)
    T = k.shape[1]
    scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(q.shape[-1])
    pos = torch.arange(T)
    at = pos if rows is None else torch.as_tensor(rows, dtype=torch.long)
    allowed = pos[None, :] <= at[:, None]
    if window:
        allowed &= (at[:, None] - pos[None, :]) < window
    scores = scores.masked_fill(~allowed[None], float("-inf"))
    return torch.matmul(torch.softmax(scores, dim=-1), v)


def swiglu_mlp(x, gate_w, up_w, down_w):
    """down(silu(gate(x)) * up(x))  (src/torchinferno/models/llama3/pipeline.py:247-250)."""
    gate = x @ gate_w.T
    return ((gate / (1 + torch.exp(-gate))) * (x @ up_w.T)) @ down_w.T


def decoder_layer(x, positions, config, weights, prefix, inv_freq):
    """One pre-norm layer (src/torchinferno/models/llama3/pipeline.py:190-245)."""
    heads, kv = config["num_attention_heads"], config["num_key_value_heads"]
    d = config.get("head_dim") or config["hidden_size"] // heads
    eps = config["rms_norm_eps"]
    T = x.shape[0]
    n = rms_norm(x, weights[prefix + "input_layernorm.weight"], eps)
    q = (n @ weights[prefix + "self_attn.q_proj.weight"].T).view(T, heads, d).transpose(0, 1)
    k = (n @ weights[prefix + "self_attn.k_proj.weight"].T).view(T, kv, d).transpose(0, 1)
    v = (n @ weights[prefix + "self_attn.v_proj.weight"].T).view(T, kv, d).transpose(0, 1)
    q, k = rotary(q, positions, inv_freq), rotary(k, positions, inv_freq)
    a = causal_attention(q, k, v, heads // kv).transpose(0, 1).reshape(T, heads * d)
    x = x + a @ weights[prefix + "self_attn.o_proj.weight"].T
    n = rms_norm(x, weights[prefix + "post_attention_layernorm.weight"], eps)
    return x + swiglu_mlp(n, weights[prefix + "mlp.gate_proj.weight"], weights[prefix + "mlp.up_proj.weight"],
                          weights[prefix + "mlp.down_proj.weight"])


def forward(config, weights, token_ids, rows=None):
    """Logits [T, vocab] of one whole sequence (src/torchinferno/models/llama3/pipeline.py:371-401);
    with ``rows`` only those positions are projected to the vocabulary: [len(rows), vocab]."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    x = weights["model.embed_tokens.weight"][ids]
    positions = torch.arange(len(ids))
    inv_freq = inverse_frequencies(config)
    for layer in range(config["num_hidden_layers"]):
        x = decoder_layer(x, positions, config, weights, f"model.layers.{layer}.", inv_freq)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    x = rms_norm(x, weights["model.norm.weight"], config["rms_norm_eps"])
    head = weights["model.embed_tokens.weight"] if config.get("tie_word_embeddings") or \
        "lm_head.weight" not in weights else weights["lm_head.weight"]
    return x @ head.T


# ----------------------------------------------------------------- sampling
def greedy(logits):
    """argmax, first index among equals (src/torchinferno/runtime/sampling.py:8-9)."""
    return int(torch.argmax(torch.as_tensor(logits), dim=-1))


def generate_greedy(config, weights, prompt, new_tokens):
    """Re-run the whole prefix for each token (src/torchinferno/models/llama3/model.py:110-127)."""
    ids = list(prompt)
    for _ in range(new_tokens):
        ids.append(greedy(forward(config, weights, ids)[-1]))
    return ids[len(prompt):]


def philox4x32(counter, key, rounds=10):
    """Philox4x32-10 on numpy uint32 arrays: counter [..., 4], key [2]."""
    c = [np.asarray(counter[..., i], dtype=np.uint64) for i in range(4)]
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(rounds):
        p0 = np.uint64(0xD2511F53) * c[0]
        p1 = np.uint64(0xCD9E8D57) * c[2]
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c = [(hi1 ^ c[1] ^ k0) & mask, lo1, (hi0 ^ c[3] ^ k1) & mask, lo0]
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return np.stack(c, axis=-1).astype(np.uint32)


def gumbel_scores(logits, temperature, seed, position):
    """logits / T - log(-log u), u from Philox keyed by seed, counter (index / 4, position).

    The Gumbel-max form of temperature sampling
    (src/torchinferno/models/llama3/tensor_parallel.py:9946-9996); it draws from
    softmax(logits / T) (src/torchinferno/runtime/sampling.py:10-11).
    """
    logits = np.asarray(logits, dtype=np.float64)
    vocab = logits.shape[-1]
    index = np.arange(vocab, dtype=np.uint64)
    counter = np.zeros((vocab, 4), dtype=np.uint64)
    counter[:, 0] = index >> np.uint64(2)
    counter[:, 1] = np.uint64(position)
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    words = philox4x32(counter, (seed & 0xFFFFFFFF, seed >> 32))
    r = words[np.arange(vocab), (index & np.uint64(3)).astype(np.int64)]
    u = ((r >> np.uint32(8)).astype(np.float64) + 0.5) / 16777216.0
    return logits / temperature - np.log(-np.log(u))
