"""Typed model configuration read from a checkpoint's ``config.json``.

The reference keeps one dataclass per family with ``from_dict`` that maps
aliases and drops unknown keys (src/torchinferno/models/llama3/config.py:6-53).
This module keeps that shape, but no size has a default here: every size and
constant comes from ``config.json`` and a missing key is an error that names
all missing keys at once.  Keys the reference ignores silently but which would
change the arithmetic (``hidden_act``, ``attention_bias``, ``mlp_bias``, an
unknown ``rope_type``) are rejected instead.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping


class ConfigError(ValueError):
    """A ``config.json`` that cannot describe a model this engine runs."""


@dataclass(frozen=True)
class RopeScaling:
    """The ``rope_scaling`` block.  ``rope_type`` selects the scaling law.

    llama3 law: src/torchinferno/models/llama3/pipeline.py:537-552.  The four
    numbers have no defaults there (``float(scaling[...])``) nor here.
    """

    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @classmethod
    def from_dict(cls, data: Mapping[str, Any] | None) -> "RopeScaling | None":
        if data is None:
            return None
        if not isinstance(data, Mapping):
            raise ConfigError(f"rope_scaling must be an object or null, got {type(data).__name__}")
        kind = data.get("rope_type", data.get("type"))
        if kind is None:
            raise ConfigError("rope_scaling has neither 'rope_type' nor 'type'")
        kind = str(kind)
        if kind == "default":
            return None
        if kind != "llama3":
            raise ConfigError(
                f"rope_scaling.rope_type={kind!r} is not supported (supported: 'llama3', 'default')"
            )
        needed = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
        missing = [key for key in needed if key not in data]
        if missing:
            raise ConfigError(f"rope_scaling (llama3) lacks keys: {missing}")
        scaling = cls(
            rope_type=kind,
            factor=float(data["factor"]),
            low_freq_factor=float(data["low_freq_factor"]),
            high_freq_factor=float(data["high_freq_factor"]),
            original_max_position_embeddings=int(data["original_max_position_embeddings"]),
        )
        if scaling.factor <= 0:
            raise ConfigError("rope_scaling.factor must be positive")
        if scaling.high_freq_factor == scaling.low_freq_factor:
            raise ConfigError("rope_scaling.high_freq_factor must differ from low_freq_factor")
        if scaling.original_max_position_embeddings <= 0:
            raise ConfigError("rope_scaling.original_max_position_embeddings must be positive")
        return scaling

    def to_dict(self) -> dict[str, Any]:
        return {
            "rope_type": self.rope_type,
            "factor": self.factor,
            "low_freq_factor": self.low_freq_factor,
            "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


# Alias → canonical key, as the reference accepts them
# (src/torchinferno/models/llama3/config.py:40-47).
_ALIASES = {
    "num_layers": "num_hidden_layers",
    "n_layers": "num_hidden_layers",
    "num_heads": "num_attention_heads",
    "n_heads": "num_attention_heads",
    "num_kv_heads": "num_key_value_heads",
    "max_seq_len": "max_position_embeddings",
}

_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "num_key_value_heads",
    "max_position_embeddings",
    "rope_theta",
    "rms_norm_eps",
)


@dataclass(frozen=True)
class LlamaConfig:
    """Llama 3 sizes and constants (keys: src/torchinferno/models/llama3/config.py:8-18).

    ``head_dim`` is a derived property in the reference (config.py:28-30); here
    it is also accepted as an explicit key, defaulting to
    ``hidden_size // num_attention_heads``.
    """

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    rope_scaling: RopeScaling | None = None
    tie_word_embeddings: bool = False
    torch_dtype: str = "bfloat16"
    architectures: tuple[str, ...] = ("LlamaForCausalLM",)
    model_type: str = "llama"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def __post_init__(self) -> None:
        positive = (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
            "max_position_embeddings",
        )
        for name in positive:
            value = getattr(self, name)
            if not isinstance(value, int) or isinstance(value, bool) or value < 1:
                raise ConfigError(f"{name} must be a positive integer, got {value!r}")
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                "num_attention_heads must be divisible by num_key_value_heads "
                f"({self.num_attention_heads} vs {self.num_key_value_heads})"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError("head_dim must be even for rotary position encoding")
        if not (self.rope_theta > 0):
            raise ConfigError("rope_theta must be positive")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("rms_norm_eps must be positive")

    # -- construction ---------------------------------------------------
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "LlamaConfig":
        normalized = dict(data)
        for source, target in _ALIASES.items():
            if source in normalized and target not in normalized:
                normalized[target] = normalized[source]
        missing = [key for key in _REQUIRED if key not in normalized]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        act = normalized.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act={act!r} is not supported (the feed-forward is SwiGLU: 'silu')")
        for flag in ("attention_bias", "mlp_bias"):
            if normalized.get(flag, False):
                raise ConfigError(f"{flag}=true is not supported (projections have no bias)")
        hidden = _as_int(normalized, "hidden_size")
        heads = _as_int(normalized, "num_attention_heads")
        if "head_dim" in normalized and normalized["head_dim"] is not None:
            head_dim = _as_int(normalized, "head_dim")
        else:
            if heads < 1 or hidden % heads != 0:
                raise ConfigError(
                    "hidden_size must be divisible by num_attention_heads when head_dim is not given"
                )
            head_dim = hidden // heads
        known = set(_REQUIRED) | {
            "head_dim", "rope_scaling", "tie_word_embeddings", "torch_dtype",
            "architectures", "model_type", "hidden_act", "attention_bias", "mlp_bias",
        } | set(_ALIASES)
        return cls(
            vocab_size=_as_int(normalized, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_as_int(normalized, "intermediate_size"),
            num_hidden_layers=_as_int(normalized, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=_as_int(normalized, "num_key_value_heads"),
            head_dim=head_dim,
            max_position_embeddings=_as_int(normalized, "max_position_embeddings"),
            rope_theta=float(normalized["rope_theta"]),
            rms_norm_eps=float(normalized["rms_norm_eps"]),
            rope_scaling=RopeScaling.from_dict(normalized.get("rope_scaling")),
            tie_word_embeddings=bool(normalized.get("tie_word_embeddings", False)),
            torch_dtype=str(normalized.get("torch_dtype", normalized.get("dtype", "bfloat16"))),
            architectures=tuple(str(a) for a in (normalized.get("architectures") or ("LlamaForCausalLM",))),
            model_type=str(normalized.get("model_type", "llama")),
            extra={k: v for k, v in normalized.items() if k not in known},
        )

    @classmethod
    def from_json_file(cls, path: str | Path) -> "LlamaConfig":
        return cls.from_dict(read_config_json(path))

    def to_dict(self) -> dict[str, Any]:
        return {
            "architectures": list(self.architectures),
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "rope_theta": self.rope_theta,
            "rope_scaling": None if self.rope_scaling is None else self.rope_scaling.to_dict(),
            "rms_norm_eps": self.rms_norm_eps,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": self.torch_dtype,
        }

    @property
    def group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def parameter_count(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        q = self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        per_layer = h * q + 2 * h * kv + q * h + 3 * h * i + 2 * h
        total = self.num_hidden_layers * per_layer + v * h + h
        if not self.tie_word_embeddings:
            total += v * h
        return total


def _as_int(data: Mapping[str, Any], key: str) -> int:
    value = data[key]
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
        raise ConfigError(f"{key} must be an integer, got {value!r}")
    return int(value)


def read_config_json(path: str | Path) -> dict[str, Any]:
    """Read ``config.json`` from a model folder (or the file itself)."""
    path = Path(path)
    if path.is_dir():
        path = path / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json at {path}")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as exc:
        raise ConfigError(f"{path} is not valid JSON: {exc}") from exc
    if not isinstance(data, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return data
