"""One registry from an architecture's name to its configuration class and model builder.

The reference resolves a checkpoint's family from ``model_type`` and
``architectures`` and raises when the two disagree
(src/torchinferno/models/identity.py:7-58).  The same rule is kept: names are
case-folded, a recognised ``model_type`` and a recognised architecture must
point at the same entry.

An architecture is registered with

    register_architecture(ArchitectureEntry(
        name="LlamaForCausalLM", model_types=("llama", "llama3"),
        config_class=LlamaConfig, build=build_llama))

``config_class.from_dict(config_json)`` returns the typed configuration and
``build(config)`` returns a :class:`torchinferno_b200.models.spec.ModelSpec`
(a description made of parts; no tensors).  Nothing else in the engine knows
architecture names.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_class: Any
    build: Callable[[Any], Any]
    model_types: tuple[str, ...] = ()
    aliases: tuple[str, ...] = ()


_BY_ARCHITECTURE: dict[str, ArchitectureEntry] = {}
_BY_MODEL_TYPE: dict[str, ArchitectureEntry] = {}


def register_architecture(entry: ArchitectureEntry, *, replace: bool = False) -> ArchitectureEntry:
    names = [entry.name, *entry.aliases]
    for name in names:
        key = name.strip().lower()
        if not replace and key in _BY_ARCHITECTURE and _BY_ARCHITECTURE[key] is not entry:
            raise ValueError(f"architecture {name!r} is already registered")
    for model_type in entry.model_types:
        key = model_type.strip().lower()
        if not replace and key in _BY_MODEL_TYPE and _BY_MODEL_TYPE[key] is not entry:
            raise ValueError(f"model_type {model_type!r} is already registered")
    for name in names:
        _BY_ARCHITECTURE[name.strip().lower()] = entry
    for model_type in entry.model_types:
        _BY_MODEL_TYPE[model_type.strip().lower()] = entry
    return entry


def unregister_architecture(name: str) -> None:
    entry = _BY_ARCHITECTURE.get(name.strip().lower())
    if entry is None:
        return
    for table in (_BY_ARCHITECTURE, _BY_MODEL_TYPE):
        for key in [k for k, v in table.items() if v is entry]:
            del table[key]


def registered_architectures() -> tuple[str, ...]:
    return tuple(sorted({entry.name for entry in _BY_ARCHITECTURE.values()}))


def entry_for_kind(kind: str) -> ArchitectureEntry | None:
    """The entry a user's ``model_kind`` names (an architecture name, an alias or a ``model_type``), or None."""
    _ensure_builtin()
    key = str(kind).strip().lower()
    return _BY_ARCHITECTURE.get(key) or _BY_MODEL_TYPE.get(key)


def known_kinds() -> tuple[str, ...]:
    _ensure_builtin()
    return tuple(sorted(set(_BY_ARCHITECTURE) | set(_BY_MODEL_TYPE)))


def resolve_architecture(config: Mapping[str, Any]) -> ArchitectureEntry:
    """Pick the registered entry that ``config.json`` names, or raise."""
    _ensure_builtin()
    model_type = str(config.get("model_type", "") or "").strip().lower()
    by_type = _BY_MODEL_TYPE.get(model_type)
    architectures = [str(value) for value in (config.get("architectures") or ())]
    by_arch = {
        _BY_ARCHITECTURE[key].name: _BY_ARCHITECTURE[key]
        for value in architectures
        if (key := value.strip().lower()) in _BY_ARCHITECTURE
    }
    if len(by_arch) > 1:
        raise ValueError(f"conflicting model architectures: {sorted(by_arch)}")
    arch_entry = next(iter(by_arch.values()), None)
    if by_type is not None and arch_entry is not None and by_type is not arch_entry:
        raise ValueError(
            "conflicting model identity: "
            f"model_type={model_type!r} names {by_type.name}, architectures name {arch_entry.name}"
        )
    entry = arch_entry or by_type
    if entry is None:
        raise ValueError(
            f"unsupported model identity: model_type={model_type!r}, architectures={architectures}; "
            f"registered: {list(registered_architectures())}"
        )
    return entry


_BUILTIN_LOADED = False


def _ensure_builtin() -> None:
    """Import the package's own architectures once (they register themselves)."""
    global _BUILTIN_LOADED
    if _BUILTIN_LOADED:
        return
    _BUILTIN_LOADED = True
    from torchinferno_b200.models import llama  # noqa: F401
