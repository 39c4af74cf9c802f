"""Request and result types of the Python entry point.

The classes, their field names, order and defaults are the public request /
result schema of the reference (src/torchinferno/engine/types.py:10-77), kept so
that code written against it runs here: ``SamplingConfig(max_tokens, temperature,
stop_token_ids)``, ``GenerateRequest`` with one prompt source, ``TokenOutput`` per
streamed token, ``GenerateOutput`` with ``finish_reason`` in {"length", "stop",
"cancelled"} and ``Usage``.  ``seed`` is added for the seeded sampler.  The
checks below are this engine's own.
"""
from __future__ import annotations

from collections.abc import Mapping, Sequence
from dataclasses import dataclass, field

ChatMessage = Mapping[str, object]


def _token_tuple(ids, what: str) -> tuple[int, ...]:
    """Token ids as a tuple of plain ints; refuses what is no integer or is negative."""
    out = []
    for t in ids:
        if isinstance(t, bool) or int(t) != t or int(t) < 0:
            raise ValueError(f"{what}: {t!r} is not a token id")
        out.append(int(t))
    return tuple(out)


@dataclass(frozen=True)
class SamplingConfig:
    max_tokens: int = 256
    temperature: float = 0.0
    stop_token_ids: tuple[int, ...] = ()
    seed: int = 0

    def __post_init__(self) -> None:
        for name in ("max_tokens", "temperature"):
            if getattr(self, name) < 0:
                raise ValueError(f"SamplingConfig.{name} = {getattr(self, name)!r}: a negative value has no meaning")
        object.__setattr__(self, "stop_token_ids", _token_tuple(self.stop_token_ids, "stop_token_ids"))


@dataclass(frozen=True)
class GenerateRequest:
    request_id: str
    prompt: str | None = None
    messages: Sequence[ChatMessage] = ()
    prompt_token_ids: Sequence[int] | None = None
    sampling: SamplingConfig = field(default_factory=SamplingConfig)
    stream: bool = False

    def _prompt_sources(self) -> list[str]:
        """Names of the prompt fields that were given."""
        given = {"prompt": self.prompt is not None, "messages": len(self.messages) > 0,
                 "prompt_token_ids": self.prompt_token_ids is not None}
        return [name for name, present in given.items() if present]

    def __post_init__(self) -> None:
        if self.request_id in ("", None):
            raise ValueError("a request needs a request_id (it names the request in results and in cancel())")
        sources = self._prompt_sources()
        if len(sources) != 1:
            raise ValueError("a request takes its prompt from one of prompt, messages and prompt_token_ids; "
                             f"given: {', '.join(sources) or 'none'}")
        object.__setattr__(self, "messages", tuple({**m} for m in self.messages))
        if sources == ["prompt_token_ids"]:
            object.__setattr__(self, "prompt_token_ids", _token_tuple(self.prompt_token_ids, "prompt_token_ids"))


@dataclass(frozen=True)
class Usage:
    prompt_tokens: int
    completion_tokens: int

    @property
    def total_tokens(self) -> int:
        return self.prompt_tokens + self.completion_tokens


@dataclass(frozen=True)
class TokenOutput:
    request_id: str
    token_id: int | None
    text: str
    index: int
    finished: bool = False
    finish_reason: str | None = None
    usage: Usage | None = None


@dataclass(frozen=True)
class GenerateOutput:
    request_id: str
    token_ids: tuple[int, ...]
    text: str
    finish_reason: str
    usage: Usage
