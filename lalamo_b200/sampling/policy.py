"""Generation and sampling options, with the reference's names and meanings.

``GenerationConfig`` mirrors ``lalamo/models/language_model.py:73-116`` and ``SamplingPolicy``
mirrors ``lalamo/sampling.py:20-92``: an option that is ``None`` or at its neutral value is off;
``temperature == 0`` means greedy; the processors run in the order ban, repetition, presence,
frequency, temperature, top-k, top-p, min-p (``lalamo/sampling.py:187-196``).
"""

from __future__ import annotations

from dataclasses import dataclass, fields, replace
from typing import Iterable

__all__ = ["GenerationConfig", "MAX_BANNED_TOKENS", "SamplingPolicy"]

MAX_BANNED_TOKENS = 16  # lalamo/sampling.py:15


@dataclass(frozen=True)
class SamplingPolicy:
    temperature: float | None = None
    top_k: int | None = None
    top_p: float | None = None
    min_p: float | None = None
    banned_tokens: tuple[int, ...] = ()
    repetition_penalty: float | None = None
    presence_penalty: float | None = None
    frequency_penalty: float | None = None
    suffix_repetition_length: int | None = None

    @classmethod
    def init(
        cls,
        temperature: float | None = None,
        top_k: int | None = None,
        top_p: float | None = None,
        min_p: float | None = None,
        banned_tokens: Iterable[int] | None = None,
        repetition_penalty: float | None = None,
        presence_penalty: float | None = None,
        frequency_penalty: float | None = None,
        suffix_repetition_length: int | None = None,
    ) -> "SamplingPolicy":
        """Normalises the options as ``SamplingPolicy.init`` does (``lalamo/sampling.py:32-73``)."""
        banned = () if banned_tokens is None else tuple(int(token) for token in banned_tokens)
        if len(banned) > MAX_BANNED_TOKENS:
            raise ValueError(f"At most {MAX_BANNED_TOKENS} banned tokens are supported.")
        if any(token < 0 for token in banned):
            raise ValueError("Banned tokens must be non-negative token ids.")
        if repetition_penalty is not None and repetition_penalty <= 0.0:
            raise ValueError("repetition_penalty must be positive.")
        if temperature is not None and temperature < 0.0:
            raise ValueError("temperature must not be negative.")
        return cls(
            temperature=None if temperature is None or temperature == 1.0 else float(temperature),
            top_k=None if top_k is None or top_k <= 0 else int(top_k),
            top_p=None if top_p is None or top_p >= 1.0 else float(top_p),
            min_p=None if min_p is None or min_p <= 0.0 else float(min_p),
            banned_tokens=banned,
            repetition_penalty=None if repetition_penalty is None or repetition_penalty == 1.0 else float(repetition_penalty),
            presence_penalty=None if presence_penalty is None or presence_penalty == 0.0 else float(presence_penalty),
            frequency_penalty=None if frequency_penalty is None or frequency_penalty == 0.0 else float(frequency_penalty),
            suffix_repetition_length=None if suffix_repetition_length is None or suffix_repetition_length <= 0 else int(suffix_repetition_length),
        )

    @property
    def is_greedy(self) -> bool:
        return self.temperature == 0.0

    @property
    def has_count_penalties(self) -> bool:
        return self.repetition_penalty is not None or self.presence_penalty is not None or self.frequency_penalty is not None

    @property
    def is_plain_greedy(self) -> bool:
        """Greedy with nothing that changes the arg-max: the arg-max kernel alone will do."""
        return self.is_greedy and not self.banned_tokens and not self.has_count_penalties


@dataclass(frozen=True)
class GenerationConfig:
    stop_token_ids: tuple[int, ...] = ()
    temperature: float | None = None
    top_k: int | None = None
    top_p: float | None = None
    min_p: float | None = None
    banned_tokens: tuple[int, ...] | None = None
    repetition_penalty: float | None = None
    presence_penalty: float | None = None
    frequency_penalty: float | None = None
    suffix_repetition_length: int | None = None

    def override_with(self, other: "GenerationConfig") -> "GenerationConfig":
        """Fields of ``other`` that differ from the defaults win; stop and banned tokens are
        merged (``lalamo/models/language_model.py:85-102``)."""
        default = GenerationConfig()
        merged = {"stop_token_ids", "banned_tokens"}
        overrides = {}
        for item in fields(GenerationConfig):
            ours, theirs, neutral = getattr(self, item.name), getattr(other, item.name), getattr(default, item.name)
            if theirs == neutral:
                continue
            if item.name in merged and ours != neutral:
                overrides[item.name] = tuple(sorted({*ours, *theirs}))
            else:
                overrides[item.name] = theirs
        return replace(self, **overrides)

    def default_policy(self) -> SamplingPolicy:
        return SamplingPolicy.init(
            temperature=self.temperature,
            top_k=self.top_k,
            top_p=self.top_p,
            min_p=self.min_p,
            banned_tokens=self.banned_tokens,
            repetition_penalty=self.repetition_penalty,
            presence_penalty=self.presence_penalty,
            frequency_penalty=self.frequency_penalty,
            suffix_repetition_length=self.suffix_repetition_length,
        )
