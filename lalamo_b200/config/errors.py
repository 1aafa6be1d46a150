"""Errors of the configuration layer."""

from __future__ import annotations

__all__ = ["ConfigError", "UnknownArchitectureError"]


class ConfigError(ValueError):
    """A key of ``config.json`` is missing, of the wrong type or contradicts another key."""

    def __init__(self, key: str, why: str) -> None:
        super().__init__(f"config.json: {key!r} {why}")
        self.key = key
        self.why = why


class UnknownArchitectureError(ValueError):
    def __init__(self, name: str, known: list[str]) -> None:
        super().__init__(f"no model is registered for architecture {name!r}; registered: {sorted(known)}")
        self.name = name
