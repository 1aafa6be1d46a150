"""The registry from an architecture's name to its configuration class.

The reference maps repositories to ``ModelSpec`` objects whose ``config_type`` builds the
model (``lalamo/model_registry.py:45-58``, ``lalamo/model_import/model_spec.py:45-66``).  Here the
key is the name in ``config.json``'s ``architectures`` list: the configuration class it maps to
turns the file into a :class:`~lalamo_b200.config.plan.ModelPlan` and names the checkpoint
tensors of every part.  A new architecture is one more ``register_architecture`` call.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping, Protocol

from .errors import ConfigError, UnknownArchitectureError
from .plan import ModelPlan

__all__ = ["ArchitectureConfig", "architectures", "config_from_dict", "load_config", "register_architecture"]


class ArchitectureConfig(Protocol):
    """What a registered configuration class must offer."""

    architecture: str

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ArchitectureConfig": ...

    def to_plan(self) -> ModelPlan: ...

    def checkpoint_names(self, path: tuple, local: str) -> list[str]: ...

    def to_json_dict(self) -> dict[str, Any]: ...


_ARCHITECTURES: dict[str, type] = {}


def register_architecture(name: str, config_type: type) -> None:
    _ARCHITECTURES[name] = config_type


def architectures() -> dict[str, type]:
    return dict(_ARCHITECTURES)


def config_from_dict(raw: Mapping[str, Any]) -> ArchitectureConfig:
    names = raw.get("architectures")
    if not isinstance(names, list) or not names or not isinstance(names[0], str):
        raise ConfigError("architectures", "must be a non-empty list of architecture names")
    config_type = _ARCHITECTURES.get(names[0])
    if config_type is None:
        raise UnknownArchitectureError(names[0], list(_ARCHITECTURES))
    return config_type.from_dict(raw)


def load_config(model_dir: str | Path) -> ArchitectureConfig:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"{path} does not exist")
    with open(path) as stream:
        return config_from_dict(json.load(stream))
