"""The random-weights mode: writes a model folder (``config.json`` + ``model.safetensors``)
from a configuration and a seed.

Each tensor is drawn from its own generator seeded by ``(seed, crc32(name))``, so a tensor's
values depend only on the seed, its checkpoint name and its shape.  Matrices and convolution
taps are ``N(0, std)``; norm scales are ``1 + N(0, std)``.  The reference's counterpart is
``RandomInitializer`` (``lalamo/initializer.py:170-253``), used by its tests only.
"""

from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Any, Mapping

import torch

from ..config.registry import ArchitectureConfig, config_from_dict
from ..parts.model import plan_tensor_decls
from .safetensors_io import write_safetensors

__all__ = ["random_tensors", "write_random_model"]

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def random_tensors(config: ArchitectureConfig, seed: int, std: float = 0.02, dtype: str = "bfloat16") -> dict[str, torch.Tensor]:
    """Checkpoint-named random tensors of the model ``config`` describes."""
    if dtype not in _DTYPES:
        raise ValueError(f"random weights are stored as bfloat16 or float32, not {dtype!r}")
    tensors: dict[str, torch.Tensor] = {}
    shape_hook = getattr(config, "checkpoint_shape", None)
    for (path, local), decl in plan_tensor_decls(config.to_plan()).items():
        name = config.checkpoint_names(path, local)[0]
        generator = torch.Generator(device="cpu")
        generator.manual_seed((int(seed) * 1_000_003 + zlib.crc32(name.encode())) % (2**63))
        if decl.role == "table":
            raise ValueError(f"no random initialisation for integer table {name}")
        if decl.init == "zeros":
            values = torch.zeros(decl.shape, dtype=torch.float32)
        else:
            values = torch.randn(decl.shape, generator=generator, dtype=torch.float32) * std
            if decl.init == "ones":
                values += 1.0
        storage = torch.float32 if decl.role == "vector" else _DTYPES[dtype]
        shape = shape_hook(path, local, decl.shape) if shape_hook else decl.shape
        tensors[name] = values.to(storage).reshape(shape)
    return tensors


def write_random_model(
    model_dir: str | Path,
    config: ArchitectureConfig | Mapping[str, Any],
    seed: int,
    std: float = 0.02,
    dtype: str = "bfloat16",
) -> Path:
    """Writes ``config.json`` and ``model.safetensors`` into ``model_dir``; returns the folder.

    ``config`` is a typed configuration or the raw ``config.json`` mapping (written back as given,
    so alternative spellings of keys survive).
    """
    model_dir = Path(model_dir)
    model_dir.mkdir(parents=True, exist_ok=True)
    if isinstance(config, Mapping):
        raw = dict(config)
        typed = config_from_dict(raw)
    else:
        typed = config
        raw = typed.to_json_dict()
    with open(model_dir / "config.json", "w") as stream:
        json.dump(raw, stream, indent=2)
    write_safetensors(
        model_dir / "model.safetensors",
        random_tensors(typed, seed, std, dtype),
        metadata={"format": "pt", "seed": str(seed), "std": repr(std)},
    )
    return model_dir
