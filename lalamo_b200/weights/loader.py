"""Loading a model's tensors from safetensors, by name.

Every tensor the plan's parts declare is looked up under the names the architecture gives it
(first match among the aliases wins), its shape is checked (singleton dimensions are ignored, so
a depthwise convolution stored as ``[dim, 1, taps]`` or ``[dim, taps, 1]`` fits ``[dim, taps]``),
and everything that does not fit is reported in *one* error: missing tensors, unexpected
tensors and wrong shapes together.

Storage types are kept: bfloat16 stays bfloat16 and a tensor stored in 32-bit stays 32-bit
(float16 and float64 become float32); integer tables become int32.  Casting to the compute type is the model's business.
The reference casts to its template's type at load (``lalamo/utils/surgery.py:37-45``) and
reports one problem at a time.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from pathlib import Path

import torch

from ..config.plan import ModelPlan
from ..config.registry import ArchitectureConfig
from ..parts.base import TensorDecl
from ..parts.model import TensorKey, plan_tensor_decls
from .safetensors_io import Checkpoint, open_checkpoint

__all__ = ["WeightsError", "load_weights", "squeezed"]


def squeezed(shape: tuple[int, ...]) -> tuple[int, ...]:
    return tuple(extent for extent in shape if extent != 1) or (1,) if shape else ()


@dataclass
class WeightsError(ValueError):
    """The checkpoint does not fit the model.  All problems are listed."""

    missing: list[str] = field(default_factory=list)
    unexpected: list[str] = field(default_factory=list)
    wrong_shape: list[tuple[str, tuple[int, ...], tuple[int, ...]]] = field(default_factory=list)
    wrong_dtype: list[tuple[str, str]] = field(default_factory=list)

    def __str__(self) -> str:
        lines = ["the checkpoint does not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}):")
            lines += [f"    {name}" for name in self.missing]
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}):")
            lines += [f"    {name}" for name in self.unexpected]
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}):")
            lines += [f"    {name}: expected {list(expected)}, found {list(found)}" for name, expected, found in self.wrong_shape]
        if self.wrong_dtype:
            lines.append(f"  unusable types ({len(self.wrong_dtype)}):")
            lines += [f"    {name}: {dtype}" for name, dtype in self.wrong_dtype]
        return "\n".join(lines)

    def __bool__(self) -> bool:
        return bool(self.missing or self.unexpected or self.wrong_shape or self.wrong_dtype)


_FLOAT_STORAGE = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float32, "F64": torch.float32}
_INT_STORAGE = {"I64", "I32", "I16", "I8", "U8"}


def _convert(tensor: torch.Tensor, storage: str, decl: TensorDecl) -> torch.Tensor:
    if decl.role == "table":
        return tensor.to(torch.int32)
    return tensor.to(_FLOAT_STORAGE[storage])


def load_weights(
    model_dir: str | Path,
    config: ArchitectureConfig,
    plan: ModelPlan | None = None,
    checkpoint: Checkpoint | None = None,
) -> dict[TensorKey, torch.Tensor]:
    """All tensors of the model as ``(path, local name) -> CPU tensor`` in storage type."""
    plan = plan or config.to_plan()
    checkpoint = checkpoint or open_checkpoint(model_dir)
    decls = plan_tensor_decls(plan)
    problems = WeightsError()
    used: set[str] = set()
    found: dict[TensorKey, str] = {}
    for key, decl in decls.items():
        path, local = key
        candidates = config.checkpoint_names(path, local)
        name = next((candidate for candidate in candidates if candidate in checkpoint), None)
        if name is None:
            problems.missing.append(candidates[0] if len(candidates) == 1 else f"{candidates[0]} (or {', '.join(candidates[1:])})")
            continue
        used.add(name)
        info = checkpoint[name]
        if squeezed(info.shape) != squeezed(decl.shape):
            problems.wrong_shape.append((name, decl.shape, info.shape))
            continue
        wanted_int = decl.role == "table"
        if (wanted_int and info.dtype not in _INT_STORAGE) or (not wanted_int and info.dtype not in _FLOAT_STORAGE):
            problems.wrong_dtype.append((name, info.dtype))
            continue
        found[key] = name
    problems.unexpected = sorted(name for name in checkpoint if name not in used)
    if problems:
        raise problems
    return {key: _convert(checkpoint.read(name), checkpoint[name].dtype, decls[key]).reshape(decls[key].shape) for key, name in found.items()}
