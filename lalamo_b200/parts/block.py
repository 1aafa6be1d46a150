"""The arrangement of norm, mixer and feed-forward in one block
(``lalamo/modules/transformer_layer.py:220-377``): pre-norm with two residual sums.

The residual stream is a 32-bit tensor that the block updates in place.  A block returns its
feed-forward output *not yet added*: the next norm (the next block's, or the model's final
norm) adds it while it normalises, which saves one pass over the stream.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.plan import BlockSpec
from .base import CacheView, FeedForward, Mixer, Norm, Runtime, StepInputs, TensorDecl, build_part, part_type

__all__ = ["Block", "block_tensor_decls"]

_ROLES = ("pre_mixer_norm", "mixer", "pre_ffn_norm", "ffn")


def block_tensor_decls(spec: BlockSpec) -> dict[tuple[str, str], TensorDecl]:
    """``(role, local name) -> declaration`` for every tensor of the block's parts."""
    decls: dict[tuple[str, str], TensorDecl] = {}
    for role in _ROLES:
        part_spec = getattr(spec, role)
        for local, decl in part_type(part_spec).tensor_decls(part_spec).items():
            decls[(role, local)] = decl
    return decls


class Block:
    def __init__(self, spec: BlockSpec, tensors: Mapping[tuple[str, str], torch.Tensor], runtime: Runtime) -> None:
        if spec.arrangement != "pre_norm":
            raise ValueError(f"unknown block arrangement {spec.arrangement!r}; known: 'pre_norm'")
        self.spec = spec

        def tensors_of(role: str) -> dict[str, torch.Tensor]:
            return {local: tensor for (owner, local), tensor in tensors.items() if owner == role}

        self.pre_mixer_norm: Norm = build_part(spec.pre_mixer_norm, tensors_of("pre_mixer_norm"), runtime)  # type: ignore[assignment]
        self.mixer: Mixer = build_part(spec.mixer, tensors_of("mixer"), runtime)  # type: ignore[assignment]
        self.pre_ffn_norm: Norm = build_part(spec.pre_ffn_norm, tensors_of("pre_ffn_norm"), runtime)  # type: ignore[assignment]
        self.ffn: FeedForward = build_part(spec.ffn, tensors_of("ffn"), runtime)  # type: ignore[assignment]

    def forward(
        self,
        residual: torch.Tensor,
        pending: torch.Tensor | None,
        step: StepInputs,
        cache: CacheView | None,
    ) -> torch.Tensor | None:
        """``residual`` holds the stream minus ``pending`` (the previous block's feed-forward
        output, or ``None`` if that was added already).  Returns this block's feed-forward output, to
        be added by the next norm, or ``None`` if the feed-forward added it itself."""
        normed = self.pre_mixer_norm.residual_forward(residual, pending)
        if self.mixer.can_accumulate:
            mixed = self.mixer.forward(normed, step, cache, residual=residual)
        else:
            mixed = self.mixer.forward(normed, step, cache)
        normed = self.pre_ffn_norm.residual_forward(residual, mixed)
        if self.ffn.can_accumulate:
            return self.ffn.forward(normed, step, residual=residual)
        return self.ffn.forward(normed, step)
