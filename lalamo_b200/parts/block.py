"""The arrangement of norms, mixer and feed-forward in one block, and the registry of arrangements.

An arrangement is a :class:`Block` subclass registered under the name a layer's specification
carries in ``arrangement``.  It names the *roles* of its parts (fields of the specification that
hold part specifications), gets them built, and says in ``forward`` how they are wired around the
residual stream.  The built-in one is ``"pre_norm"`` (``lalamo/modules/transformer_layer.py:220-377``):
``h = x + mixer(norm1(x)); y = h + ffn(norm2(h))``.

The residual stream is a 32-bit tensor that the block updates in place.  A block returns its last
sub-block's output *not yet added* (or ``None`` if it added it itself): the next norm (the next
block's, or the model's final norm) adds it while it normalises, which saves one pass over the stream.
What is not yet added is a tensor of the activation type or an ``ops.SlicedSum`` (a product left as the
partial sums of its K slices); ``Norm.residual_forward`` and ``ops.residual_add`` take either.
"""

from __future__ import annotations

from typing import Any, Callable, ClassVar, Mapping

import torch

from .base import CacheView, FeedForward, Mixer, Norm, Part, Runtime, StepInputs, TensorDecl, build_part, part_type

__all__ = ["Block", "PreNormBlock", "block_tensor_decls", "block_type", "build_block", "register_arrangement"]

_ARRANGEMENTS: dict[str, type["Block"]] = {}


def register_arrangement(name: str) -> Callable[[type["Block"]], type["Block"]]:
    """Class decorator: layers whose specification says ``arrangement == name`` are run by the class."""

    def decorate(block_class: type[Block]) -> type[Block]:
        _ARRANGEMENTS[name] = block_class
        return block_class

    return decorate


def block_type(spec: Any) -> type["Block"]:
    name = getattr(spec, "arrangement", None)
    if name not in _ARRANGEMENTS:
        raise ValueError(f"unknown block arrangement {name!r}; known: {sorted(_ARRANGEMENTS)}")
    return _ARRANGEMENTS[name]


def _role_specs(spec: Any) -> list[tuple[str, Any]]:
    """The part specifications of a layer, by role; roles whose field is ``None`` are left out."""
    return [(role, getattr(spec, role)) for role in block_type(spec).roles if getattr(spec, role, None) is not None]


def block_tensor_decls(spec: Any) -> dict[tuple[str, str], TensorDecl]:
    """``(role, local name) -> declaration`` for every tensor of the block's parts."""
    decls: dict[tuple[str, str], TensorDecl] = {}
    for role, part_spec in _role_specs(spec):
        for local, decl in part_type(part_spec).tensor_decls(part_spec).items():
            decls[(role, local)] = decl
    return decls


class Block:
    """Base of the arrangements.  Building sets one attribute per role (the built part, or ``None``
    where the specification leaves the role empty); one of the roles must be ``"mixer"``, since the
    model asks the block's mixer what cache it needs."""

    roles: ClassVar[tuple[str, ...]] = ()
    mixer: Mixer

    def __init__(self, spec: Any, tensors: Mapping[tuple[str, str], torch.Tensor], runtime: Runtime) -> None:
        if "mixer" not in self.roles:
            raise TypeError(f"{type(self).__name__}.roles must contain 'mixer'")
        self.spec = spec
        self.runtime = runtime
        for role in self.roles:
            setattr(self, role, None)
        for role, part_spec in _role_specs(spec):
            role_tensors = {local: tensor for (owner, local), tensor in tensors.items() if owner == role}
            setattr(self, role, build_part(part_spec, role_tensors, runtime))

    def parts(self) -> list[Part]:
        return [getattr(self, role) for role in self.roles if getattr(self, role) is not None]

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, step: StepInputs, cache: CacheView | None) -> torch.Tensor | None:
        """``residual`` holds the stream minus ``pending`` (the previous block's last output, or
        ``None`` if that was added already).  Returns this block's last output, to be added by the
        next norm, or ``None`` if the block added it itself."""
        raise NotImplementedError


@register_arrangement("pre_norm")
class PreNormBlock(Block):
    roles = ("pre_mixer_norm", "mixer", "pre_ffn_norm", "ffn")
    pre_mixer_norm: Norm
    pre_ffn_norm: Norm
    ffn: FeedForward

    def forward(self, residual: torch.Tensor, pending: torch.Tensor | None, step: StepInputs, cache: CacheView | None) -> torch.Tensor | None:
        normed = self.pre_mixer_norm.residual_forward(residual, pending)
        if self.mixer.can_accumulate:
            mixed = self.mixer.forward(normed, step, cache, residual=residual)
        else:
            mixed = self.mixer.forward(normed, step, cache)
        normed = self.pre_ffn_norm.residual_forward(residual, mixed)
        if self.ffn.can_accumulate:
            return self.ffn.forward(normed, step, residual=residual)
        return self.ffn.forward(normed, step)


def build_block(spec: Any, tensors: Mapping[tuple[str, str], torch.Tensor], runtime: Runtime) -> Block:
    return block_type(spec)(spec, tensors, runtime)
