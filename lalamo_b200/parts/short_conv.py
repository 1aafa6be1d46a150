"""The gated short-convolution mixer (``lalamo/modules/token_mixers/short_conv.py:102-154``):
in-projection to ``(B, C, x)``, ``u = B * x``, a depthwise causal convolution of ``kernel_size``
taps over ``[state ; u]``, the gate ``C`` and the out-projection.  The state (the last
``kernel_size - 1`` rows of ``u``) lives in a per-request slot."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import ShortConvSpec
from .base import CacheNeed, Mixer, Runtime, SlotStateNeed, SlotStateView, StepInputs, TensorDecl, register_part

__all__ = ["ShortConv"]


@register_part(ShortConvSpec)
class ShortConv(Mixer):
    graph_safe = True
    def __init__(self, spec: ShortConvSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if spec.kernel_size < 1:
            raise ValueError(f"kernel_size must be at least 1, got {spec.kernel_size}")
        self.in_proj = runtime.matrix(tensors["in_proj"])
        self.out_proj = runtime.matrix(tensors["out_proj"])
        self.conv_weight = runtime.vector(tensors["conv_weight"].reshape(spec.model_dim, spec.kernel_size))
        self.conv_bias = runtime.vector(tensors["conv_bias"]) if spec.has_bias else None

    @classmethod
    def tensor_decls(cls, spec: ShortConvSpec) -> dict[str, TensorDecl]:
        decls = {
            "in_proj": TensorDecl((3 * spec.model_dim, spec.model_dim)),
            "conv_weight": TensorDecl((spec.model_dim, spec.kernel_size), role="vector"),
            "out_proj": TensorDecl((spec.model_dim, spec.model_dim)),
        }
        if spec.has_bias:
            decls["conv_bias"] = TensorDecl((spec.model_dim,), role="vector")
        return decls

    def cache_need(self) -> CacheNeed | None:
        return SlotStateNeed(shape=(max(self.spec.kernel_size - 1, 1), self.spec.model_dim))

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs, cache: SlotStateView, residual: torch.Tensor | None = None) -> torch.Tensor | None:  # type: ignore[override]
        if not cache.owns:
            raise ValueError("a short-convolution layer cannot read another layer's state")
        state = cache.state
        if self.spec.kernel_size == 1:
            state = state[:, :0]
        gated = ops.short_conv_linear(
            x,
            self.in_proj,
            state,
            self.conv_weight,
            self.conv_bias,
            token_segment=step.token_segment,
            segment_start=step.segment_start,
            segment_length=step.segment_length,
            segment_slot=cache.segment_slot,
            segments=step.segments,
            status=self.runtime.status,
        )
        if residual is not None:
            return ops.linear_accumulate(gated, self.out_proj, residual, status=self.runtime.status)
        return ops.linear(gated, self.out_proj, status=self.runtime.status)
