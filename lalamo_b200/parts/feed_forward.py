"""Dense gated feed-forward (``lalamo/modules/mlp.py:233-262``): ``down(up(x) * act(gate(x)))``
with the up and gate projections fused into one product, rows ordered ``[up ; gate]``."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import GatedMLPSpec
from .base import FeedForward, Runtime, StepInputs, TensorDecl, register_part

__all__ = ["GatedMLP"]


@register_part(GatedMLPSpec)
class GatedMLP(FeedForward):
    def __init__(self, spec: GatedMLPSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.up_gate = runtime.matrix(torch.cat([tensors["up_proj"], tensors["gate_proj"]], dim=0))
        self.down = runtime.matrix(tensors["down_proj"])

    @classmethod
    def tensor_decls(cls, spec: GatedMLPSpec) -> dict[str, TensorDecl]:
        return {
            "gate_proj": TensorDecl((spec.hidden_dim, spec.model_dim)),
            "up_proj": TensorDecl((spec.hidden_dim, spec.model_dim)),
            "down_proj": TensorDecl((spec.model_dim, spec.hidden_dim)),
        }

    can_accumulate = True

    def forward(self, x: torch.Tensor, step: StepInputs | None = None, residual: torch.Tensor | None = None) -> torch.Tensor | None:
        hidden = ops.gated_linear(x, self.up_gate, self.spec.activation, status=self.runtime.status)
        if residual is not None:
            early = ops.gated_linear_starts_successor_early(x.shape[0], self.up_gate.shape[0], x.shape[1])
            return ops.linear_accumulate(hidden, self.down, residual, status=self.runtime.status, started_early=early)
        return ops.linear(hidden, self.down, status=self.runtime.status)
