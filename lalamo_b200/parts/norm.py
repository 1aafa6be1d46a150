"""RMS norm (``lalamo/modules/normalization.py:89-126``): statistics in 32-bit, the
normalised value rounded to the activation type before the multiplication by the scale."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import RMSNormSpec
from .base import Norm, Runtime, TensorDecl, register_part

__all__ = ["RMSNorm"]


@register_part(RMSNormSpec)
class RMSNorm(Norm):
    def __init__(self, spec: RMSNormSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.scale = runtime.vector(tensors["scale"])

    @classmethod
    def tensor_decls(cls, spec: RMSNormSpec) -> dict[str, TensorDecl]:
        return {"scale": TensorDecl((spec.dim,), role="vector", init="ones")}

    def _out(self, x: torch.Tensor, rows: torch.Tensor | None, num_rows: int | None) -> torch.Tensor:
        count = x.shape[0] if rows is None else (rows.numel() if num_rows is None else num_rows)
        return self.runtime.empty(count, self.spec.dim)

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None, num_rows: int | None = None) -> torch.Tensor:
        out = self._out(x, rows, num_rows)
        ops.rmsnorm(x, self.scale, out, self.spec.eps, rows=rows, scale_offset=self.spec.scale_offset)
        return out

    def residual_forward(
        self,
        residual: torch.Tensor,
        delta: "torch.Tensor | ops.SlicedSum | None",
        rows: torch.Tensor | None = None,
        num_rows: int | None = None,
    ) -> torch.Tensor:
        out = self._out(residual, rows, num_rows)
        ops.rmsnorm(
            residual,
            self.scale,
            out,
            self.spec.eps,
            delta=delta,
            rows=rows,
            scale_offset=self.spec.scale_offset,
            write_back=delta is not None and rows is None,
        )
        return out
