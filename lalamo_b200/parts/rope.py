"""Rotary position embedding (``lalamo/modules/rope.py:94-102``): the inverse frequencies
``theta ** (-2i / rotary_dim)`` as a 32-bit table; angles, sines and cosines are computed
in 32-bit inside the kernel that applies them."""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.plan import RopeSpec
from .base import PositionEncoding, Runtime, register_part

__all__ = ["Rope"]


@register_part(RopeSpec)
class Rope(PositionEncoding):
    def __init__(self, spec: RopeSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if spec.rotary_dim % 2 or spec.rotary_dim <= 0:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        channel = torch.arange(0, spec.rotary_dim, 2, dtype=torch.float32)
        inverse = 1.0 / (torch.tensor(spec.theta, dtype=torch.float32) ** (channel / spec.rotary_dim))
        self.rotary_dim = spec.rotary_dim
        self.inv_freq = inverse.to(device=runtime.device, dtype=torch.float32).contiguous()
