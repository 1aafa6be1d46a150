"""The parts at the model's two ends: the token embedding (``lalamo/modules/embedding.py``) that
starts the 32-bit residual stream, and the read-out that turns normed rows into 32-bit logits.

A read-out declares ``tied = True`` if it has no table of its own; the model then hands it the
embedding's table under the local name ``"weight"``."""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import EmbeddingSpec, HeadSpec
from .base import Part, Runtime, TensorDecl, register_part

__all__ = ["Embedding", "Head", "LMHead", "TokenEmbedding"]


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, tokens: int) -> torch.Tensor:
        """The residual stream ``[tokens, model_dim]`` in 32-bit for these token ids."""
        raise NotImplementedError


class Head(Part):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """32-bit logits ``[rows, vocab]`` for normed rows ``x``."""
        raise NotImplementedError


@register_part(EmbeddingSpec)
class TokenEmbedding(Embedding):
    def __init__(self, spec: EmbeddingSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        self.weight = runtime.matrix(tensors["weight"])

    @classmethod
    def tensor_decls(cls, spec: EmbeddingSpec) -> dict[str, TensorDecl]:
        return {"weight": TensorDecl((spec.vocab_size, spec.model_dim))}

    def forward(self, token_ids: torch.Tensor, tokens: int) -> torch.Tensor:
        residual = self.runtime.empty(tokens, self.spec.model_dim, dtype=torch.float32)
        ops.embed(self.weight, token_ids, residual, self.spec.scale, self.runtime.status)
        return residual


@register_part(HeadSpec)
class LMHead(Head):
    def __init__(self, spec: HeadSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        weight = tensors["weight"]
        # a tied read-out is handed the embedding's table as the embedding holds it: no second copy
        self.weight = weight if weight.is_cuda and weight.dtype == runtime.dtype and weight.is_contiguous() else runtime.matrix(weight)

    @classmethod
    def tensor_decls(cls, spec: HeadSpec) -> dict[str, TensorDecl]:
        return {} if spec.tied else {"weight": TensorDecl((spec.vocab_size, spec.model_dim))}

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32, status=self.runtime.status)
