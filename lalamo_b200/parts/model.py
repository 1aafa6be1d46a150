"""The decoder: embedding, the scheduled blocks, final norm and LM head
(``lalamo/modules/decoder.py:220-317``, ``lalamo/modules/transformer.py:95-263``).

It runs the tokens of one :class:`~lalamo_b200.parts.base.StepInputs` and returns 32-bit logits
at the wanted rows only.
"""

from __future__ import annotations

from typing import Mapping

import torch

from .. import ops
from ..config.plan import ModelPlan
from .base import CacheNeed, CacheView, Norm, Part, Runtime, StepInputs, TensorDecl, build_part, part_type
from .block import Block, block_tensor_decls

__all__ = ["DecoderModel", "plan_tensor_decls"]

TensorKey = tuple[tuple, str]


def plan_tensor_decls(plan: ModelPlan) -> dict[TensorKey, TensorDecl]:
    """Every tensor of the model: ``(path of the part, local name) -> declaration``."""
    decls: dict[TensorKey, TensorDecl] = {
        (("embedding",), "weight"): TensorDecl((plan.vocab_size, plan.model_dim)),
    }
    for index, layer in enumerate(plan.layers):
        for (role, local), decl in block_tensor_decls(layer).items():
            decls[(("layers", index, role), local)] = decl
    for local, decl in part_type(plan.final_norm).tensor_decls(plan.final_norm).items():
        decls[(("final_norm",), local)] = decl
    if not plan.tie_embeddings:
        decls[(("lm_head",), "weight")] = TensorDecl((plan.vocab_size, plan.model_dim))
    return decls


class DecoderModel:
    def __init__(self, plan: ModelPlan, tensors: Mapping[TensorKey, torch.Tensor], runtime: Runtime) -> None:
        self.plan = plan
        self.runtime = runtime
        self.embedding = runtime.matrix(tensors[(("embedding",), "weight")])
        self.lm_head = self.embedding if plan.tie_embeddings else runtime.matrix(tensors[(("lm_head",), "weight")])
        self.blocks: list[Block] = []
        for index, layer in enumerate(plan.layers):
            block_tensors = {
                (path[2], local): tensor
                for (path, local), tensor in tensors.items()
                if len(path) == 3 and path[0] == "layers" and path[1] == index
            }
            self.blocks.append(Block(layer, block_tensors, runtime))
        final_tensors = {local: tensor for (path, local), tensor in tensors.items() if path == ("final_norm",)}
        self.final_norm: Norm = build_part(plan.final_norm, final_tensors, runtime)  # type: ignore[assignment]

    def cache_needs(self) -> list[CacheNeed | None]:
        """For each schedule entry the cache it owns (``None``: it owns none)."""
        needs: list[CacheNeed | None] = []
        for entry in self.plan.schedule:
            need = self.blocks[entry.layer].mixer.cache_need()
            needs.append(None if entry.cache_from is not None else need)
        return needs

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once: all parts' tensors and the LM head (of the
        embedding table a step reads only its tokens' rows).  For roofline arithmetic."""
        seen: dict[int, int] = {self.lm_head.data_ptr(): self.lm_head.numel() * self.lm_head.element_size()}

        def visit(obj: object, depth: int = 0) -> None:
            for value in vars(obj).values():
                if isinstance(value, torch.Tensor):
                    if value.is_cuda and value.data_ptr() != self.runtime.status.data_ptr():
                        seen[value.data_ptr()] = value.numel() * value.element_size()
                elif isinstance(value, (Part, Block)) and depth < 4:
                    visit(value, depth + 1)

        for entry in self.plan.schedule:
            visit(self.blocks[entry.layer])
        visit(self.final_norm)
        return sum(seen.values())

    def forward(self, step: StepInputs, caches: list[CacheView | None]) -> torch.Tensor:
        runtime = self.runtime
        residual = runtime.empty(step.tokens, self.plan.model_dim, dtype=torch.float32)
        ops.embed(self.embedding, step.token_ids, residual, self.plan.embedding_scale or 1.0, runtime.status)
        pending: torch.Tensor | None = None
        for position, entry in enumerate(self.plan.schedule):
            pending = self.blocks[entry.layer].forward(residual, pending, step, caches[position])
        if step.wanted == 0:
            return runtime.empty(0, self.plan.vocab_size, dtype=torch.float32)
        normed = self.final_norm.residual_forward(residual, pending, step.want_rows, step.wanted)
        return ops.linear(normed, self.lm_head, out_dtype=torch.float32, status=self.runtime.status)
