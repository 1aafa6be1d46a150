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
from .embedding import Embedding, Head
from .block import Block, block_tensor_decls, build_block

__all__ = ["DecoderModel", "plan_tensor_decls"]

TensorKey = tuple[tuple, str]


def plan_tensor_decls(plan: ModelPlan) -> dict[TensorKey, TensorDecl]:
    """Every tensor of the model: ``(path of the part, local name) -> declaration``."""
    decls: dict[TensorKey, TensorDecl] = {}
    for local, decl in part_type(plan.embedding).tensor_decls(plan.embedding).items():
        decls[(("embedding",), local)] = decl
    for index, layer in enumerate(plan.layers):
        for (role, local), decl in block_tensor_decls(layer).items():
            decls[(("layers", index, role), local)] = decl
    for local, decl in part_type(plan.final_norm).tensor_decls(plan.final_norm).items():
        decls[(("final_norm",), local)] = decl
    for local, decl in part_type(plan.head).tensor_decls(plan.head).items():
        decls[(("lm_head",), local)] = decl
    return decls


class DecoderModel:
    def __init__(self, plan: ModelPlan, tensors: Mapping[TensorKey, torch.Tensor], runtime: Runtime) -> None:
        self.plan = plan
        self.runtime = runtime
        embedding_tensors = {local: tensor for (path, local), tensor in tensors.items() if path == ("embedding",)}
        self.embedding: Embedding = build_part(plan.embedding, embedding_tensors, runtime)  # type: ignore[assignment]
        head_tensors = {local: tensor for (path, local), tensor in tensors.items() if path == ("lm_head",)}
        if getattr(plan.head, "tied", False):
            head_tensors = {**head_tensors, "weight": self.embedding.weight}
        self.head: Head = build_part(plan.head, head_tensors, runtime)  # type: ignore[assignment]
        self.blocks: list[Block] = []
        for index, layer in enumerate(plan.layers):
            block_tensors = {
                (path[2], local): tensor
                for (path, local), tensor in tensors.items()
                if len(path) == 3 and path[0] == "layers" and path[1] == index
            }
            self.blocks.append(build_block(layer, block_tensors, runtime))
        final_tensors = {local: tensor for (path, local), tensor in tensors.items() if path == ("final_norm",)}
        self.final_norm: Norm = build_part(plan.final_norm, final_tensors, runtime)  # type: ignore[assignment]

    def cache_needs(self) -> list[CacheNeed | None]:
        """For each schedule entry the cache it owns (``None``: it owns none)."""
        needs: list[CacheNeed | None] = []
        for entry in self.plan.schedule:
            need = self.blocks[entry.layer].mixer.cache_need()
            needs.append(None if entry.cache_from is not None else need)
        return needs

    def step_planners(self) -> list[Part]:
        """The parts that plan work on the host for every step (one per plan key)."""
        planners: dict[object, Part] = {}
        for entry in self.plan.schedule:
            block = self.blocks[entry.layer]
            for part in block.parts():
                if type(part).plan_step is not Part.plan_step:
                    planners.setdefault(part.step_plan_key(), part)
        return list(planners.values())

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once: all parts' tensors and the LM head (of the
        embedding table a step reads only its tokens' rows).  For roofline arithmetic."""
        seen: dict[int, int] = {}

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
        visit(self.head)
        return sum(seen.values())

    def forward(self, step: StepInputs, caches: list[CacheView | None]) -> torch.Tensor:
        runtime = self.runtime
        residual = self.embedding.forward(step.token_ids, step.tokens)
        pending: torch.Tensor | None = None
        for position, entry in enumerate(self.plan.schedule):
            pending = self.blocks[entry.layer].forward(residual, pending, step, caches[position])
        if step.wanted == 0:
            return runtime.empty(0, self.plan.vocab_size, dtype=torch.float32)
        normed = self.final_norm.residual_forward(residual, pending, step.want_rows, step.wanted)
        return self.head.forward(normed)
