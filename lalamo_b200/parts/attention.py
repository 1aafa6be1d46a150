"""Grouped-query causal attention over a paged cache
(``lalamo/modules/token_mixers/attention.py:511-620``): fused q/k/v projection, per-head RMS
norm of queries and keys, position encoding, keys and values written to the request's pages,
softmax attention in 32-bit over the visible keys, out-projection."""

from __future__ import annotations

import os

from typing import Mapping

import numpy as np
import torch

from .. import ops
from ..config.plan import AttentionSpec, RMSNormSpec, RopeSpec
from .base import REPLAY_MAX_TOKENS, CacheNeed, HostSegments, Mixer, PagedKVNeed, PagedKVView, Runtime, StepInputs, TensorDecl, build_part, register_part

__all__ = ["ALONE_LIMIT", "TILE_TOKENS", "Attention", "shared_tile_keys"]

# How the attention kernels divide a step: tokens of portions of at most ALONE_LIMIT tokens attend
# alone (split over the keys); longer portions are cut into tiles of at most TILE_TOKENS consecutive tokens.
ALONE_LIMIT = 16
TILE_TOKENS = ops.PREFILL_TILE
EARLY_ATTENTION = os.environ.get("LALAMO_B200_EARLY_ATTENTION", "1") != "0"  # the split-key attention starts under the q/k/v rewrite
SHARED_TILE_KEYS = 512  # where tiles are shared, a tile that sees at least this many keys is worked on by two CTAs
LONG_TILE_KEYS = 3072  # a launch's tiles count as long if they see this many keys on average


def _slot_use(ctas: int, slots: int) -> float:
    """The share of the resident-CTA slots that ``ctas`` CTAs keep busy over the rounds they need."""
    return ctas / (-(-ctas // slots) * slots)


def shared_tile_keys(num_tiles: int, num_heads: int, num_groups: int, sms: int, tokens: int, lengths: tuple[int, ...] = (),
                     contexts: tuple[int, ...] = ()) -> int:
    """From how many visible keys on a tile of the tcgen05 prefill attention is worked on by two CTAs (each half of
    the keys, merged at the end); 0: never, the launch has one CTA per tile.  Two CTAs per tile pay where that
    fills the SMs better: with fewer CTAs than SMs; or, in steps that are never replayed (so that the answer may
    depend on the contexts), where tiles mostly see thousands of keys and their CTAs fill the resident slots
    (three per SM) badly, as 512 CTAs fill 444.  Launching as clusters costs 12 to 25 % by itself, so whole
    prompts from position 0, whose early tiles are short, stay unpaired."""
    per_group = num_heads // num_groups
    parts = -(-TILE_TOKENS // max(1, min(TILE_TOKENS, 128 // per_group)))
    ctas = num_tiles * num_groups * parts
    if ctas <= sms:
        return SHARED_TILE_KEYS
    if tokens > REPLAY_MAX_TOKENS and contexts:
        keys = sum(length * (context + length / 2) for length, context in zip(lengths, contexts))
        if keys / max(1, sum(lengths)) >= LONG_TILE_KEYS and _slot_use(2 * ctas, 3 * sms) > _slot_use(ctas, 3 * sms) + 0.1:
            return SHARED_TILE_KEYS
    return 0


@register_part(AttentionSpec)
class Attention(Mixer):
    graph_safe = True
    def __init__(self, spec: AttentionSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime) -> None:
        super().__init__(spec, tensors, runtime)
        if spec.num_heads % spec.num_groups:
            raise ValueError(f"num_heads={spec.num_heads} is not a multiple of num_groups={spec.num_groups}")
        if spec.window is not None and spec.window < 1:
            raise ValueError(f"window must be positive, got {spec.window}")
        self.qkv = runtime.matrix(torch.cat([tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]], dim=0))
        self.out_proj = runtime.matrix(tensors["out_proj"])
        self.q_norm = self.k_norm = None
        self.norm_eps, self.norm_offset = 0.0, 0.0
        if spec.qk_norm is not None:
            if not isinstance(spec.qk_norm, RMSNormSpec) or spec.qk_norm.dim != spec.head_dim:
                raise ValueError("the per-head norm must be an RMS norm over head_dim")
            self.q_norm = runtime.vector(tensors["q_norm"])
            self.k_norm = runtime.vector(tensors["k_norm"])
            self.norm_eps, self.norm_offset = spec.qk_norm.eps, spec.qk_norm.scale_offset
        self.position = None
        if spec.position is not None:
            if not isinstance(spec.position, RopeSpec):
                raise ValueError(f"attention applies rotary position encodings, not {type(spec.position).__name__}")
            self.position = build_part(spec.position, {}, runtime)
        self.scale = spec.scale if spec.scale is not None else spec.head_dim**-0.5

    @classmethod
    def tensor_decls(cls, spec: AttentionSpec) -> dict[str, TensorDecl]:
        decls = {
            "q_proj": TensorDecl((spec.num_heads * spec.head_dim, spec.model_dim)),
            "k_proj": TensorDecl((spec.num_groups * spec.head_dim, spec.model_dim)),
            "v_proj": TensorDecl((spec.num_groups * spec.head_dim, spec.model_dim)),
            "out_proj": TensorDecl((spec.model_dim, spec.num_heads * spec.head_dim)),
        }
        if spec.qk_norm is not None:
            decls["q_norm"] = TensorDecl((spec.head_dim,), role="vector", init="ones")
            decls["k_norm"] = TensorDecl((spec.head_dim,), role="vector", init="ones")
        return decls

    def cache_need(self) -> CacheNeed | None:
        return PagedKVNeed(num_groups=self.spec.num_groups, head_dim=self.spec.head_dim, window=self.spec.window)

    # The kernels' work lists depend on where the portions start and how long they are, not on what
    # the cache holds, and they are the same for every attention layer.
    step_plan_uses_context = False

    def step_plan_key(self) -> object:
        return ("attention", ALONE_LIMIT, TILE_TOKENS)

    def plan_step(self, segments: HostSegments) -> dict[str, np.ndarray]:
        """``alone``: the rows that attend alone; ``tiles``: ``(first row, count)`` of each tile."""
        alone: list[int] = []
        tiles: list[tuple[int, int]] = []
        for start, length in zip(segments.start, segments.length):
            if length <= ALONE_LIMIT:
                alone.extend(range(start, start + length))
            else:
                tiles.extend((first, min(TILE_TOKENS, start + length - first)) for first in range(start, start + length, TILE_TOKENS))
        return {"alone": np.asarray(alone, dtype=np.int32), "tiles": np.asarray(tiles, dtype=np.int32).reshape(-1)}

    can_accumulate = True

    def _project_out(self, mixed: torch.Tensor, residual: torch.Tensor | None) -> torch.Tensor | None:
        if residual is not None:
            return ops.linear_accumulate(mixed, self.out_proj, residual, status=self.runtime.status)
        return ops.linear(mixed, self.out_proj, status=self.runtime.status)

    def forward(self, x: torch.Tensor, step: StepInputs, cache: PagedKVView, residual: torch.Tensor | None = None) -> torch.Tensor | None:  # type: ignore[override]
        spec = self.spec
        qkv = ops.linear(x, self.qkv, status=self.runtime.status)
        queries = self.runtime.empty(step.tokens, spec.num_heads * spec.head_dim)
        ops.qk_norm_rope_write(
            qkv,
            queries,
            cache.k_pages,
            cache.v_pages,
            q_weight=self.q_norm,
            k_weight=self.k_norm,
            eps=self.norm_eps,
            scale_offset=self.norm_offset,
            inv_freq=self.position.inv_freq if self.position is not None else None,
            rotary_dim=self.position.rotary_dim if self.position is not None else 0,
            positions=step.positions,
            token_segment=step.token_segment,
            block_table=cache.block_table,
            num_heads=spec.num_heads,
            num_groups=spec.num_groups,
            head_dim=spec.head_dim,
            write_kv=cache.owns,
            status=self.runtime.status,
        )
        mixed = self.runtime.empty(step.tokens, spec.num_heads * spec.head_dim)
        page_size = cache.k_pages.shape[1]
        common = dict(
            positions=step.positions,
            token_segment=step.token_segment,
            block_table=cache.block_table,
            num_heads=spec.num_heads,
            num_groups=spec.num_groups,
            head_dim=spec.head_dim,
            scale=self.scale,
            window=spec.window,
            status=self.runtime.status,
        )
        alone_ok = ops.decode_attention_supported(self.runtime.dtype, spec.head_dim, page_size)
        tiles_ok = ops.prefill_attention_supported(self.runtime.dtype, spec.num_heads, spec.num_groups, spec.head_dim, page_size)
        if alone_ok:
            lists, host_lists = step.plan_of(self)
            num_alone, num_tiles = host_lists["alone"].size, host_lists["tiles"].size // 2
        if alone_ok and (tiles_ok or num_tiles == 0):
            # Tokens of short portions attend alone (split over the keys); long portions run in tiles.
            if num_alone:
                everything = num_alone == step.tokens
                # The rewrite of q, k and v just above is the kernel before this one and writes, for any token that
                # attends alone, no more than the newest ALONE_LIMIT positions it sees (its own portion's).
                ops.attention_decode(queries, cache.k_pages, cache.v_pages, mixed, max_context=step.max_context,
                                     token_list=None if everything else lists["alone"], num_listed=num_alone,
                                     fresh_keys=ALONE_LIMIT if cache.owns and EARLY_ATTENTION else None, **common)
            if num_tiles:
                split_tiles = 0
                if spec.head_dim == 64 and ops.USE_TCGEN05_ATTENTION:
                    split_tiles = shared_tile_keys(num_tiles, spec.num_heads, spec.num_groups, ops.sm_count(), step.tokens,
                                                   step.host_segment_length, step.host_segment_context) // 64
                ops.attention_prefill(queries, cache.k_pages, cache.v_pages, mixed, tiles=lists["tiles"], num_tiles=num_tiles, split_tiles=split_tiles, **common)
            return self._project_out(mixed, residual)
        ops.paged_attention_plain(
            queries,
            cache.k_pages,
            cache.v_pages,
            mixed,
            positions=step.positions,
            token_segment=step.token_segment,
            block_table=cache.block_table,
            num_heads=spec.num_heads,
            num_groups=spec.num_groups,
            head_dim=spec.head_dim,
            scale=self.scale,
            window=spec.window,
            status=self.runtime.status,
        )
        return self._project_out(mixed, residual)
