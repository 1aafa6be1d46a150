"""Runs the sampling kernels for the rows of one step.

Each row carries its request's policy, its own random key (derived from the generation seed and
the request's number, so its tokens do not depend on what else is in the batch; the reference
derives per-sequence keys for the same reason, ``lalamo/inference/batch_scheduler.py:792-794``)
and the number of tokens it has drawn before.  Token counts for the repetition, presence and
frequency penalties are per-request state in the cache manager's slots.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import ops
from ..cache.manager import CacheManager
from .policy import MAX_BANNED_TOKENS, SamplingPolicy

__all__ = ["PendingSample", "SampleRow", "Sampler", "pack_rows", "request_key"]

_MASK64 = (1 << 64) - 1


def request_key(seed: int, request_number: int) -> tuple[int, int]:
    """A 64-bit key for a request from the generation seed (SplitMix64 finaliser)."""
    z = (int(seed) * 0x9E3779B97F4A7C15 + int(request_number) * 0xBF58476D1CE4E5B9 + 0x94D049BB133111EB) & _MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
    z ^= z >> 31
    return z & 0xFFFFFFFF, z >> 32


@dataclass
class SampleRow:
    policy: SamplingPolicy
    key: tuple[int, int]
    draw: int
    count_slot: int = -1


def pack_rows(rows: list[SampleRow]) -> np.ndarray:
    """The kernel's parameter records, ``[rows, 27]`` int32 words."""
    packed = np.zeros((len(rows), ops.SAMPLE_PARAM_WORDS), dtype=np.int32)
    as_float = packed.view(np.float32)
    as_unsigned = packed.view(np.uint32)
    for index, row in enumerate(rows):
        policy = row.policy
        as_float[index, 0] = -1.0 if policy.temperature is None else policy.temperature
        packed[index, 1] = 0 if policy.top_k is None else policy.top_k
        as_float[index, 2] = 1.0 if policy.top_p is None else policy.top_p
        as_float[index, 3] = 0.0 if policy.min_p is None else policy.min_p
        as_float[index, 4] = 1.0 if policy.repetition_penalty is None else policy.repetition_penalty
        as_float[index, 5] = 0.0 if policy.presence_penalty is None else policy.presence_penalty
        as_float[index, 6] = 0.0 if policy.frequency_penalty is None else policy.frequency_penalty
        packed[index, 7] = row.count_slot if policy.has_count_penalties else -1
        as_unsigned[index, 8] = row.key[0]
        as_unsigned[index, 9] = row.key[1]
        as_unsigned[index, 10] = row.draw & 0xFFFFFFFF
        banned = list(policy.banned_tokens) + [-1] * (MAX_BANNED_TOKENS - len(policy.banned_tokens))
        packed[index, 11:27] = banned
    return packed


@dataclass
class PendingSample:
    """The tokens of one step, sampled and on their way to the host.  ``device`` holds them on the
    device (the next step may take its token ids from there); :meth:`wait` returns them on the host."""

    device: torch.Tensor
    host: torch.Tensor | None
    copied: torch.cuda.Event | None

    def wait(self) -> list[int]:
        if self.host is None:
            return []
        assert self.copied is not None
        self.copied.synchronize()
        return self.host.tolist()


class Sampler:
    PINNED_BUFFERS = 3  # results in flight: a buffer is written again two calls after it was handed out

    def __init__(self, cache: CacheManager, vocab_size: int, device: torch.device) -> None:
        self.cache = cache
        self.vocab_size = vocab_size
        self.device = device
        self._work: torch.Tensor | None = None
        self._counts: torch.Tensor | None = None
        self._pinned: list[torch.Tensor | None] = [None] * self.PINNED_BUFFERS
        self._turn = 0
        self.last_d2h_bytes = 0

    def counts(self) -> torch.Tensor:
        if self._counts is None:
            self._counts = self.cache.add_slot_state("sampler_token_counts", (self.vocab_size,), torch.int32)
        return self._counts

    def set_counts(self, slot: int, tokens: list[int]) -> None:
        """Sets a request's counts to the counts of ``tokens`` (its prompt, or the last tokens of
        it when the policy counts a suffix only; ``lalamo/sampling.py:118-149``)."""
        histogram = np.bincount(np.asarray(tokens, dtype=np.int64), minlength=self.vocab_size).astype(np.int32)
        self.counts()[slot].copy_(torch.from_numpy(histogram), non_blocking=False)

    def update_counts(self, slots: list[int], add: list[int], remove: list[int]) -> None:
        if not slots:
            return
        packed = torch.tensor([slots, add, remove], dtype=torch.int32).to(self.device)
        ops.update_counts(self.counts(), packed[0].contiguous(), packed[1].contiguous(), packed[2].contiguous())

    def sample(self, logits: torch.Tensor, rows: list[SampleRow]) -> list[int]:
        """One token per row of ``logits``; returns them on the host."""
        return self.sample_async(logits, rows).wait()

    def sample_async(self, logits: torch.Tensor, rows: list[SampleRow]) -> PendingSample:
        """Launches the sampling of one token per row of ``logits`` and their copy to the host, and
        returns without waiting.  At most ``PINNED_BUFFERS - 1`` results may be outstanding."""
        count = logits.shape[0]
        if count != len(rows):
            raise ValueError(f"{count} logit rows for {len(rows)} sampling rows")
        if count == 0:
            self.last_d2h_bytes = 0
            return PendingSample(torch.empty(0, dtype=torch.int32, device=self.device), None, None)
        out = torch.empty(count, dtype=torch.int32, device=self.device)
        if all(row.policy.is_plain_greedy for row in rows):
            ops.argmax(logits, out)
        else:
            if self._work is None or self._work.numel() < count * self.vocab_size:
                self._work = torch.empty(max(count, 8) * self.vocab_size, dtype=torch.float32, device=self.device)
            params = torch.from_numpy(pack_rows(rows)).to(self.device)
            needs_counts = any(row.policy.has_count_penalties for row in rows)
            ops.sample(logits, self._work, self.counts() if needs_counts else None, params, out)
        index = self._turn
        self._turn = (self._turn + 1) % self.PINNED_BUFFERS
        pinned = self._pinned[index]
        if pinned is None or pinned.numel() < count:
            pinned = torch.empty(max(64, count), dtype=torch.int32, pin_memory=True)
            self._pinned[index] = pinned
        host = pinned[:count]
        host.copy_(out, non_blocking=True)
        copied = torch.cuda.Event()
        copied.record()
        self.last_d2h_bytes = count * 4
        return PendingSample(out, host, copied)
