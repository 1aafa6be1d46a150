"""A plain NumPy restatement of the reference's logit processors (lalamo/sampling.py:187-300) and of
the engine's draw (arg-max of logit + Gumbel noise from Philox-4x32-10).  It sorts where the engine
searches, and shares no code with it."""

from __future__ import annotations

import numpy as np

NEG_INF = np.float32(-np.inf)


def process_logits(
    logits: np.ndarray,
    *,
    temperature: float | None = None,
    top_k: int | None = None,
    top_p: float | None = None,
    min_p: float | None = None,
    banned_tokens: tuple[int, ...] = (),
    repetition_penalty: float | None = None,
    presence_penalty: float | None = None,
    frequency_penalty: float | None = None,
    token_counts: np.ndarray | None = None,
) -> np.ndarray:
    """ban -> repetition -> presence -> frequency -> temperature -> top-k -> top-p -> min-p
    (lalamo/sampling.py:187-196), in float32 as the reference computes."""
    x = logits.astype(np.float32).copy()
    vocab = x.shape[0]
    counts = np.zeros(vocab, np.int32) if token_counts is None else token_counts
    for token in banned_tokens:  # sampling.py:219-228
        x[token] = NEG_INF
    if repetition_penalty is not None:  # sampling.py:236-242
        penalised = np.where(x > 0, x / np.float32(repetition_penalty), x * np.float32(repetition_penalty))
        x = np.where(counts > 0, penalised, x).astype(np.float32)
    if presence_penalty is not None:  # sampling.py:244-248
        x = np.where(counts > 0, x - np.float32(presence_penalty), x).astype(np.float32)
    if frequency_penalty is not None:  # sampling.py:250-254
        x = (x - np.float32(frequency_penalty) * counts.astype(np.float32)).astype(np.float32)
    if temperature is not None:  # sampling.py:256-266
        if temperature == 0.0:
            best = int(np.argmax(x))
            x = np.full(vocab, NEG_INF, np.float32)
            x[best] = 1.0
        else:
            x = (x / np.float32(temperature)).astype(np.float32)
    if top_k is not None and top_k > 0:  # sampling.py:268-276: stable descending sort, exactly k kept
        k = min(max(top_k, 1), vocab)
        order = np.argsort(-x, kind="stable")
        ranks = np.empty(vocab, np.int64)
        ranks[order] = np.arange(vocab)
        x = np.where(ranks < k, x, NEG_INF).astype(np.float32)
    if top_p is not None and top_p < 1.0:  # sampling.py:278-292
        order = np.argsort(-x, kind="stable")
        sorted_logits = x[order]
        shifted = sorted_logits - sorted_logits[0]
        probabilities = np.exp(shifted.astype(np.float64))
        probabilities /= probabilities.sum()
        before = np.cumsum(probabilities) - probabilities
        remove = np.zeros(vocab, bool)
        remove[order] = before >= top_p
        x = np.where(remove, NEG_INF, x).astype(np.float32)
    if min_p is not None and min_p > 0.0:  # sampling.py:294-300
        cutoff = x.max() + np.float32(np.log(np.float32(min_p)))
        x = np.where(x >= cutoff, x, NEG_INF).astype(np.float32)
    return x


def philox_first_word(counter0: np.ndarray, counter1: int, key0: int, key1: int) -> np.ndarray:
    """Philox-4x32-10 of counters (counter0, counter1, 0, 0) under key (key0, key1); word 0."""
    mask = np.uint64(0xFFFFFFFF)
    c0 = counter0.astype(np.uint64)
    c1 = np.full_like(c0, counter1, dtype=np.uint64)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = np.uint64(key0), np.uint64(key1)
    for _ in range(10):
        p0 = np.uint64(0xD2511F53) * c0
        p1 = np.uint64(0xCD9E8D57) * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & mask
        hi1, lo1 = p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = (hi1 ^ c1 ^ k0) & mask, lo1, (hi0 ^ c3 ^ k1) & mask, lo0
        k0 = (k0 + np.uint64(0x9E3779B9)) & mask
        k1 = (k1 + np.uint64(0xBB67AE85)) & mask
    return c0.astype(np.uint32)


def gumbel_scores(processed: np.ndarray, key: tuple[int, int], draw: int) -> np.ndarray:
    words = philox_first_word(np.arange(processed.shape[0]), draw, key[0], key[1])
    uniform = (np.floor(words.astype(np.float64) / 256.0) + 0.5) / 16777216.0
    noise = -np.log(-np.log(uniform))
    return np.where(np.isneginf(processed), -np.inf, processed.astype(np.float64) + noise)
