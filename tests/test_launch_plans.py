"""The launch plans that the op wrappers compute on the host are functions of sizes alone: they must
cover the work for every size, and they must not depend on anything but the sizes (a recorded CUDA
graph is replayed for every step of its shape).  No GPU needed."""

from __future__ import annotations

import random

import pytest


@pytest.fixture(scope="module")
def ops():
    from lalamo_b200 import ops as module

    return module


def test_decode_attention_plan_covers_every_block(ops):
    generator = random.Random(4)
    for _ in range(500):
        tokens = generator.choice([1, 2, 8, 16, 33, 64, 200])
        groups = generator.choice([1, 2, 3, 8])
        heads = groups * generator.choice([1, 2, 4, 7, 20])
        context = generator.choice([1, 15, 16, 17, 100, 4096, 4097, 16384, 100_000])
        window = generator.choice([None, None, 1, 16, 100, 5000])
        head_dim = generator.choice([16, 64, 80, 128])
        splits, per_split = ops.decode_attention_plan(tokens, heads, groups, context, window, head_dim, resident_ctas=148 * 4)
        span = min(context, window + 15) if window else context
        blocks = span // 16 + 1  # the visible keys may straddle one block more than their count
        assert splits >= 1 and per_split >= 1
        assert splits * per_split >= blocks, "some block of keys would belong to no split"
        assert (splits - 1) * per_split < blocks, "a split without any block"
        assert (splits, per_split) == ops.decode_attention_plan(tokens, heads, groups, context, window, head_dim, resident_ctas=148 * 4)


def test_decode_attention_plan_splits_long_contexts_of_few_tokens(ops):
    one, _ = ops.decode_attention_plan(1, 32, 8, 16384, None, resident_ctas=592)
    many, _ = ops.decode_attention_plan(256, 32, 8, 16384, None, resident_ctas=592)
    assert one > many >= 1  # few tokens: the keys are cut so that every SM has work; many tokens fill the GPU by themselves
    assert ops.decode_attention_plan(8, 32, 8, 40, None, resident_ctas=592)[0] == 1  # a handful of blocks is not worth cutting


def test_tcgen05_slices(ops):
    generator = random.Random(5)
    for _ in range(500):
        tokens = generator.choice([1, 8, 17, 32, 33, 64, 100, 128, 129, 300, 512, 2048])
        rows = generator.choice([64, 100, 2048, 3072, 6144, 16384, 65536])
        width = generator.choice([8, 64, 136, 2048, 4096, 8192, 16384])
        slices = ops.tcgen05_slices(tokens, rows, width, sms=148)
        blocks = -(-width // 64)
        assert slices >= 1
        assert slices == 1 or slices <= blocks // 4, "a slice of fewer than four 64-column blocks"
    # A product whose tiles fill the GPU is not cut, nor is one above 128 tokens whose slices would be shorter than 16 blocks.
    assert ops.tcgen05_slices(64, 16384, 2048, sms=148) == 1
    assert ops.tcgen05_slices(2048, 6144, 2048, sms=148) == 1
    assert ops.tcgen05_slices(2048, 1024, 1024, sms=148) == 1
    # Few tiles of 256 tokens and a long K: slices until the tiles fill the SMs.
    assert ops.tcgen05_slices(2048, 1024, 4608, sms=148) == 2
    assert ops.tcgen05_slices(512, 2048, 8192, sms=148) == 4
    assert ops.tcgen05_slices(512, 2048, 2048, sms=148) == 2
    # The down-projection of a decode batch (16 tiles of 128 rows, K = 8192) is.
    assert ops.tcgen05_slices(64, 2048, 8192, sms=148) > 1
    assert ops.tcgen05_slices(512, 2048, 8192, sms=148) > 1


def test_when_prefill_attention_tiles_are_shared_by_two_ctas():
    """The attention part's rule: two CTAs per tile with fewer CTAs than SMs, and in long-context steps that are never
    replayed where twice the CTAs fill the resident slots better; never a context-dependent answer for a step that
    could be replayed."""
    from lalamo_b200.parts.attention import SHARED_TILE_KEYS, shared_tile_keys
    from lalamo_b200.parts.base import REPLAY_MAX_TOKENS

    sms = 148
    # 512 tokens of one request, 32 heads over 8: 16 tiles x 8 = 128 CTAs
    assert shared_tile_keys(16, 32, 8, sms, 512, (512,), (0,)) == SHARED_TILE_KEYS
    assert shared_tile_keys(16, 32, 8, sms, 512, (512,), (16000,)) == SHARED_TILE_KEYS
    # 1,024 tokens: 256 CTAs on 444 slots; twice as many would need a second, nearly empty round
    assert shared_tile_keys(32, 32, 8, sms, 1024, (1024,), (15000,)) == 0
    # 2,048 tokens: 512 CTAs need two rounds; paired, 1,024 need 2.3: only where the tiles are long
    assert shared_tile_keys(64, 32, 8, sms, 2048, (2048,), (0,)) == 0
    assert shared_tile_keys(64, 32, 8, sms, 2048, (2048,), (14336,)) == SHARED_TILE_KEYS
    # a whole long prompt in one step: thousands of CTAs fill the slots either way
    assert shared_tile_keys(512, 32, 8, sms, 16384, (16384,), (0,)) == 0
    # replayable steps get the same answer whatever the contexts
    for tiles in range(1, REPLAY_MAX_TOKENS // 32 + 1):
        answers = {shared_tile_keys(tiles, 32, 8, sms, tiles * 32, (tiles * 32,), (context,)) for context in (0, 5000, 100000)}
        assert len(answers) == 1
    # more query heads per K/V head than fit a CTA's 128 rows with 32 tokens: more CTAs per tile record
    assert shared_tile_keys(4, 40, 2, sms, 128, (128,), (0,)) == SHARED_TILE_KEYS
