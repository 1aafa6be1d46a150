"""The sampling kernels against the plain NumPy restatement of the reference's processors."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from plain_sampling import gumbel_scores, process_logits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def tools():
    from lalamo_b200 import ops
    from lalamo_b200.sampling import SampleRow, SamplingPolicy, pack_rows, request_key

    return ops, SampleRow, SamplingPolicy, pack_rows, request_key


def run(tools, logits: np.ndarray, rows, counts: np.ndarray | None = None):
    ops, _, _, pack_rows, _ = tools
    device_logits = torch.from_numpy(logits).cuda()
    work = torch.empty_like(device_logits)
    out = torch.empty(logits.shape[0], dtype=torch.int32, device="cuda")
    params = torch.from_numpy(pack_rows(rows)).cuda()
    ops.sample(device_logits, work, None if counts is None else torch.from_numpy(counts).cuda(), params, out)
    return out.cpu().numpy(), work.cpu().numpy()


POLICIES = [
    dict(temperature=0.0),
    dict(temperature=0.7),
    dict(top_k=5),
    dict(top_k=1, temperature=1.3),
    dict(top_p=0.6),
    dict(top_p=0.05, temperature=0.5),
    dict(min_p=0.15, temperature=0.3),  # the LFM2 default of the reference
    dict(temperature=0.1, top_k=50, top_p=0.1),  # the LFM2.5 default
    dict(top_k=40, top_p=0.9, min_p=0.02, temperature=0.9),
    dict(banned_tokens=(0, 3, 17), top_k=3),
    dict(repetition_penalty=1.3, presence_penalty=0.4, frequency_penalty=0.2, temperature=0.8, top_p=0.95),
    dict(),
]


@pytest.mark.parametrize("vocab", [1000, 65536, 50257])
def test_processed_logits_and_draw_match_the_oracle(tools, vocab):
    _, SampleRow, SamplingPolicy, _, request_key = tools
    generator = np.random.default_rng(vocab)
    logits = (generator.standard_normal((len(POLICIES), vocab)) * 3).astype(np.float32)
    logits[:, 100:104] = logits[:, 100:101]  # ties
    logits[2, :8] = logits[2].max() + 1.0  # ties across the top-k boundary: lower indices win
    counts = np.zeros((len(POLICIES) + 2, vocab), np.int32)
    counted = generator.integers(0, vocab, size=300)
    np.add.at(counts[12], counted, 1)
    rows = []
    for index, options in enumerate(POLICIES):
        policy = SamplingPolicy.init(**options)
        rows.append(SampleRow(policy, request_key(99, index), draw=index * 3, count_slot=12))
    tokens, work = run(tools, logits, rows, counts)
    for index, options in enumerate(POLICIES):
        policy = rows[index].policy
        expected = process_logits(
            logits[index], temperature=policy.temperature, top_k=policy.top_k, top_p=policy.top_p, min_p=policy.min_p,
            banned_tokens=policy.banned_tokens, repetition_penalty=policy.repetition_penalty, presence_penalty=policy.presence_penalty,
            frequency_penalty=policy.frequency_penalty, token_counts=counts[12] if policy.has_count_penalties else None)
        if policy.temperature == 0.0:
            assert tokens[index] == int(np.argmax(expected)), options
            continue
        kept, kept_expected = np.isfinite(work[index]), np.isfinite(expected)
        differing = np.nonzero(kept != kept_expected)[0]
        if differing.size:  # only tokens exactly at the top-p boundary may differ (summation order)
            assert policy.top_p is not None and differing.size <= 2, (options, differing[:10])
        both = kept & kept_expected
        assert np.allclose(work[index][both], expected[both], rtol=1e-6, atol=1e-6), options
        scores = gumbel_scores(np.where(kept, work[index], -np.inf).astype(np.float32), rows[index].key, rows[index].draw)
        assert kept[tokens[index]], options
        assert scores[tokens[index]] >= scores.max() - 1e-4, options  # the drawn token has the best perturbed score


def test_top_k_ties_keep_lower_indices(tools):
    _, SampleRow, SamplingPolicy, _, request_key = tools
    logits = np.full((1, 3000), -1.0, np.float32)
    logits[0, [5, 900, 901, 2500, 2999]] = 2.0
    tokens, work = run(tools, logits, [SampleRow(SamplingPolicy.init(top_k=3), request_key(0, 0), 0)])
    assert np.nonzero(np.isfinite(work[0]))[0].tolist() == [5, 900, 901]
    assert tokens[0] in (5, 900, 901)


def test_draws_follow_the_distribution_and_the_key(tools):
    _, SampleRow, SamplingPolicy, _, request_key = tools
    vocab, draws = 64, 4000
    logits = np.tile(np.linspace(-2, 2, vocab, dtype=np.float32), (draws, 1))
    policy = SamplingPolicy.init(temperature=1.0)
    rows = [SampleRow(policy, request_key(1, 0), draw) for draw in range(draws)]
    tokens, _ = run(tools, logits, rows)
    again, _ = run(tools, logits, rows)
    assert (tokens == again).all()  # same key and draw number, same token
    other, _ = run(tools, logits, [SampleRow(policy, request_key(1, 1), draw) for draw in range(draws)])
    assert (tokens != other).mean() > 0.5
    frequencies = np.bincount(tokens, minlength=vocab) / draws
    probabilities = np.exp(logits[0].astype(np.float64))
    probabilities /= probabilities.sum()
    assert np.abs(frequencies - probabilities).max() < 4 * np.sqrt(probabilities.max() / draws)


def test_argmax_and_count_updates(tools):
    ops = tools[0]
    generator = np.random.default_rng(5)
    logits = generator.standard_normal((7, 50257)).astype(np.float32)
    logits[3, [11, 40000]] = 9.0
    out = torch.empty(7, dtype=torch.int32, device="cuda")
    ops.argmax(torch.from_numpy(logits).cuda(), out)
    assert out.cpu().tolist() == np.argmax(logits, axis=1).tolist() and out[3].item() == 11  # several blocks per row
    small = logits[:, :1000].copy()
    small[2, [7, 600]] = 9.0
    ops.argmax(torch.from_numpy(small).cuda(), out)
    assert out.cpu().tolist() == np.argmax(small, axis=1).tolist() and out[2].item() == 7  # one block per row
    counts = torch.zeros(4, 100, dtype=torch.int32, device="cuda")
    ops.update_counts(counts, torch.tensor([2, 0, -1], dtype=torch.int32).cuda(), torch.tensor([5, 7, 9], dtype=torch.int32).cuda(),
                      torch.tensor([-1, 7, 9], dtype=torch.int32).cuda())
    host = counts.cpu()
    assert host[2, 5] == 1 and host.sum() == 1  # slot 0: +1 and -1 on token 7; the row without a slot is skipped
