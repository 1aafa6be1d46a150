"""The plain implementation checked against itself and against hand-made cases: it is the oracle of
every other test, so its own properties are pinned here."""

import math

import numpy as np
import pytest
import torch

import plain_lfm2 as plain
from plain_sampling import philox_first_word, process_logits
from tiny import TINY, make_model


@pytest.fixture(scope="module", params=["A", "B"])
def model(request, tmp_path_factory):
    folder = make_model(tmp_path_factory.mktemp(f"plain_{request.param}") / "model", request.param)
    return plain.PlainModel(folder), TINY[request.param][0]


def test_config_reading(model):
    oracle, raw = model
    assert oracle.config["head_dim"] == raw["hidden_size"] // raw["num_attention_heads"]
    assert oracle.config["ffn"] in (192, 256)
    assert len(oracle.config["kinds"]) == raw["num_hidden_layers"]


def test_causality_prefix_logits_do_not_change(model):
    oracle, raw = model
    tokens = np.random.default_rng(0).integers(0, raw["vocab_size"], size=40).tolist()
    whole = oracle.logits(tokens)
    for cut in (1, 2, 7, 23):
        assert torch.allclose(oracle.logits(tokens[:cut]), whole[:cut], atol=1e-10)
    changed = list(tokens)
    changed[30] = (changed[30] + 1) % raw["vocab_size"]
    other = oracle.logits(changed)
    assert torch.allclose(other[:30], whole[:30], atol=1e-10) and not torch.allclose(other[30:], whole[30:], atol=1e-6)


def test_rms_norm_by_hand():
    x = torch.tensor([[3.0, 4.0]], dtype=plain.DTYPE)
    out = plain.rms_norm(x, torch.tensor([2.0, 0.5], dtype=plain.DTYPE), 0.0)
    scale = 1 / math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[6.0 * scale, 2.0 * scale]], dtype=plain.DTYPE))


def test_rope_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=plain.DTYPE)
    out = plain.rope(x, torch.tensor([2]), theta=100.0)
    a0, a1 = 2.0 * 1.0, 2.0 * 100.0 ** (-0.5)
    expected = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1), 3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1)]
    assert torch.allclose(out.flatten(), torch.tensor(expected, dtype=plain.DTYPE), atol=1e-6)
    assert torch.allclose(plain.rope(x, torch.tensor([0]), 100.0), x)


def test_short_conv_by_hand():
    """arange-style weights: the current token meets the last tap, earlier tokens the earlier taps,
    zeros stand before the sequence (cf. the reference's tests/unit/modules/test_short_conv.py:71-93)."""
    D, K, T = 2, 3, 4
    cfg = {"taps": K, "conv_bias": True}
    w = {
        "p.in_proj.weight": torch.cat([torch.eye(D), torch.eye(D), torch.eye(D)]).to(plain.DTYPE),  # B = C = x = input
        "p.out_proj.weight": torch.eye(D, dtype=plain.DTYPE),
        "p.conv.weight": torch.tensor([[[1.0, 10.0, 100.0]], [[2.0, 20.0, 200.0]]], dtype=plain.DTYPE),
        "p.conv.bias": torch.tensor([0.5, -0.5], dtype=plain.DTYPE),
    }
    x = torch.tensor([[1.0, 1.0], [2.0, 0.0], [3.0, -1.0], [4.0, 2.0]], dtype=plain.DTYPE)
    out = plain.short_conv_mixer(x, w, "p", cfg)
    u = x * x
    for t in range(T):
        for ch in range(D):
            taps = w["p.conv.weight"][ch, 0]
            conv = sum(taps[k] * (u[t - (K - 1) + k, ch] if t - (K - 1) + k >= 0 else 0.0) for k in range(K)) + w["p.conv.bias"][ch]
            assert math.isclose(float(out[t, ch]), float(conv * x[t, ch]), rel_tol=1e-12)


def test_attention_is_grouped_and_causal(model):
    oracle, raw = model
    cfg = oracle.config
    index = cfg["kinds"].index("full_attention")
    prefix = f"model.layers.{index}.self_attn"
    n1 = torch.randn(9, cfg["hidden"], dtype=plain.DTYPE, generator=torch.Generator().manual_seed(1))
    positions = torch.arange(9)
    full = plain.attention_mixer(n1, oracle.weights, prefix, cfg, positions)
    # a window as long as the sequence changes nothing; a window of one attends to the token itself
    assert torch.allclose(plain.attention_mixer(n1, oracle.weights, prefix, cfg, positions, window=9), full)
    alone = plain.attention_mixer(n1, oracle.weights, prefix, cfg, positions, window=1)
    H, G, hd = cfg["heads"], cfg["groups"], cfg["head_dim"]
    v = (n1 @ oracle.weights[f"{prefix}.v_proj.weight"].T).reshape(9, G, hd)
    repeated = v.repeat_interleave(H // G, dim=1).reshape(9, H * hd)
    assert torch.allclose(alone, repeated @ oracle.weights[f"{prefix}.out_proj.weight"].T, atol=1e-10)
    assert torch.allclose(full[0], alone[0], atol=1e-10)  # the first token sees itself only


def test_greedy_continuation_is_consistent(model):
    oracle, raw = model
    produced = oracle.greedy([5, 9, 2, 11], 4)
    assert len(produced) == 4 and produced[1:] == oracle.greedy([5, 9, 2, 11, produced[0]], 3)


def test_processors_by_hand():
    logits = np.array([1.0, 3.0, 3.0, -2.0, 0.5, 2.0], np.float32)
    assert np.argmax(process_logits(logits, temperature=0.0)) == 1  # first maximum wins
    assert np.isneginf(process_logits(logits, temperature=0.0)).sum() == 5
    kept = np.isfinite(process_logits(logits, top_k=2))
    assert kept.tolist() == [False, True, True, False, False, False]
    kept = np.isfinite(process_logits(logits, top_k=1))
    assert kept.tolist() == [False, True, False, False, False, False]  # ties: lower index first
    kept = np.isfinite(process_logits(logits, banned_tokens=(1, 2), top_k=1))
    assert kept.tolist() == [False, False, False, False, False, True]
    p = np.exp(logits.astype(np.float64))
    p /= p.sum()
    kept = np.isfinite(process_logits(logits, top_p=float(p[1] + p[2] + 1e-4)))
    assert kept.tolist() == [False, True, True, False, False, True]  # the token that crosses p stays
    kept = np.isfinite(process_logits(logits, min_p=0.3))
    assert kept.tolist() == [False, True, True, False, False, True]  # exp(2-3) = 0.37 >= 0.3
    counts = np.array([0, 2, 0, 1, 0, 0], np.int32)
    out = process_logits(logits, repetition_penalty=2.0, presence_penalty=0.25, frequency_penalty=0.5, token_counts=counts)
    assert np.allclose(out, [1.0, 3.0 / 2 - 0.25 - 1.0, 3.0, -4.0 - 0.25 - 0.5, 0.5, 2.0])
    assert np.allclose(process_logits(logits, temperature=0.5), logits * 2)


def test_philox_known_answers():
    """Known-answer vectors of Philox-4x32-10 (Random123's kat_vectors): zero counter and key, and the
    all-ones counter and key."""
    assert int(philox_first_word(np.array([0]), 0, 0, 0)[0]) == 0x6627E8D5
    ones = 0xFFFFFFFF
    # counter (ones, ones, 0, 0) is not in the published table; check the avalanche property instead
    a = philox_first_word(np.arange(1000), 5, 1, 2)
    b = philox_first_word(np.arange(1000), 6, 1, 2)
    assert len(set(a.tolist())) == 1000 and (a != b).all()
    assert abs(float(np.mean(a.astype(np.float64))) / ones - 0.5) < 0.05
