"""The plain implementation against a second, independent statement of the mixers: the fixtures and
the ten-line restatements of the reference's own unit tests, written out in NumPy.

The reference's model code cannot be imported here, so these are the reference's test *formulas*, not
its outputs: ``tests/unit/modules/test_short_conv.py:21-93`` (arange weights, the split of the
in-projection into pre-convolution gate, post-convolution gate and convolution input, the windowed
einsum ``"tkc,ck->tc"`` over ``[state ; inputs]``), ``tests/unit/modules/test_convolutions.py:151-161``
(a step equals the last row of a full call, the new state is the last ``K - 1`` rows of the history) and
``tests/unit/modules/test_attention.py:84-102`` (q | k | v split, ``"thc,shc->hts"`` scores times
``head_dim ** -0.5``, causal mask, softmax, ``"hts,shc->thc"``), with the grouped heads expanded as
``lalamo/modules/token_mixers/attention.py:40-46`` does (``repeat`` along the group axis: head ``h`` reads
group ``h // (heads / groups)``).  The three chunks of the in-projection, the up and gate rows of the
feed-forward and the q, k and v rows all differ here, so a permutation of any of them in the plain
implementation fails.
"""

from __future__ import annotations

from math import prod

import numpy as np
import torch

import plain_lfm2 as plain

MODEL_DIM = 4
KERNEL_SIZE = 3


def arange_weights(shape: tuple[int, ...], offset: int = 0, divisor: float = 10.0, shift: float = 1.0) -> np.ndarray:
    """``_weights`` of the reference's tests: consecutive numbers, scaled and shifted."""
    return np.arange(offset, offset + prod(shape), dtype=np.float64).reshape(shape) / divisor - shift


def linear_reference(weights: np.ndarray, inputs: np.ndarray, output_dims: tuple[int, ...]) -> list[np.ndarray]:
    """``_linear_reference``: ``einsum("...i,oi->...o")``, then split at the cumulated output dims."""
    outputs = np.einsum("ti,oi->to", inputs, weights)
    return np.split(outputs, np.cumsum(output_dims)[:-1], axis=-1)


def conv_reference(weights: np.ndarray, biases: np.ndarray | None, inputs: np.ndarray, state: np.ndarray | None = None) -> np.ndarray:
    """``_conv_reference``: windows of ``[state ; inputs]``, ``einsum("tkc,ck->tc")``, bias."""
    channels, kernel_size = weights.shape
    if state is None:
        state = np.zeros((kernel_size - 1, channels))
    history = np.concatenate((state, inputs), axis=0)
    windows = np.stack([history[token : token + kernel_size] for token in range(inputs.shape[0])])
    result = np.einsum("tkc,ck->tc", windows, weights)
    return result if biases is None else result + biases


def short_conv_reference(in_proj, conv_weights, conv_biases, out_proj, inputs, state=None) -> np.ndarray:
    """``_reference`` of test_short_conv.py:86-93."""
    dim = inputs.shape[1]
    pre_conv_gate, post_conv_gate, conv_inputs = linear_reference(in_proj, inputs, (dim, dim, dim))
    conv_outputs = conv_reference(conv_weights, conv_biases, conv_inputs * pre_conv_gate, state)
    (outputs,) = linear_reference(out_proj, conv_outputs * post_conv_gate, (dim,))
    return outputs


def as_plain(array: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(array)).to(plain.DTYPE)


def test_short_conv_mixer_equals_the_reference_tests_restatement():
    in_proj = arange_weights((3 * MODEL_DIM, MODEL_DIM))  # three different chunks: rows 0-3 gate before, 4-7 gate after, 8-11 input
    conv_weights = arange_weights((MODEL_DIM, KERNEL_SIZE), offset=100)
    conv_biases = np.array([-0.25, 0.0, 0.25, 0.5])
    out_proj = arange_weights((MODEL_DIM, MODEL_DIM), offset=200)
    inputs = np.arange(5 * MODEL_DIM, dtype=np.float64).reshape(5, MODEL_DIM) / 10
    expected = short_conv_reference(in_proj, conv_weights, conv_biases, out_proj, inputs)
    weights = {
        "p.in_proj.weight": as_plain(in_proj),
        "p.conv.weight": as_plain(conv_weights.reshape(MODEL_DIM, 1, KERNEL_SIZE)),  # the checkpoint's [D, 1, K]
        "p.conv.bias": as_plain(conv_biases),
        "p.out_proj.weight": as_plain(out_proj),
    }
    got = plain.short_conv_mixer(as_plain(inputs), weights, "p", {"taps": KERNEL_SIZE, "conv_bias": True})
    np.testing.assert_allclose(got.numpy(), expected, rtol=1e-12, atol=1e-12)
    # The fixture's consecutive numbers make every projection an affine function of its row index; with weights that have
    # no such pattern every permutation of the three chunks gives something else, so the comparison can see their order.
    in_proj = np.cos(arange_weights((3 * MODEL_DIM, MODEL_DIM)) * 37.0)
    inputs = np.sin(np.arange(5 * MODEL_DIM, dtype=np.float64).reshape(5, MODEL_DIM) * 1.3)
    expected = short_conv_reference(in_proj, conv_weights, conv_biases, out_proj, inputs)
    weights["p.in_proj.weight"] = as_plain(in_proj)
    got = plain.short_conv_mixer(as_plain(inputs), weights, "p", {"taps": KERNEL_SIZE, "conv_bias": True})
    np.testing.assert_allclose(got.numpy(), expected, rtol=1e-12, atol=1e-12)
    # (Swapping the first and the third chunk changes nothing, since u = B * x commutes: which of the two is called the gate
    # is a matter of words.  What can be told apart is which chunk multiplies *after* the convolution.)
    for order in ([1, 0, 2], [0, 2, 1], [1, 2, 0], [2, 0, 1]):
        shuffled = np.concatenate([in_proj[MODEL_DIM * chunk : MODEL_DIM * (chunk + 1)] for chunk in order])
        other = short_conv_reference(shuffled, conv_weights, conv_biases, out_proj, inputs)
        assert not np.allclose(other, expected, rtol=1e-3)
    # without a bias, and with the taps reversed (the current token must meet the *last* tap)
    weights_no_bias = {key: value for key, value in weights.items() if key != "p.conv.bias"}
    got = plain.short_conv_mixer(as_plain(inputs), weights_no_bias, "p", {"taps": KERNEL_SIZE, "conv_bias": False})
    np.testing.assert_allclose(got.numpy(), short_conv_reference(in_proj, conv_weights, None, out_proj, inputs), rtol=1e-12, atol=1e-12)
    assert not np.allclose(short_conv_reference(in_proj, conv_weights[:, ::-1], None, out_proj, inputs), got.numpy())


def test_conv_state_carry_equals_the_whole_sequence():
    """test_convolutions.py:113-161: with the state ``[K - 1, D]`` of earlier inputs in front, a later
    portion (down to one token, the decode step) gives the rows the whole sequence gives, and the new
    state is the last ``K - 1`` rows of ``[state ; inputs]``.  The plain implementation has no state: its
    whole-sequence rows must equal the reference restatement run portion by portion."""
    in_proj = arange_weights((3 * MODEL_DIM, MODEL_DIM))
    conv_weights = arange_weights((MODEL_DIM, KERNEL_SIZE), offset=100)
    conv_biases = np.array([-0.25, 0.0, 0.25, 0.5])
    out_proj = arange_weights((MODEL_DIM, MODEL_DIM), offset=200)
    inputs = np.sin(np.arange(9 * MODEL_DIM, dtype=np.float64).reshape(9, MODEL_DIM))
    weights = {"p.in_proj.weight": as_plain(in_proj), "p.conv.weight": as_plain(conv_weights), "p.conv.bias": as_plain(conv_biases),
               "p.out_proj.weight": as_plain(out_proj)}
    whole = plain.short_conv_mixer(as_plain(inputs), weights, "p", {"taps": KERNEL_SIZE, "conv_bias": True}).numpy()
    state = np.zeros((KERNEL_SIZE - 1, MODEL_DIM))
    rows = []
    start = 0
    for size in (4, 1, 1, 3):  # a portion, two single steps (one shorter than K - 1), another portion
        portion = inputs[start : start + size]
        rows.append(short_conv_reference(in_proj, conv_weights, conv_biases, out_proj, portion, state))
        pre_conv_gate, _, conv_inputs = linear_reference(in_proj, portion, (MODEL_DIM,) * 3)
        state = np.concatenate((state, conv_inputs * pre_conv_gate), axis=0)[-(KERNEL_SIZE - 1) :]
        start += size
    np.testing.assert_allclose(np.concatenate(rows), whole, rtol=1e-12, atol=1e-12)


def attention_reference(qkv: np.ndarray, out_proj: np.ndarray, inputs: np.ndarray, heads: int, groups: int, head_dim: int) -> np.ndarray:
    """``_reference`` of test_attention.py:84-102 (no norms, no position encoding), the keys and values
    of a group repeated for its heads as attention.py:40-46 repeats them."""
    queries, keys, values = linear_reference(qkv, inputs, (heads * head_dim, groups * head_dim, groups * head_dim))
    tokens = inputs.shape[0]
    queries = queries.reshape(tokens, heads, head_dim)
    keys = np.repeat(keys.reshape(tokens, groups, head_dim), heads // groups, axis=1)
    values = np.repeat(values.reshape(tokens, groups, head_dim), heads // groups, axis=1)
    logits = np.einsum("thc,shc->hts", queries, keys) * head_dim**-0.5
    causal = np.arange(tokens)[:, None] >= np.arange(tokens)[None, :]
    logits = np.where(causal[None], logits, -np.inf)
    logits = logits - logits.max(axis=-1, keepdims=True)
    weights = np.exp(logits) / np.exp(logits).sum(axis=-1, keepdims=True)
    output = np.einsum("hts,shc->thc", weights, values).reshape(tokens, heads * head_dim)
    (outputs,) = linear_reference(out_proj, output, (out_proj.shape[0],))
    return outputs


def test_attention_mixer_equals_the_reference_tests_restatement():
    """The fixture's sizes (2 heads over 2 groups of 2 channels) and a grouped case (6 heads over 2
    groups: three query heads per key head).  The fixture has no per-head norms and no position
    encoding: the plain mixer's norm is made the identity (eps 1e12 under a scale of 1e6) and its
    rotation is switched off for the call."""
    for heads, groups, head_dim, model_dim in ((2, 2, 2, 4), (6, 2, 4, 8)):
        qkv = arange_weights(((heads + 2 * groups) * head_dim, model_dim), divisor=20.0, shift=0.5)
        if heads != groups:
            qkv = np.cos(qkv * 7.0)  # the larger case: no low-rank arange pattern, every head differs
        out_proj = arange_weights((model_dim, heads * head_dim), offset=100, divisor=20.0, shift=0.5)
        inputs = np.arange(5 * model_dim, dtype=np.float64).reshape(5, model_dim) / 10
        expected = attention_reference(qkv, out_proj, inputs, heads, groups, head_dim)
        q_rows, k_rows = heads * head_dim, groups * head_dim
        weights = {
            "p.q_proj.weight": as_plain(qkv[:q_rows]), "p.k_proj.weight": as_plain(qkv[q_rows : q_rows + k_rows]),
            "p.v_proj.weight": as_plain(qkv[q_rows + k_rows :]), "p.out_proj.weight": as_plain(out_proj),
            "p.q_layernorm.weight": torch.full((head_dim,), 1e6, dtype=plain.DTYPE),
            "p.k_layernorm.weight": torch.full((head_dim,), 1e6, dtype=plain.DTYPE),
        }
        cfg = {"heads": heads, "groups": groups, "head_dim": head_dim, "block_eps": 1e12, "theta": 10000.0}
        got = attention_without_rotation(as_plain(inputs), weights, cfg, inputs.shape[0])
        np.testing.assert_allclose(got, expected, rtol=1e-9, atol=1e-10)
        if heads != groups:
            # the other way of sharing keys among heads (head h reads group h % groups) gives something else
            tokens = inputs.shape[0]
            queries, keys, values = linear_reference(qkv, inputs, (q_rows, k_rows, k_rows))
            tiled_k = np.tile(keys.reshape(tokens, groups, head_dim), (1, heads // groups, 1))
            assert not np.allclose(tiled_k, np.repeat(keys.reshape(tokens, groups, head_dim), heads // groups, axis=1))


def attention_without_rotation(inputs: torch.Tensor, weights: dict, cfg: dict, tokens: int) -> np.ndarray:
    """plain.attention_mixer with its rotation switched off (``plain.rope`` replaced by the identity for
    the call): what is left is projection order, per-head norm, grouping, mask, softmax and out-projection."""
    original = plain.rope
    plain.rope = lambda x, positions, theta: x
    try:
        return plain.attention_mixer(inputs, weights, "p", cfg, torch.arange(tokens)).numpy()
    finally:
        plain.rope = original


def test_swiglu_takes_up_from_w3_and_gate_from_w1():
    """``lalamo/modules/mlp.py:247-258`` with the names of ``loaders/huggingface.py:1306-1308``:
    ``down(up * silu(gate))``, up = w3, gate = w1, down = w2.  Distinct up and gate rows."""
    dim, hidden = 4, 6
    w1, w3 = arange_weights((hidden, dim), divisor=7.0, shift=1.5), np.cos(arange_weights((hidden, dim), offset=50))
    w2 = arange_weights((dim, hidden), offset=300, divisor=40.0, shift=7.0)
    inputs = np.arange(3 * dim, dtype=np.float64).reshape(3, dim) / 5 - 1
    up, gate = inputs @ w3.T, inputs @ w1.T
    expected = (up * gate / (1 + np.exp(-gate))) @ w2.T
    got = plain.swiglu(as_plain(inputs), {"f.w1.weight": as_plain(w1), "f.w2.weight": as_plain(w2), "f.w3.weight": as_plain(w3)}, "f")
    np.testing.assert_allclose(got.numpy(), expected, rtol=1e-12, atol=1e-12)
    swapped = ((inputs @ w1.T) * (inputs @ w3.T) / (1 + np.exp(-(inputs @ w3.T)))) @ w2.T
    assert not np.allclose(swapped, expected)
