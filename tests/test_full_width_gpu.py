"""The layer sizes of the three published shapes (LFM2-1.2B: width 2048, 32 query heads over 8 K/V heads of
64, feed-forward 8192; LFM2-350M: 1024, 16 over 8, 4608; LFM2-700M: 1536, 24 over 8, 6912; vocabulary 65536,
three taps) with three or four layers and random weights, replayed through ``bin/trace_run`` in 32-bit and in
bfloat16 and compared with the plain implementation.

The tiny models never reach the kernels that serving at these sizes uses: the walking tcgen05 product
(more than 128 tokens, several tiles per CTA, the gated epilogue over thousands of hidden rows), the one-tile
tcgen05 product (17 to 128 tokens, and the LM head and up/gate products for few tokens), the skinny
products at their real widths, and attention with two, three and four query heads per K/V head at head size 64."""

from __future__ import annotations

import numpy as np
import pytest

from lalamo_b200.weights import write_random_model
from plain_lfm2 import PlainModel
from test_replay_gpu import FLOAT32_LIMITS, RowChecker, bfloat16_limits
from trace_client import TraceRun

pytestmark = pytest.mark.gpu

def shape(hidden: int, heads: int, block_ff_dim: int, kinds: list[str]) -> dict:
    return {
        "architectures": ["Lfm2ForCausalLM"],
        "model_type": "lfm2",
        "vocab_size": 65536,
        "hidden_size": hidden,
        "num_hidden_layers": len(kinds),
        "num_attention_heads": heads,
        "num_key_value_heads": 8,
        "layer_types": kinds,
        "block_auto_adjust_ff_dim": True,
        "block_ff_dim": block_ff_dim,
        "block_ffn_dim_multiplier": 1.0,
        "block_multiple_of": 256,
        "conv_L_cache": 3,
        "conv_bias": False,
        "rope_theta": 1000000.0,
        "block_norm_eps": 1e-5,
        "norm_eps": 1e-5,
        "tie_embedding": True,
        "eos_token_id": 7,
    }


# The layer sizes of the three published shapes, a few layers each: width 2048 with four query heads per K/V
# head and a feed-forward of 8192 (1.2B); width 1024, two per K/V head, 4608 (350M); width 1536, three per K/V
# head, 6912 (700M: widths and row counts that are no multiples of 256 tokens' worth of tiles, and 32 tokens x 3
# heads in a 128-row attention tile).
SHAPES = {
    "1.2b": shape(2048, 32, 12288, ["conv", "conv", "full_attention", "conv"]),
    "350m": shape(1024, 16, 6656, ["conv", "full_attention", "conv"]),
    "700m": shape(1536, 24, 10240, ["full_attention", "conv", "conv"]),
}
FULL_WIDTH = SHAPES["1.2b"]

LENGTHS = [330, 60]


@pytest.fixture(scope="module", params=list(SHAPES))
def full_width(request, tmp_path_factory):
    root = tmp_path_factory.mktemp(f"full_width_{request.param}")
    # A spread of 0.02 as trained models have it: at this width a larger one saturates the softmax.
    model_dir = write_random_model(root / "model", SHAPES[request.param], seed=5, std=0.02, dtype="bfloat16")
    plain = PlainModel(model_dir)
    generator = np.random.default_rng(11)
    sequences = [generator.integers(0, FULL_WIDTH["vocab_size"], size=n).tolist() for n in LENGTHS]
    expected = [plain.logits(tokens) for tokens in sequences]
    return {"root": root, "model_dir": model_dir, "plain": plain, "sequences": sequences, "expected": expected}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_full_width_replay(full_width, dtype):
    sequences, expected = full_width["sequences"], full_width["expected"]
    limits = FLOAT32_LIMITS if dtype == "float32" else bfloat16_limits(full_width["plain"], sequences[1:], expected[1:])
    runner = TraceRun(full_width["model_dir"], dtype, full_width["root"] / f"out_{dtype}", 512, FULL_WIDTH["vocab_size"])
    checker = RowChecker(limits)
    long, short = sequences
    # The long prompt whole in one step (the walking product), a few rows wanted.
    places = [0, 1, 127, 128, 255, 256, 300, 329]
    got = runner.step([{"id": "whole", "tokens": long, "want": places}], end=["whole"])
    checker.add(got, expected[0][places], "long prompt in one step")
    # Again in portions that meet the one-tile product (100, 40, 17 tokens) and the skinny one (9, 2),
    # beside the short request: first its prompt, then its last tokens one by one.
    start, head = 0, len(short) - 6
    for turn, size in enumerate([100, 40, 17, 150, 9, 2, 12]):
        stop = start + size
        entries = [{"id": "cut", "tokens": long[start:stop], "want": [0, size - 1]}]
        checks = [(0, [start, stop - 1])]
        if turn == 0:
            entries.append({"id": "short", "tokens": short[:head], "want": [head - 1]})
            checks.append((1, [head - 1]))
        elif turn <= 6:
            place = head + turn - 1
            entries.append({"id": "short", "tokens": [short[place]], "want": [0]})
            checks.append((1, [place]))
        got = runner.step(entries, end=(["short"] if turn == 6 else []) + (["cut"] if stop == len(long) else []))
        row = 0
        for which, wanted in checks:
            checker.add(got[row : row + len(wanted)], expected[which][wanted], f"step {turn}, sequence {which}, positions {wanted}")
            row += len(wanted)
        start = stop
    assert start == len(long)
    checker.finish()
    assert runner.close() == 0


def test_twenty_requests_decode_together(full_width):
    """More requests than the weight-streaming kernels take in one step: their prompts in one step of twenty
    portions, then decode steps of twenty single tokens (the one-tile product in K slices, the convolution that adds
    the slices itself and updates twenty states, the norms that add the other products' slices, attention without a
    merge), with CUDA graphs on so that the later steps are replays; every row against the plain implementation."""
    from lalamo_b200.engine import Engine, EngineConfig, StepEntry

    plain = full_width["plain"]
    generator = np.random.default_rng(23)
    sequences = [generator.integers(0, FULL_WIDTH["vocab_size"], size=int(n)).tolist() for n in generator.integers(6, 27, size=20)]
    expected = [plain.logits(tokens) for tokens in sequences]
    checker = RowChecker(bfloat16_limits(plain, sequences[:4], expected[:4]))
    engine = Engine.load(full_width["model_dir"], EngineConfig(dtype="bfloat16", max_tokens=20 * 64, max_requests=20, cuda_graphs=True))
    decoded = 4
    for index in range(20):
        engine.admit(index)
    heads = [len(tokens) - decoded for tokens in sequences]
    logits = engine.step([StepEntry(index, tokens[:head], [head - 1]) for index, (tokens, head) in enumerate(zip(sequences, heads))])
    for index, head in enumerate(heads):
        checker.add(logits[index : index + 1].cpu().numpy(), expected[index][head - 1 : head], f"prompt {index}")
    for step in range(decoded):
        logits = engine.step([StepEntry(index, [tokens[head + step]], [0]) for index, (tokens, head) in enumerate(zip(sequences, heads))]).cpu().numpy()
        for index, head in enumerate(heads):
            checker.add(logits[index : index + 1], expected[index][head + step : head + step + 1], f"decode step {step}, request {index}")
    assert engine.executor.graph_replays >= decoded - 1
    checker.finish()
    engine.executor.check_status()
    for index in range(20):
        engine.release(index)
    engine.cache.check()
