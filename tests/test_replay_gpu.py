"""Replays the same requests through ``bin/trace_run`` under different cuttings and compares every
logit row with the plain implementation: whole; most in one step and the last 32 tokens one by
one; portions of changing size down to one and two tokens; and mixed, up to four live requests
with so few pages that they are used again.  In 32-bit and in bfloat16, for both tiny models."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from plain_lfm2 import PlainModel
from tiny import TINY, make_model
from trace_client import TraceRun

pytestmark = pytest.mark.gpu

# Relative L2 error of a logit row, and largest elementwise error relative to the row's largest
# magnitude.  32-bit: rounding of float32 sums only.  bfloat16: activations are rounded to 8 bits of
# mantissa after every operation (the weights are bfloat16-exact in both paths).
LIMITS = {"float32": (2e-5, 1e-4), "bfloat16": (3e-2, 6e-2)}

LENGTHS = [70, 131, 45, 300, 97, 64]
PORTIONS = [2, 5, 1, 17, 3, 2, 33, 1, 1, 16, 64, 7, 2, 128]


def check_rows(got: np.ndarray, want: torch.Tensor, dtype: str, what: str) -> None:
    want_np = want.numpy()
    assert got.shape == want_np.shape, f"{what}: shape {got.shape} != {want_np.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    l2_limit, max_limit = LIMITS[dtype]
    delta = got.astype(np.float64) - want_np
    l2 = np.linalg.norm(delta, axis=-1) / np.linalg.norm(want_np, axis=-1)
    worst = np.abs(delta).max(axis=-1) / np.abs(want_np).max(axis=-1)
    bad = np.nonzero((l2 > l2_limit) | (worst > max_limit))[0]
    assert bad.size == 0, f"{what}: first wrong row {bad[0]} of {got.shape[0]} (l2 {l2[bad[0]]:.3e}, max {worst[bad[0]]:.3e}); {bad.size} rows wrong"


def pool_tokens(lengths: list[int]) -> int:
    return sum(-(-n // 64) * 64 for n in lengths)


@pytest.fixture(scope="module", params=[("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def setup(request, tmp_path_factory):
    which, dtype = request.param
    config, seed = TINY[which]
    root = tmp_path_factory.mktemp(f"replay_{which}_{dtype}")
    model_dir = make_model(root / "model", which)
    plain = PlainModel(model_dir)
    generator = np.random.default_rng(100 + seed)
    sequences = [generator.integers(0, config["vocab_size"], size=n).tolist() for n in LENGTHS]
    expected = [plain.logits(tokens) for tokens in sequences]
    # The pool holds four requests' worth at most, far less than all sequences together.
    max_tokens = pool_tokens(sorted(LENGTHS)[-4:])
    runner = TraceRun(model_dir, dtype, root / "out", max_tokens, config["vocab_size"])
    yield {"runner": runner, "sequences": sequences, "expected": expected, "dtype": dtype, "which": which}
    assert runner.close() == 0


def test_whole(setup):
    runner = setup["runner"]
    for index, (tokens, expected) in enumerate(zip(setup["sequences"], setup["expected"])):
        got = runner.step([{"id": f"w{index}", "tokens": tokens, "want": list(range(len(tokens)))}], end=[f"w{index}"])
        check_rows(got, expected, setup["dtype"], f"whole sequence {index}")


def test_prefill_then_decode_last_32(setup):
    runner = setup["runner"]
    for index, (tokens, expected) in enumerate(zip(setup["sequences"], setup["expected"])):
        name = f"d{index}"
        head = len(tokens) - 32
        got = runner.step([{"id": name, "tokens": tokens[:head], "want": [head - 1]}])
        check_rows(got, expected[head - 1 : head], setup["dtype"], f"sequence {index}, end of the prompt portion")
        for place in range(head, len(tokens)):
            last = place == len(tokens) - 1
            got = runner.step([{"id": name, "tokens": [tokens[place]], "want": [0]}], end=[name] if last else [])
            check_rows(got, expected[place : place + 1], setup["dtype"], f"sequence {index}, decoded token at position {place}")


def test_portions_of_changing_size(setup):
    runner = setup["runner"]
    for index, (tokens, expected) in enumerate(zip(setup["sequences"], setup["expected"])):
        name = f"p{index}"
        start = 0
        turn = index  # each sequence starts elsewhere in the list of sizes
        while start < len(tokens):
            size = min(PORTIONS[turn % len(PORTIONS)], len(tokens) - start)
            turn += 1
            stop = start + size
            got = runner.step([{"id": name, "tokens": tokens[start:stop], "want": list(range(size))}], end=[name] if stop == len(tokens) else [])
            check_rows(got, expected[start:stop], setup["dtype"], f"sequence {index}, portion [{start}:{stop}]")
            start = stop


def test_mixed_with_page_reuse(setup):
    """Up to four live requests; portions of some beside decoded tokens of others; a finished
    request's pages go to the next request."""
    runner = setup["runner"]
    sequences, expected = setup["sequences"], setup["expected"]
    order = [3, 0, 1, 2, 4, 5, 0, 3, 2, 1]  # ten requests over six sequences: far more tokens than the pool holds
    waiting = list(enumerate(order))
    live: dict[str, dict] = {}
    generator = np.random.default_rng(7)
    budget = pool_tokens(sorted(LENGTHS)[-4:])
    steps = 0
    while waiting or live:
        # Admit while four are not yet live and the pool (in multiples of 64 per request) has room.
        while waiting and len(live) < 4:
            number, which = waiting[0]
            held = sum(-(-len(sequences[state["which"]]) // 64) * 64 for state in live.values())
            if held + -(-len(sequences[which]) // 64) * 64 > budget:
                break
            waiting.pop(0)
            live[f"m{number}"] = {"which": which, "done": 0, "decoding": False}
        entries, checks, ended = [], [], []
        for name, state in live.items():
            tokens = sequences[state["which"]]
            left = len(tokens) - state["done"]
            if state["decoding"] or left <= 8:
                size = 1  # decode token by token near the end
                state["decoding"] = True
            else:
                size = int(min(left - 8, generator.choice([2, 3, 9, 16, 31, 50])))
            if generator.random() < 0.15 and len(live) > 1:
                continue  # this request sits the step out
            start, stop = state["done"], state["done"] + size
            want = list(range(size)) if size <= 3 else [0, size - 1]
            entries.append({"id": name, "tokens": tokens[start:stop], "want": want})
            checks.append((state["which"], [start + w for w in want]))
            state["done"] = stop
            if stop == len(tokens):
                ended.append(name)
        if not entries:
            continue
        got = runner.step(entries, end=ended)
        row = 0
        for which, places in checks:
            rows = got[row : row + len(places)]
            check_rows(rows, expected[which][places], setup["dtype"], f"mixed step {steps}, sequence {which}, positions {places}")
            row += len(places)
        for name in ended:
            del live[name]
        steps += 1
    assert steps > 20
