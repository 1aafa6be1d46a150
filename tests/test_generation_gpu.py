"""Generation through the Python entry point and the command line, compared with the plain
implementation: greedy tokens; sampled tokens under chunked prefill mixed with decoding; streaming;
preemption when the cache is small; long decoding; the first tokens of a sequence."""

from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from plain_lfm2 import PlainModel
from plain_sampling import gumbel_scores, process_logits
from tiny import TINY, make_model

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("generation")
    return {which: make_model(root / which, which) for which in "AB"}


def prompts_for(which: str, lengths: list[int]) -> list[list[int]]:
    generator = np.random.default_rng(40 + len(lengths))
    return [generator.integers(0, TINY[which][0]["vocab_size"], size=n).tolist() for n in lengths]


def test_greedy_generation_equals_the_plain_implementation(models):
    from lalamo_b200 import GenerationConfig, LanguageModel

    model = LanguageModel.load(models["A"], dtype="float32", max_tokens=1024, max_requests=4)
    plain = PlainModel(models["A"])
    prompts = prompts_for("A", [1, 7, 16, 33])
    config = GenerationConfig(temperature=0.0)
    produced = model.generate_tokens(prompts, config, max_output_length=16, eos_token_ids=[])
    for prompt, tokens in zip(prompts, produced):
        assert tokens == plain.greedy(prompt, 16)
    # padded rows with their true lengths give the same tokens
    width = max(len(p) for p in prompts)
    padded = [p + [0] * (width - len(p)) for p in prompts]
    assert model.generate_tokens(padded, config, [len(p) for p in prompts], max_output_length=16, eos_token_ids=[]) == produced
    # a stop token ends the sequence and stays in the output
    stop = produced[2][5]
    first = produced[2].index(stop)
    assert model.generate_tokens([prompts[2]], config, max_output_length=16, eos_token_ids=[stop]) == [produced[2][: first + 1]]
    # streaming yields the same tokens one by one
    assert list(model.stream_tokens(prompts[3], config, max_output_length=16, eos_token_ids=[])) == produced[3]
    model.engine.executor.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_a_step_ahead_of_the_results_changes_no_token(models, dtype):
    """The loop that launches a step before the ids of the step before have reached the host (they go from
    the sampler to the next step's description on the device) against the loop that awaits every step:
    sampled tokens with stop tokens and different lengths, recorded graphs and all."""
    from lalamo_b200 import GenerationConfig, LanguageModel
    from lalamo_b200.engine.generation import Generator

    model = LanguageModel.load(models["B"], dtype=dtype, max_tokens=2048, max_requests=6)
    prompts = prompts_for("B", [3, 40, 9, 70, 21])
    config = GenerationConfig(temperature=0.8, top_k=20)
    lengths = [40, 12, 33, 25, 40]

    def run(run_ahead: bool, stops: list[frozenset]) -> tuple[dict, Generator]:
        generator = Generator(model.engine, seed=11, run_ahead=run_ahead)
        requests = [generator.add(prompt, config.default_policy(), stop, length, key_number=index)
                    for index, (prompt, stop, length) in enumerate(zip(prompts, stops, lengths))]
        while generator.has_work():
            generator.step()
        generator.close()
        assert model.engine.cache.free_pages() == model.engine.cache.num_pages
        return {index: (list(request.generated), request.finish_reason) for index, request in enumerate(requests)}, generator

    free, _ = run(False, [frozenset()] * 5)
    stops = [frozenset([free[0][0][17]]), frozenset(), frozenset([free[2][0][30], free[2][0][8]]), frozenset([free[3][0][24]]), frozenset()]
    awaited, _ = run(False, stops)
    ahead, generator = run(True, stops)
    assert ahead == awaited
    assert [reason for _, reason in ahead.values()].count("stop") >= 3
    assert generator.steps_run_ahead >= 30
    model.engine.executor.check_status()


def test_short_portions_at_the_end_of_a_long_context_share_their_tiles(tmp_path):
    """Head size 64 in bfloat16: after 1,200 tokens in one step, portions of 40, 2 and 60 tokens see 19 to 21 tiles of
    64 keys; such launches have few tiles, so each tile is worked on by two CTAs that merge their halves.  Every
    logit row of the portions against the plain implementation, and the same portions with the sharing switched off."""
    from plain_lfm2 import PlainModel
    from test_replay_gpu import RowChecker, bfloat16_limits
    from tiny import make_model

    from lalamo_b200.engine import Engine, EngineConfig, StepEntry
    from lalamo_b200.parts import attention

    model_dir = make_model(tmp_path / "c", "C")
    plain = PlainModel(model_dir)
    vocab = TINY["C"][0]["vocab_size"]
    tokens = np.random.default_rng(23).integers(0, vocab, size=1302).tolist()
    want = plain.logits(tokens)
    limits = bfloat16_limits(plain, [tokens[:200]], [want[:200]])
    engine = Engine.load(model_dir, EngineConfig(dtype="bfloat16", max_tokens=2048, max_requests=2))
    rows = {}
    for shared in (True, False):
        attention.SHARED_TILE_KEYS = 512 if shared else 1 << 30
        checker = RowChecker(limits)
        engine.admit("long")
        got = engine.step([StepEntry("long", tokens[:1200], [1199])])
        checker.add(got.cpu().numpy(), want[1199:1200], "the long portion's last row")
        collected = []
        for start, stop in ((1200, 1240), (1240, 1242), (1242, 1302)):
            got = engine.step([StepEntry("long", tokens[start:stop], list(range(stop - start)))])
            checker.add(got.cpu().numpy(), want[start:stop], f"portion [{start}:{stop}] after {start} tokens")
            collected.append(got.cpu())
        checker.finish()
        engine.release("long")
        rows[shared] = torch.cat(collected)
    attention.SHARED_TILE_KEYS = 512
    engine.executor.check_status()
    # the two ways of cutting the keys differ by rounding only
    assert float((rows[True] - rows[False]).abs().max()) < 0.05 * float(rows[False].abs().max())
    assert not torch.equal(rows[True], rows[False])  # and the sharing did happen


def test_greedy_bfloat16_follows_its_own_logits(models):
    """In bfloat16 a near-tie may resolve differently from float64, so each token is checked against the
    oracle's logits for the engine's own prefix: it must be (nearly) the best one."""
    from lalamo_b200 import GenerationConfig, LanguageModel

    model = LanguageModel.load(models["B"], dtype="bfloat16", max_tokens=1024, max_requests=4)
    plain = PlainModel(models["B"])
    prompts = prompts_for("B", [5, 40, 64])
    produced = model.generate_tokens(prompts, GenerationConfig(temperature=0.0), max_output_length=12, eos_token_ids=[])
    for prompt, tokens in zip(prompts, produced):
        logits = plain.logits(prompt + tokens)
        for step, token in enumerate(tokens):
            row = logits[len(prompt) + step - 1]
            assert row[token] >= row.max() - 0.1 * (row.max() - row.mean()), (step, token)


def test_sampled_generation_chunked_and_mixed(models):
    """Temperature 0.8 at a fixed seed, prompts read in portions of 8 beside decoding requests: every
    token must be the one the oracle draws from the plain logits with the same key and draw number."""
    from lalamo_b200 import GenerationConfig, LanguageModel
    from lalamo_b200.sampling import request_key

    model = LanguageModel.load(models["B"], dtype="float32", max_tokens=1024, max_requests=3, max_batch_tokens=24)
    plain = PlainModel(models["B"])
    prompts = prompts_for("B", [5, 40, 64])
    config = GenerationConfig(temperature=0.8, top_k=200, min_p=0.01)
    sequences = {s.index: s for s in model.generate_tokens_many(prompts, config, max_output_length=10, eos_token_ids=[], seed=11, chunk_size=8)}
    assert model.engine.executor.steps_run > 10  # portions and decoding did share steps
    for index, prompt in enumerate(prompts):
        tokens = sequences[index].token_ids
        assert len(tokens) == 10 and sequences[index].finish_reason == "length"
        logits = plain.logits(prompt + tokens).numpy().astype(np.float32)
        for draw, token in enumerate(tokens):
            processed = process_logits(logits[len(prompt) + draw - 1], temperature=0.8, top_k=200, min_p=0.01)
            scores = gumbel_scores(processed, request_key(11, index), draw)
            assert scores[token] >= scores.max() - 1e-3, (index, draw)
    # the same seed gives the same tokens however the prompts are cut into portions
    again = {s.index: s.token_ids for s in model.generate_tokens_many(prompts, config, max_output_length=10, eos_token_ids=[], seed=11)}
    assert all(again[i] == sequences[i].token_ids for i in range(3))  # other portion sizes, same tokens


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_on_a_small_cache_keeps_the_tokens(models, dtype):
    """A pool too small for the five requests: some are preempted and read again.  Freed pages and slots
    are overwritten with NaN, and recorded decode graphs are replayed for other requests than the ones
    they were recorded with (the batch shrinks and grows as requests are preempted and come back)."""
    from lalamo_b200 import GenerationConfig, LanguageModel

    prompts = prompts_for("A", [30, 21, 40, 17, 9])
    config = GenerationConfig(temperature=0.0)
    tight = LanguageModel.load(models["A"], dtype=dtype, max_tokens=160, max_requests=8, page_size=16, poison_freed=True)
    results = {s.index: s for s in tight.generate_tokens_many(prompts, config, max_output_length=40, eos_token_ids=[])}
    assert sum(s.preemptions for s in results.values()) > 0
    assert tight.engine.executor.graph_replays > 0 and tight.engine.executor.graph_rebinds > 0
    if dtype == "float32":
        roomy = LanguageModel.load(models["A"], dtype=dtype, max_tokens=2048, max_requests=8)
        expected = roomy.generate_tokens(prompts, config, max_output_length=40, eos_token_ids=[])
        assert [results[i].token_ids for i in range(5)] == expected
    else:
        # a near-tie may fall the other way in bfloat16: every token must be (nearly) the best by the oracle's
        # logits for the engine's own prefix
        plain = PlainModel(models["A"])
        for index, prompt in enumerate(prompts):
            tokens = results[index].token_ids
            assert len(tokens) == 40
            logits = plain.logits(prompt + tokens)
            for step, token in enumerate(tokens):
                row = logits[len(prompt) + step - 1]
                assert row[token] >= row.max() - 0.1 * (row.max() - row.mean()), (index, step, token)
    tight.engine.cache.check()
    assert tight.engine.cache.free_pages() == 10 and not tight.engine.cache.requests
    tight.engine.executor.check_status()


def test_a_stream_that_is_abandoned_leaves_nothing_behind(models):
    """The consumer stops after two tokens: the request's pages and slot go back, and the next call on the
    same model gives what a fresh engine gives."""
    from lalamo_b200 import GenerationConfig, LanguageModel

    config = GenerationConfig(temperature=0.0)
    prompts = prompts_for("A", [12, 25])
    fresh = LanguageModel.load(models["A"], dtype="float32", max_tokens=512, max_requests=4)
    expected = fresh.generate_tokens(prompts, config, max_output_length=10, eos_token_ids=[])
    model = LanguageModel.load(models["A"], dtype="float32", max_tokens=512, max_requests=4)
    pages, slots = model.engine.cache.free_pages(), model.engine.cache.slots.free_count
    taken = []
    for token in model.stream_tokens(prompts[0], config, max_output_length=10, eos_token_ids=[]):
        taken.append(token)
        if len(taken) == 2:
            break
    assert taken == expected[0][:2]  # the abandoned iterator is closed as the loop is left
    many = model.generate_tokens_many(prompts, config, max_output_length=10, eos_token_ids=[])
    first = next(many)
    many.close()  # stops with one request still running
    assert first.token_ids == expected[first.index]
    model.engine.cache.check()
    assert model.engine.cache.free_pages() == pages and model.engine.cache.slots.free_count == slots and not model.engine.cache.requests
    assert model.generate_tokens(prompts, config, max_output_length=10, eos_token_ids=[]) == expected
    # two interleaved calls on one model do not collide on request names
    left = model.generate_tokens_many(prompts[:1], config, max_output_length=10, eos_token_ids=[])
    right = model.generate_tokens_many(prompts[1:], config, max_output_length=10, eos_token_ids=[])
    assert next(left).token_ids == expected[0] and next(right).token_ids == expected[1]
    left.close(), right.close()
    model.engine.cache.check()
    assert not model.engine.cache.requests


def test_penalties_use_per_request_counts(models):
    """Repetition/presence/frequency penalties: the tokens equal a teacher-forced oracle that counts the
    prompt and the generated tokens (lalamo/sampling.py:94-177)."""
    from lalamo_b200 import GenerationConfig, LanguageModel

    model = LanguageModel.load(models["A"], dtype="float32", max_tokens=512, max_requests=4)
    plain = PlainModel(models["A"])
    prompts = prompts_for("A", [12, 25])
    config = GenerationConfig(temperature=0.0, repetition_penalty=1.5, presence_penalty=0.3, frequency_penalty=0.2)
    produced = model.generate_tokens(prompts, config, max_output_length=12, eos_token_ids=[])
    vocab = TINY["A"][0]["vocab_size"]
    for prompt, tokens in zip(prompts, produced):
        logits = plain.logits(prompt + tokens).numpy().astype(np.float32)
        for step, token in enumerate(tokens):
            counts = np.bincount(prompt + tokens[:step], minlength=vocab).astype(np.int32)
            processed = process_logits(logits[len(prompt) + step - 1], temperature=0.0, repetition_penalty=1.5, presence_penalty=0.3,
                                       frequency_penalty=0.2, token_counts=counts)
            assert token == int(np.argmax(processed)), step


def test_long_decoding_and_first_tokens(models):
    """600 tokens decoded one by one after a one-token prompt: positions 0, 1, 2 ... (the first tokens of
    a sequence, before the convolution state is full) and many page and chunk edges."""
    from lalamo_b200.engine import Engine, EngineConfig, StepEntry

    plain = PlainModel(models["B"])
    tokens = np.random.default_rng(8).integers(0, 1000, size=600).tolist()
    expected = plain.logits(tokens)
    engine = Engine.load(models["B"], EngineConfig(dtype="float32", max_tokens=640, max_requests=2))
    engine.admit("long")
    rows = []
    for token in tokens:
        rows.append(engine.step([StepEntry("long", [token], [0])])[0].cpu())
    got = torch.stack(rows).double()
    error = (got - expected).norm(dim=-1) / expected.norm(dim=-1)
    assert error.max() < 2e-5, f"first wrong position {int((error >= 2e-5).nonzero()[0])}"
    engine.executor.check_status()


def test_a_wait_that_runs_out_is_reported_and_the_engine_goes_on(models):
    """The tcgen05 kernels bound every barrier wait and report a wait that gave up in the engine's
    status word.  Here the same wait runs out on a barrier that nothing completes (1 ms, no product is
    disturbed): the status check raises, and the engine steps on afterwards with the right logits."""
    from lalamo_b200 import ops
    from lalamo_b200.engine import Engine, EngineConfig, StepEntry

    engine = Engine.load(models["A"], EngineConfig(dtype="bfloat16", max_tokens=128, max_requests=2))
    engine.admit("r")
    tokens = [5, 9, 2, 7, 11, 3]
    first = engine.step([StepEntry("r", tokens, [len(tokens) - 1])]).cpu()
    engine.executor.check_status()
    ops.tcgen05_wait_probe(engine.runtime.status, nanoseconds=1_000_000)
    with pytest.raises(RuntimeError, match="bounded wait gave up"):
        engine.executor.check_status()
    engine.executor.check_status()  # reported once, then cleared
    engine.release("r")
    engine.admit("again")
    second = engine.step([StepEntry("again", tokens, [len(tokens) - 1])]).cpu()
    assert torch.equal(first, second)
    with pytest.raises(ops.KernelError):
        ops.tcgen05_wait_probe(engine.runtime.status, nanoseconds=10**9)  # longer than a probe may take


def test_command_line(models, tmp_path):
    prompt_file = tmp_path / "prompts.txt"
    prompt_file.write_text("5 9 2 11\n7,7,7\n")
    command = [sys.executable, "-m", "lalamo_b200", "generate", str(models["A"]), "--prompt-ids-file", str(prompt_file), "--max-tokens", "6",
               "--temperature", "0", "--dtype", "float32", "--max-cache-tokens", "512", "--stats"]
    result = subprocess.run(command, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr
    lines = [json.loads(line) for line in result.stdout.splitlines() if line.startswith("{")]
    plain = PlainModel(models["A"])
    stop = TINY["A"][0]["eos_token_id"]
    for line, prompt in zip(lines, ([5, 9, 2, 11], [7, 7, 7])):
        expected = plain.greedy(prompt, 6)
        if stop in expected:
            expected = expected[: expected.index(stop) + 1]
        assert line["token_ids"] == expected
    assert "steps run" in result.stderr
    listing = subprocess.run([sys.executable, "-m", "lalamo_b200", "list-models", "--plain"], cwd=ROOT, capture_output=True, text=True, timeout=120)
    assert "LiquidAI/LFM2-1.2B" in listing.stdout.split()


def run_generate(arguments: list[str]) -> tuple[list[dict], str]:
    result = subprocess.run([sys.executable, "-m", "lalamo_b200", "generate", *arguments], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr
    return [json.loads(line) for line in result.stdout.splitlines() if line.startswith("{")], result.stderr


def test_command_line_random_weights_chunks_text_and_default_options(models, tmp_path):
    """`generate` with weights made in memory from a folder that holds only config.json, prompts read in
    portions of --chunk-size, a text prompt through tokenizer.json, and the registry's default options."""
    from tokenizers import Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace

    from tiny import TEST_STD

    config, seed = TINY["A"]
    bare = tmp_path / "bare"
    bare.mkdir()
    (bare / "config.json").write_text(json.dumps(config))
    plain = PlainModel(models["A"])  # the folder written from the same configuration, seed and spread
    prompt = [5, 9, 2, 11, 40, 41, 42, 43, 44, 45, 46, 47, 48, 300, 301, 302, 303, 17, 19, 23, 29, 31]
    common = ["--random-weights", str(seed), "--std", str(TEST_STD), "--dtype", "float32", "--max-cache-tokens", "512", "--temperature", "0", "--max-tokens", "6"]
    lines, errors = run_generate([str(bare), "--prompt-ids", ",".join(map(str, prompt)), "--chunk-size", "5", "--stats", *common])
    expected = plain.greedy(prompt, 6)
    stop = config["eos_token_id"]
    expected = expected[: expected.index(stop) + 1] if stop in expected else expected
    assert lines[0]["token_ids"] == expected
    steps = int(errors.split("steps run:")[1].split(",")[0])
    assert steps >= 5 + len(expected) - 1  # 22 prompt tokens in portions of 5, then one step per further token
    # a text prompt: words to ids through the folder's tokenizer, the reply as text too
    vocabulary = {f"w{index}": index for index in range(config["vocab_size"])}
    tokenizer = Tokenizer(WordLevel(vocabulary, unk_token="w0"))
    tokenizer.pre_tokenizer = Whitespace()
    tokenizer.save(str(bare / "tokenizer.json"))
    lines, _ = run_generate([str(bare), "--prompt", " ".join(f"w{token}" for token in prompt), *common])
    assert lines[0]["token_ids"] == expected and lines[0]["text"].split() == [f"w{token}" for token in expected]
    # a preset shape needs no folder at all (the smallest published shape, bfloat16, two tokens)
    lines, _ = run_generate(["--preset", "lfm2-350m", "--random-weights", "3", "--prompt-ids", "1 2 3 4 5", "--max-tokens", "2", "--temperature", "0",
                             "--max-cache-tokens", "256", "--max-requests", "2"])
    assert len(lines[0]["token_ids"]) in (1, 2)
    # the registry's default options (temperature 0.3, min-p 0.15 for this family) apply with --spec: the tokens are drawn, and
    # the same seed draws the same ones
    sampled = [run_generate([str(bare), "--prompt-ids", "5 9 2 11", "--spec", "LiquidAI/LFM2-350M", "--seed", "4", "--random-weights", str(seed),
                             "--std", str(TEST_STD), "--dtype", "float32", "--max-cache-tokens", "512", "--max-tokens", "12"])[0][0]["token_ids"] for _ in range(2)]
    assert sampled[0] == sampled[1] and 1 <= len(sampled[0]) <= 12
