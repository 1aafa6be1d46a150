"""The generation loop running one step ahead of its results, on the host alone: a fake step function
that knows every request's true tokens (as the device does) plays the engine, and whole workloads
must come out the same, token for token and reason for reason, as with every step awaited."""

from dataclasses import dataclass

import numpy as np
import pytest

from lalamo_b200.cache import CacheManager
from lalamo_b200.engine.generation import Generator
from lalamo_b200.parts.base import PagedKVNeed, SlotStateNeed
from lalamo_b200.sampling import GenerationConfig, SamplingPolicy

NEEDS = [SlotStateNeed(shape=(2, 8)), PagedKVNeed(num_groups=1, head_dim=16)]
VOCAB = 50


@dataclass
class FakeEngineConfig:
    max_batch_tokens: int
    max_requests: int


class FakePending:
    def __init__(self, tokens):
        self.device = list(tokens)
        self.waited = False

    def wait(self):
        self.waited = True
        return list(self.device)


class FakeRuntime:
    device = "cpu"


class FakeExecutor:
    def check_status(self):
        pass


class FakeEngine:
    """Keeps, per request, the tokens that are in its cache (the truth, as the device has it), and
    'samples' a function of them.  A step may only run if the step before has run: order is the stream's."""

    def __init__(self, num_pages, page_size, num_slots, max_batch_tokens, max_requests):
        self.cache = CacheManager(NEEDS, [None, None], None, page_size=page_size, num_pages=num_pages, num_slots=num_slots)
        self.engine_config = FakeEngineConfig(max_batch_tokens, max_requests)
        self.vocab_size = VOCAB
        self.runtime = FakeRuntime()
        self.executor = FakeExecutor()
        self.truth: dict[object, list[int]] = {}
        self.fed_from_device = 0
        self._numbers = 0

    def new_request_number(self):
        self._numbers += 1
        return self._numbers - 1

    def step(self, entries, previous_sampled=None):
        out = []
        for entry in entries:
            record = self.cache.requests[entry.request_id]
            tokens = list(entry.tokens)
            if entry.token_source >= 0:
                assert previous_sampled is not None
                tokens[-1] = previous_sampled[entry.token_source]
                self.fed_from_device += 1
            assert all(0 <= token < VOCAB for token in tokens)
            if record.length == 0:
                self.truth[entry.request_id] = []
            held = self.truth[entry.request_id]
            assert len(held) == record.length, "a step must continue where the cache ends"
            self.cache.reserve(entry.request_id, record.length + len(tokens))
            held.extend(tokens)
            for place in entry.want:
                prefix = held[: len(held) - len(tokens) + place + 1]
                out.append((sum(prefix) * 31 + len(prefix) * 7) % VOCAB)
            self.cache.commit(entry.request_id, len(held))
        self.cache.check()
        return out


class FakeSampler:
    def __init__(self):
        self.last_d2h_bytes = 0

    def sample_async(self, logits, rows):
        assert len(logits) == len(rows)
        return FakePending(logits)

    def set_counts(self, slot, tokens):
        pass

    def update_counts(self, slots, add, remove):
        pass


def run(workload, run_ahead, num_pages, max_batch_tokens, max_requests=8, chunk_size=None):
    engine = FakeEngine(num_pages=num_pages, page_size=4, num_slots=max_requests, max_batch_tokens=max_batch_tokens, max_requests=max_requests)
    generator = Generator(engine, seed=0, chunk_size=chunk_size, run_ahead=run_ahead)
    generator.sampler = FakeSampler()
    requests = []
    arrivals = sorted(workload, key=lambda item: item["arrives"])
    step = 0
    while arrivals or generator.has_work():
        while arrivals and arrivals[0]["arrives"] <= step:
            item = arrivals.pop(0)
            requests.append(generator.add(item["prompt"], SamplingPolicy(), item["stops"], item["new"], key_number=item["index"]))
        generator.step()
        step += 1
        assert step < 20000
    assert engine.cache.free_pages() == engine.cache.num_pages
    return {request.number: (list(request.generated), request.finish_reason, request.unresolved) for request in requests}, generator, engine


def random_workload(seed, count=12):
    rng = np.random.default_rng(seed)
    workload = []
    for index in range(count):
        workload.append({
            "index": index,
            "prompt": rng.integers(0, VOCAB, size=int(rng.integers(1, 30))).tolist(),
            "new": int(rng.integers(1, 25)),
            "stops": frozenset(rng.integers(0, VOCAB, size=int(rng.integers(0, 4))).tolist()),
            "arrives": int(rng.integers(0, 40)),
        })
    return workload


@pytest.mark.parametrize("seed", range(12))
def test_running_ahead_changes_no_token_and_no_reason(seed):
    workload = random_workload(seed)
    pages = [400, 400, 30, 18][seed % 4]   # roomy pools, and pools in which requests are preempted
    budget = [64, 7, 16, 32][(seed // 4) % 4]
    awaited, _, _ = run(workload, False, pages, budget)
    ahead, generator, engine = run(workload, True, pages, budget)
    assert ahead == awaited
    assert all(unresolved == 0 for _, _, unresolved in ahead.values())
    if pages == 400:
        assert generator.steps_run_ahead > 0 and engine.fed_from_device > 0


def test_a_request_that_stops_drops_the_token_sampled_past_its_end():
    # one request alone: every decode step after the first is launched before the ids of the step before are known
    prompt = [3, 4, 5]
    plain, _, _ = run([{"index": 0, "prompt": prompt, "new": 20, "stops": frozenset(), "arrives": 0}], False, 100, 16)
    tokens = plain[0][0]
    assert len(tokens) == 20 and plain[0][1] == "length"
    stop_at = 6
    stops = frozenset([tokens[stop_at]])
    first = min(i for i, token in enumerate(tokens) if token in stops)
    ahead, generator, engine = run([{"index": 0, "prompt": prompt, "new": 20, "stops": stops, "arrives": 0}], True, 100, 16)
    assert ahead[0] == (tokens[: first + 1], "stop", 0)
    assert generator.steps_run_ahead >= first


def test_the_length_limit_retires_a_request_without_a_step_past_it():
    ahead, generator, engine = run([{"index": 0, "prompt": [1, 2], "new": 5, "stops": frozenset(), "arrives": 0}], True, 100, 16)
    assert len(ahead[0][0]) == 5 and ahead[0][1] == "length"
    assert len(engine.truth[0]) == 2 + 4   # the fifth token was sampled but never fed


def test_prompts_that_want_one_token_each_follow_one_another_without_a_gap():
    """Requests that are done after their first step (one new token) and run one at a time: with nothing left
    running, the next prompt is still admitted and launched before the ids of the step in flight are awaited."""
    workload = [{"index": index, "prompt": list(range(1, 12)), "new": 1, "stops": frozenset(), "arrives": 0} for index in range(6)]
    awaited, _, _ = run(workload, run_ahead=False, num_pages=64, max_batch_tokens=12, max_requests=1)
    ahead, generator, _ = run(workload, run_ahead=True, num_pages=64, max_batch_tokens=12, max_requests=1)
    assert ahead == awaited
    assert generator.steps_run_ahead == len(workload) - 1
