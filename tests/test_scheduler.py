"""The scheduler's decisions, on the host: admission, portions under the token budget, decoding
first, finishing and freeing, and what happens when pages run out."""

import pytest

from lalamo_b200.cache import CacheManager
from lalamo_b200.engine.scheduler import Request, RequestTooLong, Scheduler
from lalamo_b200.parts.base import PagedKVNeed, SlotStateNeed

NEEDS = [SlotStateNeed(shape=(2, 8)), PagedKVNeed(num_groups=1, head_dim=16)]


def make(num_pages=64, page_size=4, num_slots=8, max_batch_tokens=32, max_requests=8, chunk_size=None):
    cache = CacheManager(NEEDS, [None, None], None, page_size=page_size, num_pages=num_pages, num_slots=num_slots)
    return cache, Scheduler(cache, max_batch_tokens=max_batch_tokens, max_requests=max_requests, chunk_size=chunk_size)


def fake_token(request: Request) -> int:
    """What a deterministic model would sample: a function of the request's tokens so far."""
    tokens = request.all_tokens()
    return (sum(tokens) * 31 + len(tokens) * 7 + request.number) % 1000 + 10


def run_step(cache, scheduler, plan):
    """Plays the step function's part: reserves and commits pages, then samples."""
    sampled = []
    for entry in plan.entries:
        cache.reserve(entry.request.request_id, entry.request.computed + entry.count)
    for entry in plan.entries:
        cache.commit(entry.request.request_id, entry.request.computed + entry.count)
        if entry.samples:
            sampled.append(fake_token(entry.request))
    cache.check()
    return scheduler.complete(plan, sampled)


def run_all(cache, scheduler, limit=10000):
    finished, plans = [], []
    for _ in range(limit):
        plan = scheduler.plan()
        if plan is None:
            finished += scheduler.finished_now
            break
        plans.append(plan)
        finished += run_step(cache, scheduler, plan)
    assert not scheduler.has_work()
    return finished, plans


def test_budget_portions_and_decode_first():
    cache, scheduler = make(max_batch_tokens=16, chunk_size=10)
    first = Request(0, list(range(1, 26)), max_new_tokens=3)
    scheduler.add(first)
    plan = scheduler.plan()
    assert [(e.request.number, e.start, e.count, e.samples) for e in plan.entries] == [(0, 0, 10, False)]
    assert plan.admitted == [first]
    run_step(cache, scheduler, plan)
    second = Request(1, list(range(1, 9)), max_new_tokens=3)
    scheduler.add(second)
    plan = scheduler.plan()
    # the running request's next portion (chunk cap 10), then the newcomer with what is left of 16
    assert [(e.request.number, e.start, e.count, e.samples) for e in plan.entries] == [(0, 10, 10, False), (1, 0, 6, False)]
    run_step(cache, scheduler, plan)
    plan = scheduler.plan()
    assert [(e.request.number, e.start, e.count, e.samples) for e in plan.entries] == [(0, 20, 5, True), (1, 6, 2, True)]
    run_step(cache, scheduler, plan)
    third = Request(2, list(range(1, 40)), max_new_tokens=2)
    scheduler.add(third)
    plan = scheduler.plan()
    # decoding requests first, one token each, then the new prompt's portion
    assert [(e.request.number, e.count, e.samples) for e in plan.entries] == [(0, 1, True), (1, 1, True), (2, 10, False)]
    assert plan.tokens <= 16


def test_finishing_rules_and_freeing():
    cache, scheduler = make()
    stopper = Request(0, [5, 6, 7], max_new_tokens=50)
    stopper.stop_token_ids = frozenset({fake_token(Request(0, [5, 6, 7], 1))})
    limited = Request(1, [9, 9], max_new_tokens=4)
    scheduler.add(stopper)
    scheduler.add(limited)
    finished, _ = run_all(cache, scheduler)
    assert [(r.number, r.finish_reason, len(r.generated)) for r in finished] == [(0, "stop", 1), (1, "length", 4)]
    assert stopper.generated[-1] in stopper.stop_token_ids  # the stop token is part of the output
    assert cache.free_pages() == 64 and cache.slots.free_count == 8 and not cache.requests


def test_request_limit_and_fifo():
    cache, scheduler = make(max_requests=2, max_batch_tokens=64)
    for number in range(5):
        scheduler.add(Request(number, [number + 1] * 5, max_new_tokens=3 + number))
    seen_running = 0
    order = []
    while scheduler.has_work():
        plan = scheduler.plan()
        seen_running = max(seen_running, len(scheduler.running))
        order += [request.number for request in plan.admitted]
        run_step(cache, scheduler, plan)
    assert seen_running == 2 and order == [0, 1, 2, 3, 4]


def reference_outputs(prompts, max_new):
    cache, scheduler = make(num_pages=4096, max_batch_tokens=4096)
    requests = [Request(i, list(p), max_new) for i, p in enumerate(prompts)]
    for request in requests:
        scheduler.add(request)
    run_all(cache, scheduler)
    return [request.generated for request in requests]


def test_preemption_when_pages_run_out_keeps_the_outputs():
    prompts = [[i + 1] * n for i, n in enumerate([13, 9, 17, 6])]
    expected = reference_outputs(prompts, 20)
    # 16 pages of 4 = 64 tokens; the four requests grow to 33 + 29 + 37 + 26 = 125 tokens
    cache, scheduler = make(num_pages=16, max_batch_tokens=32)
    requests = [Request(i, list(p), 20) for i, p in enumerate(prompts)]
    for request in requests:
        scheduler.add(request)
    finished, plans = run_all(cache, scheduler)
    assert scheduler.stats.preemptions > 0
    assert [request.generated for request in requests] == expected
    assert all(request.finish_reason == "length" for request in requests)
    assert sorted(r.number for r in finished) == [0, 1, 2, 3]
    assert cache.free_pages() == 16 and cache.slots.free_count == 8
    # the victim is the most recently admitted request, and it re-reads prompt + generated
    victim = max(requests, key=lambda r: r.preemptions)
    assert victim.preemptions >= 1 and requests[0].preemptions == 0
    replays = [e for plan in plans for e in plan.entries if e.request is victim and e.start == 0]
    assert len(replays) == victim.preemptions + 1 and replays[-1].count > len(victim.prompt)


def test_a_preempted_request_does_not_redo_its_prompt_over_and_over():
    # 40 pages of 4 = 160 tokens.  The older request grows to 20 + 100 tokens, the younger to 40 + 60: after
    # about 50 steps the two have outgrown the pool and the younger one is preempted.
    cache, scheduler = make(num_pages=40, max_batch_tokens=64)
    older, younger = Request(0, [1] * 20, max_new_tokens=100), Request(1, [2] * 40, max_new_tokens=60)
    scheduler.add(older)
    scheduler.add(younger)
    finished, plans = run_all(cache, scheduler)
    assert sorted(r.number for r in finished) == [0, 1] and all(r.finish_reason == "length" for r in finished)
    assert younger.preemptions == 1 and older.preemptions == 0
    # held back until the older request has finished, it is readmitted once and reads prompt + generated once
    admissions = [index for index, plan in enumerate(plans) if younger in plan.admitted]
    assert len(admissions) == 2
    assert all(entry.request is younger for entry in plans[admissions[1]].entries)
    assert scheduler.stats.prompt_tokens <= 20 + 40 + (40 + 60)


def test_more_decoding_requests_than_the_token_budget_take_turns():
    cache, scheduler = make(num_pages=256, max_batch_tokens=16, max_requests=8)
    requests = [Request(number, [number + 1] * 2, max_new_tokens=6) for number in range(5)]
    for request in requests:
        scheduler.add(request)
    run_step(cache, scheduler, scheduler.plan())  # all five prompts in one step; from now on they decode
    scheduler.max_batch_tokens = 3
    finished, plans = run_all(cache, scheduler)
    assert sorted(r.number for r in finished) == [0, 1, 2, 3, 4]
    assert all(len(r.generated) == 6 and r.finish_reason == "length" for r in requests)
    assert all(plan.tokens <= 3 for plan in plans)
    # five requests decode, three tokens a step: nobody sits out two steps in a row
    last_seen: dict[int, int] = {}
    longest_gap = 0
    for index, plan in enumerate(plans):
        for entry in plan.entries:
            number = entry.request.number
            if entry.count == 1 and entry.samples and number in last_seen:
                longest_gap = max(longest_gap, index - last_seen[number])
            last_seen[number] = index
    assert longest_gap == 2


def test_alone_and_out_of_cache():
    cache, scheduler = make(num_pages=4, max_batch_tokens=64)  # 16 tokens in all
    request = Request(0, [3] * 10, max_new_tokens=50)
    scheduler.add(request)
    finished, _ = run_all(cache, scheduler)
    assert finished == [request] and request.finish_reason == "out_of_cache"
    assert len(request.prompt) + len(request.generated) == 17  # 16 tokens cached, one more sampled
    assert cache.free_pages() == 4
    with pytest.raises(RequestTooLong):
        scheduler.add(Request(1, [1] * 17, max_new_tokens=1))


def test_portion_shrinks_to_the_free_pages():
    cache, scheduler = make(num_pages=8, max_batch_tokens=64)
    scheduler.add(Request(0, [1] * 14, max_new_tokens=30))
    run_step(cache, scheduler, scheduler.plan())  # 4 pages held, decoding
    scheduler.add(Request(1, [2] * 30, max_new_tokens=2))
    plan = scheduler.plan()
    # 4 pages free, one kept back for the running request: the newcomer gets 3 pages = 12 tokens
    assert [(e.request.number, e.count) for e in plan.entries] == [(0, 1), (1, 12)]
    run_step(cache, scheduler, plan)
    finished, _ = run_all(cache, scheduler)
    assert {r.number for r in finished} == {0, 1}


def test_validation():
    _, scheduler = make()
    with pytest.raises(ValueError):
        scheduler.add(Request(0, [], 3))
    with pytest.raises(ValueError):
        scheduler.add(Request(0, [1], 0))
