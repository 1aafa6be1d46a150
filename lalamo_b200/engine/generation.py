"""Generation: scheduler + step function + sampler in one loop.

Every iteration asks the scheduler for a plan, runs it as one step, samples one token for every
request whose portion reached the end of its known tokens, and hands the tokens back to the
scheduler, which finishes and frees.  The only host<->device traffic per step is the batch
description going up and the sampled token ids coming down.

Unless a policy counts tokens (penalties need every id before the next sampling) or memory has to be
taken from a running request, the loop runs one step ahead of its results: a step
is planned and launched while the step before is still on the device, taking the ids that step samples
straight from device memory, and only then are that step's ids awaited on the host.  The host's work
of a step (plan, description, launch) thus overlaps the device's work of the step before.  Requests
finish, and tokens are reported, one call of :meth:`Generator.step` later than they were sampled; a
request that stopped has one token sampled past its end, which is dropped.  ``run_ahead=False`` turns
this off (every step's ids are awaited before the next is planned).
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Iterator, Sequence

from ..sampling.policy import GenerationConfig, SamplingPolicy
from ..sampling.sampler import PendingSample, SampleRow, Sampler, request_key
from .engine import Engine
from .executor import StepEntry
from .scheduler import Request, ResultsNeeded, Scheduler, StepPlan

__all__ = ["GeneratedSequence", "Generator"]


@dataclass
class GeneratedSequence:
    index: int  # position of the prompt in the call's list
    token_ids: list[int]  # generated tokens, a stop token included if one ended the sequence
    finish_reason: str  # "stop" | "length" | "out_of_cache"
    preemptions: int = 0


@dataclass
class _Flight:
    """A launched step whose sampled ids have not been awaited."""

    plan: StepPlan
    sample: PendingSample
    row_of: dict[int, int]  # request number -> its row among the step's sampled ids
    counts_tokens: bool  # some row's policy counts tokens: the next step's sampling needs this step's ids


class Generator:
    def __init__(self, engine: Engine, seed: int = 0, chunk_size: int | None = None, max_batch_tokens: int | None = None,
                 run_ahead: bool = True) -> None:
        """``max_batch_tokens`` overrides the engine configuration's token budget for this generator."""
        self.engine = engine
        self.seed = seed
        self.run_ahead = run_ahead
        self._flight: _Flight | None = None
        self.steps_run_ahead = 0  # steps launched before the ids of the step before were on the host
        self.sampler = Sampler(engine.cache, engine.vocab_size, engine.runtime.device)
        self.scheduler = Scheduler(
            engine.cache,
            max_batch_tokens=max_batch_tokens or engine.engine_config.max_batch_tokens,
            max_requests=engine.engine_config.max_requests,
            chunk_size=chunk_size,
        )
        self._added = 0
        # Wall-clock seconds of this generator's steps by section (the device works during ``sample_and_wait``
        # and the tail of ``launch`` only): what the host costs a step.
        self.host_seconds = {"plan": 0.0, "launch": 0.0, "sample_and_wait": 0.0, "complete": 0.0}
        self._requests: list[Request] = []

    # ------------------------------------------------------------------- requests
    def add(
        self,
        prompt: Sequence[int],
        policy: SamplingPolicy,
        stop_token_ids: Sequence[int],
        max_new_tokens: int,
        key_number: int | None = None,
    ) -> Request:
        # The cache manager belongs to the engine and names requests by number: numbers come from the
        # engine, so that two generators on one engine never collide.  The random key follows the order
        # of arrival at this generator, so that a call's outputs do not depend on earlier calls.
        number = self.engine.new_request_number()
        arrival = self._added
        self._added += 1
        for token in prompt:
            if not 0 <= int(token) < self.engine.vocab_size:
                raise ValueError(f"prompt token {token} is outside the vocabulary of {self.engine.vocab_size}")
        request = Request(
            number=number,
            prompt=[int(token) for token in prompt],
            max_new_tokens=max_new_tokens,
            policy=policy,
            stop_token_ids=frozenset(int(token) for token in stop_token_ids),
            key=request_key(self.seed, arrival if key_number is None else key_number),
        )
        self.scheduler.add(request)
        self._requests.append(request)
        return request

    def close(self) -> None:
        """Ends every request of this generator that has not finished (reason ``"aborted"``), so that
        their pages and slots go back to the engine's cache.  Safe to call twice."""
        self._flight = None  # what it was sampling is of no use to anybody
        for request in self._requests:
            if request.status != "finished":
                self.scheduler.abort(request)
        self._requests = []

    # ----------------------------------------------------------------------- steps
    def _setup_admitted(self, plan: StepPlan) -> None:
        for request in plan.admitted:
            if request.policy.has_count_penalties:
                tokens = request.tokens
                window = request.policy.suffix_repetition_length
                self.sampler.set_counts(self.engine.cache.requests[request.request_id].slot, tokens[-window:] if window else tokens)

    def has_work(self) -> bool:
        """Whether :meth:`step` has anything left to do (requests to run, or results to collect)."""
        return self.scheduler.has_work() or self._flight is not None

    def _may_run_ahead(self) -> bool:
        """Whether the next step may be planned without the ids of the step in flight.  Those ids can only
        end requests, which a plan made without them does not know: it keeps their memory a step longer and
        samples one token past their end.  A plan that would have to preempt says so (``ResultsNeeded``);
        policies that count tokens need every id before the next sampling."""
        flight = self._flight
        # (with nothing running, waiting requests can still be admitted and begun: none of that needs the ids)
        return flight is not None and self.run_ahead and not flight.counts_tokens and self.scheduler.has_work()

    def _collect(self) -> None:
        """Awaits the ids of the step in flight and hands them to the scheduler."""
        flight = self._flight
        if flight is None:
            return
        self._flight = None
        sampled = flight.sample.wait()
        self._count_sampled(flight, sampled)
        self.scheduler.resolve(flight.plan, sampled)

    def step(self) -> list[Request] | None:
        """Runs one step; returns the requests that are known to have finished since the last call, or
        ``None`` when idle."""
        clock = time.perf_counter
        t0 = clock()
        scheduler = self.scheduler
        finished: list[Request] = []
        ahead = self._may_run_ahead()
        if not ahead and self._flight is not None:
            scheduler.finished_now = []
            self._collect()
            finished += scheduler.finished_now
        try:
            plan = scheduler.plan()  # starts a new list of finished requests
        except ResultsNeeded:
            scheduler.finished_now = []
            self._collect()
            finished += scheduler.finished_now
            plan = scheduler.plan()
        finished += scheduler.finished_now
        if plan is None:
            if self._flight is not None:
                scheduler.finished_now = []
                self._collect()
                finished += scheduler.finished_now
            self.host_seconds["plan"] += clock() - t0
            return finished or None
        self._setup_admitted(plan)
        previous = self._flight
        entries, rows, row_of = [], [], {}
        counts_tokens = False
        for planned in plan.entries:
            request = planned.request
            tokens = request.tokens[planned.start : planned.start + planned.count]
            source = -1
            if request.unresolved and planned.start + planned.count == len(request.tokens):
                # the portion ends with the token the step in flight is sampling: the device hands it over
                assert previous is not None and request.unresolved == 1
                source = previous.row_of[request.number]
                tokens[-1] = 0
            entries.append(StepEntry(request.request_id, tokens, [planned.count - 1] if planned.samples else [], source))
            if planned.samples:
                slot = self.engine.cache.requests[request.request_id].slot
                row_of[request.number] = len(rows)
                rows.append(SampleRow(request.policy, request.key, request.num_generated, slot))
                counts_tokens = counts_tokens or request.policy.has_count_penalties
        t1 = clock()
        logits = self.engine.step(entries, previous.sample.device if previous is not None else None)
        t2 = clock()
        sample = self.sampler.sample_async(logits, rows)
        scheduler.advance(plan)
        if previous is not None:
            self.steps_run_ahead += 1
            scheduler.finished_now = []
            self._collect()  # the step before: its ids were awaited only now
            finished += scheduler.finished_now
        self._flight = _Flight(plan, sample, row_of, counts_tokens)
        t3 = clock()
        if not self.run_ahead:
            scheduler.finished_now = []
            self._collect()
            finished += scheduler.finished_now
        t4 = clock()
        spent = self.host_seconds
        spent["plan"] += t1 - t0
        spent["launch"] += t2 - t1
        spent["sample_and_wait"] += t3 - t2
        spent["complete"] += t4 - t3
        return finished

    def _count_sampled(self, flight: _Flight, sampled: list[int]) -> None:
        """Adds a step's sampled tokens to the counts of the requests whose policies count tokens (and
        takes out what leaves a counted suffix); runs before the scheduler learns the tokens, so a
        request's last token is still the placeholder of this step."""
        if not flight.counts_tokens:
            return
        slots, add, remove = [], [], []
        tokens = iter(sampled)
        for planned in flight.plan.entries:
            if not planned.samples:
                continue
            token = next(tokens)
            request = planned.request
            policy = request.policy
            if not policy.has_count_penalties or request.status != "running":
                continue  # a request that has left the running set is not sampled for again
            slots.append(self.engine.cache.requests[request.request_id].slot)
            add.append(token)
            window = policy.suffix_repetition_length
            known = planned.token_index  # tokens before the one this step sampled
            remove.append(request.tokens[known - window] if window and known >= window else -1)
        self.sampler.update_counts(slots, add, remove)

    # ------------------------------------------------------------------ whole calls
    def generate_many(
        self,
        prompts: Sequence[Sequence[int]],
        generation_config: GenerationConfig | Sequence[GenerationConfig],
        max_output_length: int,
        on_step: Callable[["Generator"], None] | None = None,
    ) -> Iterator[GeneratedSequence]:
        """Generates for all prompts; yields sequences in the order they finish.  ``on_step`` is called
        with this generator after every step (for statistics: step times, pages in use)."""
        configs = [generation_config] * len(prompts) if isinstance(generation_config, GenerationConfig) else list(generation_config)
        if len(configs) != len(prompts):
            raise ValueError("one generation config per prompt, or one for all")
        index_of: dict[int, int] = {}
        try:
            for index, (prompt, config) in enumerate(zip(prompts, configs)):
                request = self.add(prompt, config.default_policy(), config.stop_token_ids, max_output_length, key_number=index)
                index_of[request.number] = index
            while self.has_work():
                finished = self.step()
                if on_step is not None:
                    on_step(self)
                for request in finished or []:
                    yield GeneratedSequence(index_of[request.number], list(request.generated), request.finish_reason or "", request.preemptions)
            # Kernels report what they refused (a block-table entry outside the pool, a wait that gave up)
            # in a status word on the device: read once per call, it costs one synchronisation.
            self.engine.executor.check_status()
        finally:
            # A consumer that stops early, or a step that raises, must not leave requests in the cache.
            self.close()
