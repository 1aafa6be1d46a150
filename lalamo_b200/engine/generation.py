"""Generation: scheduler + step function + sampler in one loop.

Every iteration asks the scheduler for a plan, runs it as one step, samples one token for every
request whose portion reached the end of its known tokens, and hands the tokens back to the
scheduler, which finishes and frees.  The only host<->device traffic per step is the batch
description going up and the sampled token ids coming down.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Iterator, Sequence

from ..sampling.policy import GenerationConfig, SamplingPolicy
from ..sampling.sampler import SampleRow, Sampler, request_key
from .engine import Engine
from .executor import StepEntry
from .scheduler import Request, Scheduler, StepPlan

__all__ = ["GeneratedSequence", "Generator"]


@dataclass
class GeneratedSequence:
    index: int  # position of the prompt in the call's list
    token_ids: list[int]  # generated tokens, a stop token included if one ended the sequence
    finish_reason: str  # "stop" | "length" | "out_of_cache"
    preemptions: int = 0


class Generator:
    def __init__(self, engine: Engine, seed: int = 0, chunk_size: int | None = None, max_batch_tokens: int | None = None) -> None:
        """``max_batch_tokens`` overrides the engine configuration's token budget for this generator."""
        self.engine = engine
        self.seed = seed
        self.sampler = Sampler(engine.cache, engine.vocab_size, engine.runtime.device)
        self.scheduler = Scheduler(
            engine.cache,
            max_batch_tokens=max_batch_tokens or engine.engine_config.max_batch_tokens,
            max_requests=engine.engine_config.max_requests,
            chunk_size=chunk_size,
        )
        self._added = 0
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

    def step(self) -> list[Request] | None:
        """Runs one step; returns the requests that finished in it, or ``None`` when idle."""
        plan = self.scheduler.plan()
        if plan is None:
            return list(self.scheduler.finished_now) or None
        self._setup_admitted(plan)
        entries, rows = [], []
        for planned in plan.entries:
            request = planned.request
            tokens = request.tokens[planned.start : planned.start + planned.count]
            entries.append(StepEntry(request.request_id, tokens, [planned.count - 1] if planned.samples else []))
            if planned.samples:
                slot = self.engine.cache.requests[request.request_id].slot
                rows.append(SampleRow(request.policy, request.key, request.num_generated, slot))
        logits = self.engine.step(entries)
        sampled = self.sampler.sample(logits, rows)
        self._count_sampled(plan, sampled)
        return list(self.scheduler.complete(plan, sampled))

    def _count_sampled(self, plan: StepPlan, sampled: list[int]) -> None:
        slots, add, remove = [], [], []
        tokens = iter(sampled)
        for planned in plan.entries:
            if not planned.samples:
                continue
            token = next(tokens)
            policy = planned.request.policy
            if not policy.has_count_penalties:
                continue
            slots.append(self.engine.cache.requests[planned.request.request_id].slot)
            add.append(token)
            window = policy.suffix_repetition_length
            history = planned.request.tokens
            remove.append(history[len(history) - window] if window and len(history) >= window else -1)
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
            while self.scheduler.has_work():
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
