"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  It decides; the step function runs what it decided.

Every live request always has *pending* tokens, the part of ``prompt + generated`` that is not in
the cache yet: a long tail while its prompt is being read, exactly one (the token sampled last)
while it decodes.  A step takes, in this order and while the token budget lasts,

1. one token of every decoding request (those that sat out longest first, so that a budget smaller
   than the number of decoding requests serves them in turns),
2. the next portion of every request still reading its prompt (oldest first),
3. first portions of waiting requests (first come, first served), which admits them.

A request is admitted only if a state slot is free, its first portion fits into the free pages, and
one free page remains for every running request after it (so admission does not starve decoding).

**When pages run out.**  If a portion of a prompt does not fit, it is shortened to what fits, or the
request sits the step out.  If a decoding request needs a page and none is free, the most
recently admitted running request is *preempted*: its pages and slot are freed and it goes back to
the head of the waiting queue with ``prompt + generated so far`` as its prompt; when readmitted it
recomputes its cache and then continues (its random stream and token budget are untouched, so the
output does not change).  A preempted request is held back until a running request has finished or
the free pages cover all its tokens beside a page for every running request: readmitted earlier it
would read until the pool is full, be preempted again at the next page an older request needs, and
redo its prompt every time.  While requests decode, a prompt portion leaves them a page each for the
same reason.  A request that runs out of pages while it is the only one running is
finished with reason ``"out_of_cache"``; a request whose prompt can never fit is refused at
:meth:`Scheduler.add` with :class:`RequestTooLong`.

The reference's scheduler keeps a fixed number of lines, each with a full-capacity cache, and never
mixes prompt reading with decoding (``lalamo/inference/batch_scheduler.py:993-1097``); its finishing
rules are kept: a stop token ends the request and is part of the output, as is reaching the length
limit (``batch_scheduler.py:655-658``, ``lalamo/models/language_model.py:142-150``).

**Results that arrive late.**  :meth:`Scheduler.complete` is two halves that a caller may pull apart so
that the host prepares the next step while the device still runs this one.  :meth:`Scheduler.advance`
(right after the launch) counts the step's tokens as computed and appends a placeholder,
``PENDING_TOKEN``, for every token being sampled; a request that reaches its length limit with it is
*retired*: it leaves the running set and gives its cache back at once, and is reported when its
tokens are known.  :meth:`Scheduler.resolve` (when the sampled ids have reached the host) replaces the
placeholders and applies the stop tokens.  In between, a request with a placeholder as its last token
can be planned as any decoding request (the step function takes the id from the device); if it turns
out to have stopped, the token that was sampled for it meanwhile is dropped.  A request with
placeholders is never preempted: :meth:`Scheduler.plan` raises :class:`ResultsNeeded` instead, having
changed nothing, and the caller resolves and plans again.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..sampling.policy import SamplingPolicy

__all__ = ["PENDING_TOKEN", "PlannedEntry", "Request", "RequestTooLong", "ResultsNeeded", "Scheduler", "SchedulerStats", "StepPlan"]

PENDING_TOKEN = -1  # stands in ``Request.tokens`` for a token that was sampled but has not reached the host


class RequestTooLong(ValueError):
    pass


class ResultsNeeded(RuntimeError):
    """:meth:`Scheduler.plan` has to take memory from a request whose last tokens are placeholders:
    nothing has been changed; :meth:`Scheduler.resolve` the step in flight and plan again."""


@dataclass
class Request:
    number: int  # order of arrival; also names the request in the cache manager
    prompt: list[int]
    max_new_tokens: int
    policy: SamplingPolicy = field(default_factory=SamplingPolicy)
    stop_token_ids: frozenset[int] = frozenset()
    key: tuple[int, int] = (0, 0)
    computed: int = 0  # tokens of prompt + generated that are in the cache
    status: str = "waiting"  # waiting | running | finishing (retired, last tokens not yet known) | finished
    finish_reason: str | None = None
    preemptions: int = 0
    held: bool = False  # preempted and not to be readmitted before memory has been freed
    last_step: int = -1  # the scheduler step that last ran a token of this request
    unresolved: int = 0  # placeholders at the end of ``tokens``
    tokens: list[int] = field(default_factory=list)  # prompt + generated, grown in place

    def __post_init__(self) -> None:
        if not self.tokens:
            self.tokens = list(self.prompt)

    @property
    def request_id(self) -> int:
        return self.number

    @property
    def generated(self) -> list[int]:
        return self.tokens[len(self.prompt) :]

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - len(self.prompt)

    def all_tokens(self) -> list[int]:
        return self.tokens

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.computed


@dataclass
class PlannedEntry:
    request: Request
    start: int  # first pending token taken (index into prompt + generated)
    count: int
    samples: bool  # the portion reaches the end of the known tokens: its last logits are sampled
    token_index: int = -1  # where in ``request.tokens`` the sampled token goes (set by ``advance``)


@dataclass
class StepPlan:
    entries: list[PlannedEntry]
    admitted: list[Request]  # admitted by this plan (their per-request state must be set up)

    @property
    def tokens(self) -> int:
        return sum(entry.count for entry in self.entries)


@dataclass
class SchedulerStats:
    steps: int = 0
    prompt_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batch_tokens: int, max_requests: int, chunk_size: int | None = None) -> None:
        if max_batch_tokens < 1 or max_requests < 1:
            raise ValueError("max_batch_tokens and max_requests must be positive")
        self.cache = cache
        self.max_batch_tokens = max_batch_tokens
        self.max_requests = min(max_requests, cache.num_slots)
        self.chunk_size = chunk_size or max_batch_tokens
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.finished_now: list[Request] = []
        self.stats = SchedulerStats()

    # ---------------------------------------------------------------------- requests
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if request.max_new_tokens < 1:
            raise ValueError("max_new_tokens must be at least 1")
        pages = -(-(len(request.prompt)) // self.cache.page_size)
        if pages > self.cache.num_pages:
            raise RequestTooLong(
                f"a prompt of {len(request.prompt)} tokens needs {pages} pages of {self.cache.page_size}; the pool has {self.cache.num_pages}"
            )
        request.status = "waiting"
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def _finish(self, request: Request, reason: str) -> None:
        request.status = "finished"
        request.finish_reason = reason
        if request in self.running:
            self.running.remove(request)
            self.cache.release(request.request_id)
            for other in self.waiting:
                other.held = False  # memory came back: preempted requests may try again
        self.finished_now.append(request)
        self.stats.finished += 1

    def abort(self, request: Request) -> None:
        """Ends a waiting or running request now (reason ``"aborted"``) and frees what it holds."""
        if request in self.waiting:
            self.waiting.remove(request)
        if request.status != "finished":
            self._finish(request, "aborted")

    def _retire(self, request: Request) -> None:
        """The request needs no further step, but its last tokens are not on the host yet: it leaves the
        running set and frees its cache now and is reported by :meth:`resolve`."""
        request.status = "finishing"
        self.running.remove(request)
        self.cache.release(request.request_id)
        for other in self.waiting:
            other.held = False

    def _preempt(self, request: Request) -> None:
        self.running.remove(request)
        self.cache.release(request.request_id)
        request.computed = 0
        request.status = "waiting"
        request.preemptions += 1
        request.held = True
        self.waiting.appendleft(request)
        self.stats.preemptions += 1

    # -------------------------------------------------------------------------- plan
    def _fit(self, request: Request, wanted: int, free: int) -> int:
        """The largest count <= wanted whose new pages fit into ``free`` pages."""
        covered = (self.cache.blocks_held(request.request_id) + free) * self.cache.page_size
        return max(0, min(wanted, covered - request.computed))

    def _try_plan(self) -> StepPlan | None:
        """A plan, or ``None`` if a running request must be preempted first."""
        budget = self.max_batch_tokens
        free = self.cache.free_pages()
        entries: list[PlannedEntry] = []
        decoding = sorted((r for r in self.running if r.pending == 1), key=lambda r: r.last_step)  # stable: oldest first among equals
        reading = [r for r in self.running if r.pending > 1]
        for request in decoding:
            if budget == 0:
                break
            need = self.cache.pages_needed(request.request_id, request.computed + 1)
            if need > free:
                return None
            free -= need
            budget -= 1
            entries.append(PlannedEntry(request, request.computed, 1, True))
        for request in reading:
            if budget == 0:
                break
            # a page stays free for every decoding request, as at admission
            count = self._fit(request, min(request.pending, budget, self.chunk_size), max(0, free - len(decoding)))
            if count == 0:
                continue
            free -= self.cache.pages_needed(request.request_id, request.computed + count)
            budget -= count
            entries.append(PlannedEntry(request, request.computed, count, count == request.pending))
        if not entries and self.running:
            return None  # nobody can move: free something
        admitted: list[Request] = []
        while self.waiting and budget > 0 and len(self.running) + len(admitted) < self.max_requests:
            request = self.waiting[0]
            reserve = len(self.running) + len(admitted)  # one page for every request already running
            wanted = min(request.pending, budget, self.chunk_size)
            page = self.cache.page_size
            count = min(wanted, max(0, free - reserve) * page)
            if count < min(wanted, page) and (self.running or admitted):
                break  # not even a page's worth fits beside the running requests
            if request.held and (self.running or admitted) and (free - reserve) * page < len(request.tokens) + 1:
                break  # preempted: it waits until somebody finishes or all of it fits
            if count == 0:
                break
            self.waiting.popleft()
            admitted.append(request)
            free -= -(-count // page)
            budget -= count
            entries.append(PlannedEntry(request, 0, count, count == request.pending))
        return StepPlan(entries, admitted)

    def plan(self) -> StepPlan | None:
        """Decides the next step (admitting and preempting as needed); ``None`` when idle.
        Requests that had to be finished while planning are in ``finished_now``."""
        self.finished_now = []
        while self.has_work():
            plan = self._try_plan()
            if plan is None:
                victim = self.running[-1]
                if victim.unresolved:
                    raise ResultsNeeded(f"request {victim.number} has {victim.unresolved} tokens that are not on the host yet")
                if len(self.running) == 1:
                    self._finish(victim, "out_of_cache")
                else:
                    self._preempt(victim)
                continue
            if not plan.entries:
                if self.waiting and not self.running:
                    # the head of the queue fits nowhere although the cache is empty
                    request = self.waiting.popleft()
                    self._finish(request, "out_of_cache")
                    continue
                return None
            for request in plan.admitted:
                self.cache.admit(request.request_id)
                request.status = "running"
                self.running.append(request)
            return plan
        return None

    # ------------------------------------------------------------------------ results
    def complete(self, plan: StepPlan, sampled: list[int]) -> list[Request]:
        """Records a step's results (``sampled``: one token per sampling entry, in plan order).
        Returns the requests that finished since :meth:`plan` was called (those it had to finish
        itself first), their cache already freed."""
        self.advance(plan)
        return self.resolve(plan, sampled)

    def advance(self, plan: StepPlan) -> None:
        """The step has been launched: its tokens count as computed, and every token it samples
        stands in ``Request.tokens`` as ``PENDING_TOKEN`` until :meth:`resolve` brings its value."""
        self.stats.steps += 1
        for entry in plan.entries:
            request = entry.request
            request.computed += entry.count
            request.last_step = self.stats.steps
            if entry.count == 1 and entry.start >= len(request.prompt):
                self.stats.decode_tokens += 1
            else:
                self.stats.prompt_tokens += entry.count
            if not entry.samples:
                continue
            entry.token_index = len(request.tokens)
            request.tokens.append(PENDING_TOKEN)
            request.unresolved += 1
            if request.num_generated >= request.max_new_tokens:
                self._retire(request)

    def resolve(self, plan: StepPlan, sampled: list[int]) -> list[Request]:
        """The sampled tokens of an advanced step (one per sampling entry, in plan order) are known.
        Returns the requests that finished since :meth:`plan` was last called."""
        tokens = iter(sampled)
        for entry in plan.entries:
            if not entry.samples:
                continue
            token = int(next(tokens))
            request = entry.request
            if request.status == "finished":
                continue  # it stopped at an earlier token; this one was sampled past its end
            request.tokens[entry.token_index] = token
            request.unresolved -= 1
            if token in request.stop_token_ids:
                del request.tokens[entry.token_index + 1 :]  # placeholders of tokens sampled past the stop
                request.unresolved = 0
                self._finish(request, "stop")
            elif request.status == "finishing" and request.unresolved == 0:
                self._finish(request, "length")
        return self.finished_now
