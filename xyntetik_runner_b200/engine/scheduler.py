"""The scheduler above the step function: admit, cut prompts under a token budget, decode, finish, free.

The reference runs fixed slots and lets prefill chunks (``-b``, src/engine.c:875-883) and batched decode
steps take turns on the device (src/scheduler.c:101-125, 153-220).  Here one step holds both: every live
request that is decoding contributes its one token first; what is left of the step's token budget goes to
requests that are still reading their prompt, in the order they were admitted, as portions; then waiting
requests are admitted (first come, first served) while a slot and pages are free.  A request finishes on a
stop id, on its token limit, or at the longest length the engine holds (src/engine.c:1834, 1844-1854), and
gives its pages and slot back in the same tick.

When pages run out:
 1. a prompt portion is shrunk to what fits (possibly to nothing: the request waits);
 2. if a decoding request cannot get the page its next token needs, the most recently admitted live
    request is preempted: its pages are freed and it goes back to the FRONT of the waiting queue with
    prompt + generated so far as its new prompt (recompute; its sampler state is kept, so it goes on
    with the same tokens);
 3. the same happens when no live request can make progress at all;
 4. a request that could never fit the pool alone is refused when it is added; one that outgrows the
    pool while it is the only live request finishes with reason "length".

This module is host logic only.  It talks to the cache manager for reservations and to an executor
(``run(plan) -> {request id: sampled token}``) for the step, so its decisions are testable without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple

from ..cache.pages import CacheManager
from ..sampling.sampler import RequestSampler, SamplingParams

WAITING, LIVE, FINISHED = "waiting", "live", "finished"


@dataclass
class Request:
    id: object
    prompt: List[int]
    max_new_tokens: int = 256
    sampling: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Tuple[int, ...] = ()
    ignore_eos: bool = False
    # ---- run-time state ----
    tokens: List[int] = field(default_factory=list)      # prompt + generated
    generated: List[int] = field(default_factory=list)
    computed: int = 0                                     # tokens whose keys are in the cache
    status: str = WAITING
    finish_reason: Optional[str] = None
    admitted_at: int = -1
    preemptions: int = 0
    sampler: Optional[RequestSampler] = None

    @property
    def pending(self) -> int:
        return len(self.tokens) - self.computed


IN_FLIGHT = -1       # stands in a request's tokens for one that a launched step has not delivered yet


class _IdentitySet:
    """Membership by identity (requests are dataclasses: their equality compares fields)."""

    def __init__(self, items=()):
        self._ids = {id(x) for x in items}

    def __contains__(self, x) -> bool:
        return id(x) in self._ids


class _NoLookAhead(Exception):
    """Planning ahead met a decision that needs the running step's outcome (a preemption, a request to end)."""


@dataclass
class PlannedEntry:
    request: Request
    start: int
    count: int
    wants_token: bool

    @property
    def tokens(self) -> List[int]:
        return self.request.tokens[self.start:self.start + self.count]


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[object] = field(default_factory=list)
    finished: List[object] = field(default_factory=list)     # requests that planning itself ended (pool too small)
    admitted: List["Request"] = field(default_factory=list)  # requests that this plan took from the queue

    @property
    def n_tokens(self) -> int:
        return sum(e.count for e in self.entries)


@dataclass
class SchedulerParams:
    max_step_tokens: int = 2048      # token budget of one step
    prefill_chunk: Optional[int] = None   # cap on one request's portion (the reference's -b); None: the budget
    # Launch the next decode step before the tokens of the running one have been read (needs an executor with
    # `launch` / `wait`): the host's planning then overlaps the device's work.  See Scheduler.step.
    look_ahead: bool = True


class Scheduler:
    def __init__(self, cache: CacheManager, executor, params: Optional[SchedulerParams] = None, open_request=None):
        self.cache, self.executor = cache, executor
        # opening a request takes a state slot; an engine also zeroes the slot's per-request state
        self._open = open_request or cache.open
        self.params = params or SchedulerParams()
        self.waiting: Deque[Request] = deque()
        self.live: List[Request] = []           # in admission order
        self.finished: Dict[object, Request] = {}
        self._tick = 0
        self._ahead = None                      # (plan, executor's handle) of a step launched ahead of its turn
        self._ended_unreported: List[object] = []   # ended by a plan whose step then failed to launch
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0, "max_batch": 0,
                      "steps_launched_ahead": 0}

    # ---- adding ---------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError(f"request {req.id!r}: empty prompt")     # src/main.c:1522-1529
        limit = self.cache.max_pages_per_request * self.cache.page_size
        if len(req.prompt) >= limit:
            raise ValueError(f"request {req.id!r}: prompt of {len(req.prompt)} tokens does not fit the "
                             f"longest request the engine holds ({limit})")
        if any(g.window is None for g in self.cache.groups) or not self.cache.groups:
            pool = min((p.n_pages for p in self.cache.pools), default=1 << 30)
            if -(-(len(req.prompt) + 1) // self.cache.page_size) > pool:
                raise ValueError(f"request {req.id!r}: prompt of {len(req.prompt)} tokens can never fit a pool of "
                                 f"{pool} pages of {self.cache.page_size}")
        if req.max_new_tokens == 0:
            raise ValueError("max_new_tokens must not be 0")
        req.tokens = [t if t >= 0 else 0 for t in req.prompt]      # an id below zero reads row 0, as one beyond the table does
        req.generated = []
        req.computed = 0
        req.status = WAITING
        req.sampler = RequestSampler(req.sampling, no_penalty=req.stop_ids)
        for t in req.prompt:
            req.sampler.accept(t)                # the prompt seeds the penalty window (src/engine.c:881)
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.live)

    def abort(self, request_id) -> bool:
        """End a request now, whatever its state (the reference's callback abort and cancel, src/engine.c:1844-1848,
        src/scheduler.c:383-385): a waiting one leaves the queue, a live one gives its pages and its slot back in this
        call; what it has generated so far stays in `finished` with the reason "abort".  False if it is not known
        (or already finished).  A step launched ahead that still holds a row for it computes that row for nothing;
        the pages it writes are handed to nobody before that step has run (the next step follows it on the stream)."""
        for r in self.waiting:
            if r.id == request_id:
                self.waiting.remove(r)
                self._finish(r, "abort")
                return True
        for r in self.live:
            if r.id == request_id:
                if r.tokens and r.tokens[-1] == IN_FLIGHT:
                    r.tokens.pop()               # the mark of a token that nobody will read
                self._finish(r, "abort")
                return True
        return False

    # ---- planning -----------------------------------------------------------------------
    def _preempt(self, victim: Request, plan: StepPlan) -> int:
        """Push `victim` back to the queue.  Returns the tokens of the step's budget that its planned entry held."""
        given_back = 0
        for e in list(plan.entries):
            if e.request is victim:
                plan.entries.remove(e)
                given_back += e.count
        self.cache.cancel(victim.id)
        self.cache.close(victim.id)
        self.live.remove(victim)
        victim.computed = 0
        victim.status = WAITING
        victim.preemptions += 1
        self.waiting.appendleft(victim)
        plan.preempted.append(victim.id)
        self.stats["preemptions"] += 1
        return given_back

    def _fit(self, req: Request, want: int) -> int:
        """Largest portion <= want whose pages can be reserved now (0: none)."""
        if want < 1:
            return 0
        if self.cache.can_reserve(req.id, want):
            return want
        lo, hi = 0, want            # can_reserve is monotone in the count
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.cache.can_reserve(req.id, mid):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def _undo(self, plan: StepPlan) -> None:
        """Take back what a plan that will not run has done: its reservations and its admissions."""
        for e in plan.entries:
            self.cache.cancel(e.request.id)
        for r in reversed(plan.admitted):
            self.cache.close(r.id)
            self.live.remove(r)
            r.status, r.admitted_at = WAITING, -1
            self._tick -= 1
            self.waiting.appendleft(r)
        plan.entries.clear()
        plan.admitted.clear()

    def plan(self, ahead: bool = False, skip=()) -> StepPlan:
        """The next step: who runs how many tokens.  `ahead`: the plan is made while the step before it is still
        running, for the state that step will leave (its tokens standing in the requests as IN_FLIGHT marks);
        requests in `skip` (known to end with that step) take no part, and a decision that needs that step's outcome
        -- preempting, ending a request -- is not made: everything is undone and ``_NoLookAhead`` raised."""
        plan = StepPlan()
        try:
            return self._plan(plan, ahead, skip)
        except _NoLookAhead:
            self._undo(plan)
            raise

    def _plan(self, plan: StepPlan, ahead: bool, skip) -> StepPlan:
        budget = self.params.max_step_tokens
        chunk_cap = self.params.prefill_chunk or budget
        # 1. decoding requests: one token each; pages for them come before anything else
        i = 0
        while i < len(self.live):
            r = self.live[i]
            if r.pending != 1 or budget < 1 or r in skip:
                i += 1
                continue
            if self.cache.can_reserve(r.id, 1):
                self.cache.reserve(r.id, 1)
                plan.entries.append(PlannedEntry(r, r.computed, 1, True))
                budget -= 1
                i += 1
                continue
            if ahead:
                raise _NoLookAhead()
            if len(self.live) == 1:
                self._finish(r, "length")          # alone and still no page: the pool is its limit
                plan.finished.append(r.id)
                continue
            victim = self.live[-1]
            vi = len(self.live) - 1
            budget += self._preempt(victim, plan)
            if vi < i:
                i -= 1
            # try the same index again (it is r again unless r itself was the victim)
        # 2. requests still reading their prompt, in admission order
        for r in self.live:
            if r.pending < 1 or budget < 1 or r in skip or any(e.request is r for e in plan.entries):
                continue
            n = self._fit(r, min(r.pending, budget, chunk_cap))
            if n > 0:
                self.cache.reserve(r.id, n)
                plan.entries.append(PlannedEntry(r, r.computed, n, n == r.pending))
                budget -= n
        # 3. admissions, first come first served
        #    (not in a step that had to preempt, and only while a page per live request stays free, so that
        #    a request that was just pushed out does not take the pages the older ones are about to need)
        while self.waiting and budget > 0 and self.cache.has_free_slot() and not plan.preempted:
            r = self.waiting[0]
            self._open(r.id)
            n = self._fit(r, min(r.pending, budget, chunk_cap))
            if n > 0 and self.live:
                need = self.cache.pages_needed(r.id, n)
                while n > 0 and any(f - q < len(self.live) for f, q in zip(self.cache.free_pages(), need)):
                    n = (n - 1) // self.cache.page_size * self.cache.page_size if n > self.cache.page_size else 0
                    need = self.cache.pages_needed(r.id, n) if n > 0 else need
            if n < 1:
                self.cache.close(r.id)
                break
            self.waiting.popleft()
            self.cache.reserve(r.id, n)
            r.status = LIVE
            r.admitted_at = self._tick
            self._tick += 1
            self.live.append(r)
            plan.admitted.append(r)
            plan.entries.append(PlannedEntry(r, r.computed, n, n == r.pending))
            budget -= n
        # 4. nobody can move: free the newest request's pages for the older ones
        if not plan.entries and self.live and ahead:
            return plan                       # (decided when the running step's outcome is known)
        if not plan.entries and self.live:
            if len(self.live) == 1:
                plan.finished.append(self.live[0].id)
                self._finish(self.live[0], "length")
            else:
                self._preempt(self.live[-1], plan)
                inner = self.plan()
                inner.preempted = plan.preempted + inner.preempted
                inner.finished = plan.finished + inner.finished
                return inner
        return plan

    # ---- stepping -------------------------------------------------------------------------
    def _finish(self, r: Request, reason: str) -> None:
        r.status, r.finish_reason = FINISHED, reason
        if self.cache.is_open(r.id):
            self.cache.cancel(r.id)
            self.cache.close(r.id)
        if r in self.live:
            self.live.remove(r)
        self.finished[r.id] = r

    def step(self) -> List[Tuple[object, Optional[int], bool]]:
        """Plan and run one step.  Returns [(request id, new token or None, finished)] for requests that
        got a token or finished in this step.

        Looking ahead.  What the step after this one holds does not depend on the tokens this one samples, only on
        whether they end a request (see ``_plan_ahead``).  So the next step -- decodes, prompt portions, admissions --
        is planned and launched BEFORE this step's tokens are read; the device feeds it the sampled ids itself
        (executor's `feed`), and the host does its planning while the device works.  A request that turns out to have
        met a stop token in this step has one more row computed in the next; that row is dropped when its turn comes.
        A step launched ahead is the next call's step."""
        plan = handle = None
        if self._ahead is not None:
            plan, handle = self._ahead
            self._ahead = None
            if all(e.request.status == FINISHED for e in plan.entries):
                plan = handle = None         # every request of it ended in the step before: nothing to collect
        ended_by_plan: List[object] = []
        if plan is None:
            plan = self.plan()
            ended_by_plan = plan.finished
            if not plan.entries:
                return [(rid, None, True) for rid in ended_by_plan]
            # A step that fails to launch leaves nothing behind: the executor gives the reservations back, and what
            # planning did (admissions, preemptions) stands as a consistent state from which the next call plans anew.
            # Requests that planning itself ended are reported by that call.
            try:
                handle = self.executor.launch(plan) if hasattr(self.executor, "launch") else None
            except BaseException:
                self._ended_unreported.extend(ended_by_plan)
                raise
        if self._ended_unreported:
            ended_by_plan = self._ended_unreported + list(ended_by_plan)
            self._ended_unreported = []
        advanced = False
        if handle is not None and self.params.look_ahead:
            nxt = self._plan_ahead(plan)
            if nxt is not None:
                # (the tokens this step will bring stand in their requests as marks now, see _plan_ahead)
                advanced = True
                rows = {e.request.id: j for j, e in enumerate(e2 for e2 in plan.entries if e2.wants_token)}
                try:
                    self._ahead = (nxt, self.executor.launch(nxt, feed_rows=rows))
                    self.stats["steps_launched_ahead"] += 1
                except Exception:
                    # the step ahead could not be launched (its reservations are given back already): take the marks
                    # out again and go on as if it had not been tried; the next call plans and launches it in its turn,
                    # and a fault that lasts is raised from there
                    advanced = False
                    self._ahead = None
                    self._unmark(plan)
                    self.stats["ahead_launches_failed"] = self.stats.get("ahead_launches_failed", 0) + 1
        if handle is not None:
            sampled: Dict[object, int] = self.executor.wait(handle)
        else:
            try:
                sampled = self.executor.run(plan)
            except BaseException:
                for e in plan.entries:             # an executor without `launch`: the plan's pages are still reserved
                    if self.cache.is_open(e.request.id):
                        self.cache.cancel(e.request.id)
                self._ended_unreported.extend(ended_by_plan)
                raise
        self.stats["steps"] += 1
        self.stats["max_batch"] = max(self.stats["max_batch"], len(plan.entries))
        out = [(rid, None, True) for rid in ended_by_plan]
        limit = self.cache.max_pages_per_request * self.cache.page_size
        for e in plan.entries:
            r = e.request
            if r.status == FINISHED:
                continue                     # it stopped in the step before; this row was computed for nothing
            if not advanced:
                r.computed += e.count
            if e.count == 1 and r.generated:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += e.count
            if not e.wants_token:
                continue
            tok = int(sampled[r.id])
            if advanced:
                r.tokens.pop()               # the mark; the token itself is appended below if the request goes on
            r.sampler.accept(tok)
            if not r.ignore_eos and tok in r.stop_ids:            # src/engine.c:1849-1854
                self._finish(r, "stop")
                out.append((r.id, None, True))
                continue
            r.generated.append(tok)
            r.tokens.append(tok)
            done = None
            if 0 < r.max_new_tokens <= len(r.generated):
                done = "length"
            elif len(r.tokens) >= limit:                            # src/engine.c:1834
                done = "length"
            if done:
                self._finish(r, done)
            out.append((r.id, tok, done is not None))
        return out

    def _unmark(self, plan: StepPlan) -> None:
        for e in plan.entries:
            e.request.computed -= e.count
            if e.wants_token:
                e.request.tokens.pop()

    def _plan_ahead(self, plan: StepPlan) -> Optional[StepPlan]:
        """The step after `plan`, planned while `plan` runs.  What the next step holds does not depend on the tokens
        that `plan` samples, only on whether they end a request: a prompt's next portion is known, a request that
        gets a token decodes one more (the device feeds it the token itself), waiting requests are admitted by the
        slots and pages that are free now.  A request that reaches its length with this step's token is known to
        end and is left out; one that meets a stop token is not, and has one row computed for nothing.  Not planned
        ahead: a step whose sampling needs the token on the host (a repeat-penalty window with an executor that cannot
        complete it on the device), and a step that would have to preempt or end a request (``plan`` decides that with the outcome in hand).  On success the tokens to come
        stand in their requests as IN_FLIGHT marks and the next step's pages are reserved; else nothing is changed."""
        limit = self.cache.max_pages_per_request * self.cache.page_size
        ending = []
        for e in plan.entries:
            r = e.request
            if r.status != LIVE:
                return None                  # it ended in the step before this one: let the queue settle first
            if e.wants_token:
                if r.sampler.needs_window() and not (getattr(self.executor, "windows_on_device", False) and r.sampler.window_on_device_ok()):
                    return None
                if 0 < r.max_new_tokens <= len(r.generated) + 1 or len(r.tokens) + 1 >= limit:
                    ending.append(r)
        for e in plan.entries:
            e.request.computed += e.count
            if e.wants_token:
                e.request.tokens.append(IN_FLIGHT)
        try:
            nxt = self.plan(ahead=True, skip=_IdentitySet(ending))
        except _NoLookAhead:
            nxt = None
        if nxt is None or not nxt.entries:
            if nxt is not None:
                self._undo(nxt)
            self._unmark(plan)
            return None
        return nxt

    def run_to_completion(self, max_steps: int = 1 << 30) -> None:
        n = 0
        while self.has_work() and n < max_steps:
            before = len(self.finished)
            res = self.step()
            n += 1
            if not res and not self.has_work():
                break
            if not res and len(self.finished) == before and not self.live and self.waiting:
                # nothing live and the head of the queue cannot be admitted: it can never run
                r = self.waiting.popleft()
                self._finish(r, "rejected")
