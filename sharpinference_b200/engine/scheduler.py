"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  It decides; the step function runs what it decided.

Reference: ``ContinuousBatchingEngine.BatcherLoop`` (src/SharpInference.Engine/ContinuousBatchingEngine.cs:257-502):
FIFO admission under a batch-slot limit and a reservation of ``prompt + max_new`` cache tokens
(:511-580), a prefill budget split over the prompts being prefilled (:588-684), then one decode
step for every active sequence (:314-347), retirement on a stop token, ``MaxNewTokens`` or
cancellation (:394-407).  Differences, because pages are taken as needed instead of reserved up
front: one step mixes decodes and prompt portions; and pages can run out mid-flight, which is
decided as follows.

**When pages run out.**  Decodes come first.  If the running requests' next tokens do not all
fit, the most recently admitted running request is *preempted*: its pages and state slot are
given back, it returns to the FRONT of the waiting queue, and when it is admitted again it is
recomputed from its prompt and the tokens it had generated (its sampler stream and its output
continue where they were).  This repeats until the rest fits.  A request that does not fit even
when it is the only one running can never finish: it ends with ``finish_reason="cache_full"``
and the others go on.  Prompt portions only take pages that decodes left over; a portion shrinks
to what fits, and a waiting request is admitted only when at least one of its tokens fits.  A
plan that preempted admits nobody: the request it sent back would otherwise return at once and
be sent back again.

**More decodes than the token budget.**  The requests that ran least recently go first (ties:
the one that has generated least, then the older one), so every running request gets its turn
equally often; pages are taken only for the decodes that are planned.

**Failures.**  ``fail`` ends one request with ``finish_reason="error"`` and the message;
``fail_all`` ends every running and waiting request that way.  The reference's batching loop
does the same: a request that cannot be prepared fails alone (ContinuousBatchingEngine.cs:529-535),
a failed pass fails the requests in it (:662-672), a loop that dies completes everything in
flight with the error and disposes the caches (:465-501).
"""
from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence, Tuple

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams
from ..sampling.sampler import SamplerState

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    request_id: Hashable
    prompt: List[int]
    params: SamplingParams
    stop_set: Tuple[int, ...] = ()
    generated: List[int] = field(default_factory=list)
    status: str = WAITING
    computed: int = 0                   # tokens of prompt + generated whose keys and values are cached
    finish_reason: Optional[str] = None
    stop_token: Optional[int] = None
    admitted_order: int = -1
    preemptions: int = 0
    sampler: Optional[SamplerState] = None
    last_step: int = -1                 # number of the last step that ran tokens of this request
    error: Optional[str] = None         # why, when finish_reason is "error"

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    def token_slice(self, start: int, count: int) -> List[int]:
        """``tokens[start:start + count]`` without building the whole list (a decode step asks for one token
        of a sequence that may be very long)."""
        n = len(self.prompt)
        if start >= n:
            return self.generated[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.generated[:start + count - n]

    @property
    def pending(self) -> int:
        """Tokens not yet run: the rest of the prompt, or the one token sampled last."""
        return len(self.prompt) + len(self.generated) - self.computed


@dataclass
class PlannedEntry:
    request: Request
    start: int          # index into request.tokens of the first token of the portion
    count: int
    want_last: bool     # the portion reaches the request's last token: sample from its last row


@dataclass
class StepPlan:
    entries: List[PlannedEntry] = field(default_factory=list)
    preempted: List[Request] = field(default_factory=list)
    failed: List[Request] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batch: int, max_tokens_per_step: int):
        if max_batch <= 0 or max_tokens_per_step <= 0:
            raise ValueError("max_batch and max_tokens_per_step must be positive")
        self.cache = cache
        self.max_batch = min(max_batch, cache.max_requests)
        self.max_tokens_per_step = max_tokens_per_step
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []            # in admission order
        self._order = itertools.count()
        # counters
        self.num_preemptions = 0
        self.num_finished = 0
        self.num_steps = 0

    # -- intake --------------------------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError(f"request {request.request_id!r}: the prompt is empty")
        request.status = WAITING
        self.waiting.append(request)

    def abort(self, request_id: Hashable) -> Optional[Request]:
        for req in list(self.running):
            if req.request_id == request_id:
                self._finish(req, "abort")
                return req
        for req in list(self.waiting):
            if req.request_id == request_id:
                self.waiting.remove(req)
                req.status, req.finish_reason = FINISHED, "abort"
                return req
        return None

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- planning ------------------------------------------------------------------------
    def _fits(self, req: Request, n: int, left: Dict[int, int]) -> bool:
        need = self.cache.pages_needed(req.request_id, n)
        return all(need[g] <= left[g] for g in need)

    def _take(self, req: Request, n: int, left: Dict[int, int]) -> None:
        for g, k in self.cache.pages_needed(req.request_id, n).items():
            left[g] -= k

    def _largest_fit(self, req: Request, n_max: int, left: Dict[int, int]) -> int:
        if n_max <= 0 or self._fits(req, n_max, left):
            return max(n_max, 0)
        lo, hi = 0, n_max            # fits(lo) holds (0 tokens need nothing), fits(hi) does not
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if self._fits(req, mid, left):
                lo = mid
            else:
                hi = mid
        return lo

    def _preempt(self, req: Request, plan: StepPlan) -> None:
        self.cache.free_request(req.request_id)
        self.running.remove(req)
        req.status, req.computed = WAITING, 0
        req.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)
        plan.preempted.append(req)

    def _finish(self, req: Request, reason: str) -> None:
        if req.status == RUNNING:
            self.cache.free_request(req.request_id)
            self.running.remove(req)
        elif req.status == WAITING and req in self.waiting:
            self.waiting.remove(req)
        req.status, req.finish_reason = FINISHED, reason
        self.num_finished += 1

    def fail(self, req: Request, error: str) -> None:
        """End one request with ``finish_reason="error"``; its pages and state slot are given back."""
        if req.status == FINISHED:
            return
        req.error = error
        self._finish(req, "error")

    def fail_all(self, error: str) -> List[Request]:
        """End every running and every waiting request with the error.  Returns them."""
        failed = list(self.running) + list(self.waiting)
        for req in failed:
            self.fail(req, error)
        return failed

    def preempt_newest(self, plan: Optional[StepPlan] = None) -> Optional[Request]:
        """The out-of-pages rule, applied from outside a plan (the step function found fewer pages than the
        plan counted on): the newest running request goes back to the queue; alone, it ends ``cache_full``."""
        if not self.running:
            return None
        victim = self.running[-1]
        plan = plan if plan is not None else StepPlan()
        if len(self.running) == 1:
            self._finish(victim, "cache_full")
            plan.failed.append(victim)
        else:
            self._preempt(victim, plan)
        return victim

    def plan(self) -> StepPlan:
        plan = StepPlan()
        budget = self.max_tokens_per_step

        # 1. decodes: every running request whose prompt is done brings its one pending token; if there are
        # more of them than the budget, those that ran least recently.
        while True:
            left = dict(self.cache.free_pages())
            decodes = [r for r in self.running if r.pending == 1 and r.computed >= len(r.prompt)]
            if len(decodes) > budget:
                decodes = sorted(decodes, key=lambda r: (r.last_step, len(r.generated), r.admitted_order))[:budget]
            ok = True
            for req in decodes:
                need = self.cache.pages_needed(req.request_id, 1)
                if any(k > left[g] for g, k in need.items()):
                    ok = False
                    break
                for g, k in need.items():
                    left[g] -= k
            if ok:
                break
            victim = self.running[-1]
            if len(self.running) == 1:
                self._finish(victim, "cache_full")
                plan.failed.append(victim)
            else:
                self._preempt(victim, plan)
        for req in decodes:
            plan.entries.append(PlannedEntry(req, req.computed, 1, True))
        budget -= len(plan.entries)
        planned = {e.request.request_id for e in plan.entries}

        # 2. portions of prompts already admitted, oldest first.
        for req in self.running:
            if budget <= 0:
                break
            if req.request_id in planned or req.pending <= 0:
                continue
            n = self._largest_fit(req, min(req.pending, budget), left)
            if n <= 0:
                continue
            self._take(req, n, left)
            plan.entries.append(PlannedEntry(req, req.computed, n, n == req.pending))
            planned.add(req.request_id)
            budget -= n

        # 3. admission, first come first served; a request enters only if a token of it fits, and nobody
        # enters a plan that had to send a request back.
        while self.waiting and budget > 0 and len(self.running) < self.max_batch \
                and self.cache.state_slots.free_count > 0 and not plan.preempted:
            req = self.waiting[0]
            self.cache.add_request(req.request_id)
            n = self._largest_fit(req, min(req.pending, budget), left)
            if n <= 0:
                self.cache.free_request(req.request_id)
                if not self.running:
                    # alone and still no room for one token: it can never run
                    self.waiting.popleft()
                    req.status, req.finish_reason = FINISHED, "cache_full"
                    self.num_finished += 1
                    plan.failed.append(req)
                    continue
                break
            self.waiting.popleft()
            req.status = RUNNING
            req.admitted_order = next(self._order)
            self.running.append(req)
            self._take(req, n, left)
            plan.entries.append(PlannedEntry(req, req.computed, n, n == req.pending))
            budget -= n

        # A running request that holds pages but could not move while nothing else moves either
        # would wait for ever: the cache is too small for it.
        if not plan.entries and self.running and not plan.preempted:
            victim = self.running[-1]
            if len(self.running) == 1:
                self._finish(victim, "cache_full")
                plan.failed.append(victim)
            else:
                self._preempt(victim, plan)
        return plan

    # -- after the step --------------------------------------------------------------------
    def complete(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """Record the step: ``sampled`` holds one token for every planned entry with ``want_last``,
        in plan order.  Returns the requests that finished."""
        finished = []
        it = iter(sampled)
        self.num_steps += 1
        for e in plan.entries:
            req = e.request
            req.computed += e.count
            req.last_step = self.num_steps
            if not e.want_last:
                continue
            token = int(next(it))
            if token in req.stop_set:
                req.stop_token = token
                self._finish(req, "stop")
                finished.append(req)
                continue
            req.generated.append(token)
            if len(req.generated) >= req.params.max_new_tokens:
                self._finish(req, "length")
                finished.append(req)
        return finished
