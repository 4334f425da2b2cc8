"""The scheduler: which request runs which of its pending tokens in the next step.

A step is planned in ONE pass over the requests in order of seniority (arrival), against a `Budget` that is set up
before the pass. What a request asks for is its pending tokens (`Request.pending`): one for a request that generates,
the next part of the prompt for one that is still reading it, everything it knows for one that lost its pages. The
policy is the reference scheduler's (fusezap/serve/scheduler.py:1-19, 235-298), which this engine keeps:

  * first come, first served; the head of the queue is never overtaken by a request behind it;
  * rows for the requests that generate are set aside first (one each), the prompt budget is what is left, capped by
    `max_prefill_tokens`, and further by `mixed_prefill_tokens` / `prefill_every` while someone generates
    (scheduler.py:265-268); at most `max_prefill_seqs` requests get a prompt portion in one step (scheduler.py:271-285);
  * a waiting request is admitted while the prompt budget, `max_num_seqs` and the free pages allow
    (scheduler.py:286-298);
  * `prefill_first = n`: while prompt work is pending and some request generates, up to n consecutive steps run prompt
    portions alone and the generating requests wait, then one step includes them again (scheduler.py:145-167, 235-251).

All rows of a step run as one batch (the reference runs prompt portions and generated tokens as two forwards).

Out of pages (scheduler.py:120-138, 256-259): a request that needs a page takes it from the *most junior* live request
junior to itself (`CacheManager.reclaim` frees the victims); since the pass goes by seniority, nothing junior has been
planned yet when a senior request asks, so a victim never runs in the step that evicted it. The victim keeps what it
generated, gives back every page and queues again at its old place in line; once admitted again, all it knows is
pending and is recomputed in portions (nothing is sampled twice). A generating request with nobody junior to take from
steps back itself; a prompt portion in that position shrinks to what the free pages hold. The most senior request
therefore always makes progress, and since `submit` refuses a request that could not fit the cache alone, every
request ends.
"""
from __future__ import annotations
import bisect
from dataclasses import dataclass, field

from ..cache import CacheManager
from ..config import EngineConfig
from .request import Phase, Request


@dataclass
class Work:
    """One request's share of a step: `count` tokens from position `start`."""
    request: Request
    start: int
    count: int
    decode: bool         # a single generated token (its logits are always wanted)


@dataclass
class StepPlan:
    work: list[Work] = field(default_factory=list)
    evicted: list[Request] = field(default_factory=list)
    held_back: int = 0   # generating requests that wait in this step (prefill-first)

    @property
    def decode(self) -> list[Request]:
        return [w.request for w in self.work if w.decode]

    @property
    def portions(self) -> list[tuple[Request, int, int]]:
        return [(w.request, w.start, w.count) for w in self.work if not w.decode]

    @property
    def num_tokens(self) -> int:
        return sum(w.count for w in self.work)

    @property
    def empty(self) -> bool:
        return not self.work


@dataclass
class Budget:
    """What a step may still take while it is planned."""
    decode_rows: int      # rows set aside for generated tokens
    prompt_rows: int      # rows for prompt portions
    portions: int         # requests that may still get a portion

    def portion(self, wanted: int) -> int:
        return min(wanted, self.prompt_rows) if self.portions > 0 else 0

    def spend_portion(self, n: int) -> None:
        self.prompt_rows -= n
        self.portions -= 1


class Scheduler:
    def __init__(self, cfg: EngineConfig, cache: CacheManager):
        if cfg.max_model_len is None or cfg.max_prefill_tokens is None:
            cfg = cfg.resolved(cache.max_model_len)
        self.cfg, self.cache = cfg, cache
        self.queue: list[Request] = []      # by seniority; an evicted request returns to its place, ahead of later arrivals
        self.live: list[Request] = []       # by seniority
        self.steps = 0
        self.evictions = 0
        self.streak = 0                     # consecutive steps that held the generating requests back
        self.steps_held_back = 0

    # ---- requests in and out
    @property
    def capacity(self) -> int:
        return self.cache.capacity_tokens

    def has_unfinished(self) -> bool:
        return bool(self.queue or self.live)

    def submit(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("empty prompt")
        most = len(req.prompt) + req.params.max_tokens
        if most > self.capacity:
            raise ValueError(f"prompt ({len(req.prompt)}) + max_tokens ({req.params.max_tokens}) = {most} exceeds the "
                             f"cache's capacity of {self.capacity} tokens for one request")
        req.phase = Phase.QUEUED
        self._enqueue(req)

    def retire(self, req: Request, why: str) -> None:
        """The request ends (`why`: stop, length or abort) and gives back what it holds."""
        self.cache.free(req.rid)
        for line in (self.live, self.queue):
            if req in line:
                line.remove(req)
        req.phase, req.ended_by, req.ended_in = Phase.DONE, why, self.steps

    def evict(self, req: Request) -> None:
        """The request gives back its pages and queues again; what it knows will be recomputed."""
        self.cache.free(req.rid)
        self._requeue(req)

    def _requeue(self, req: Request) -> None:
        self.live.remove(req)
        req.cached, req.phase, req.evicted_in = 0, Phase.QUEUED, self.steps
        req.evictions += 1
        self.evictions += 1
        self._enqueue(req)

    def _enqueue(self, req: Request) -> None:
        bisect.insort(self.queue, req, key=lambda r: r.order)

    # ---- one step
    def plan(self) -> StepPlan:
        self.steps += 1
        generating = [r for r in self.live if r.decoding]
        plan = StepPlan()
        if generating and self.cfg.prefill_first > self.streak and self._prompt_work():
            self._pass(plan, hold=True, generating=len(generating))
            if plan.work:
                self.streak += 1
                self.steps_held_back += 1
                plan.held_back = len(generating)
                return plan
        self._pass(plan, hold=False, generating=sum(1 for r in self.live if r.decoding))
        if plan.decode:
            self.streak = 0
        return plan

    def _prompt_work(self) -> bool:
        if any(not r.decoding for r in self.live):
            return True
        return bool(self.queue) and len(self.live) < self.cfg.max_num_seqs and self.queue[0].evicted_in != self.steps

    def _budget(self, hold: bool, generating: int) -> Budget:
        cfg = self.cfg
        rows = cfg.token_budget
        decode_rows = 0 if hold else min(generating, rows)
        prompt_rows = min(cfg.max_prefill_tokens, rows - decode_rows)
        if decode_rows:
            if cfg.mixed_prefill_tokens:
                prompt_rows = min(prompt_rows, cfg.mixed_prefill_tokens)
            if cfg.prefill_every > 1 and self.steps % cfg.prefill_every:
                prompt_rows = 0
        return Budget(decode_rows, prompt_rows, cfg.max_prefill_seqs or cfg.max_num_seqs)

    def _pass(self, plan: StepPlan, hold: bool, generating: int) -> None:
        cache, budget = self.cache, self._budget(hold, generating)
        # live requests, most senior first
        for req in list(self.live):
            if req.phase is not Phase.LIVE:          # evicted by a senior request earlier in this pass
                continue
            if req.decoding:
                if hold or budget.decode_rows <= 0:
                    continue
                if not self._room(req, req.cached + 1, plan):
                    self.evict(req)
                    plan.evicted.append(req)
                    continue
                cache.ensure(req.rid, req.cached + 1)
                plan.work.append(Work(req, req.cached, 1, True))
                budget.decode_rows -= 1
                continue
            n = budget.portion(req.pending)
            if n <= 0:
                continue
            if not self._room(req, req.cached + n, plan):
                n = self._most_that_fits(req, n)
                if n <= 0:
                    continue
            cache.ensure(req.rid, req.cached + n)
            plan.work.append(Work(req, req.cached, n, False))
            budget.spend_portion(n)
        # admissions, in line order; whoever is at the head is never overtaken
        while self.queue and len(self.live) < self.cfg.max_num_seqs:
            req = self.queue[0]
            n = budget.portion(req.pending)
            if n <= 0 or req.evicted_in == self.steps or not cache.can_ensure(req.rid, n):
                break
            self.queue.pop(0)
            req.phase = Phase.LIVE
            if req.admitted_in < 0:
                req.admitted_in = self.steps
            bisect.insort(self.live, req, key=lambda r: r.order)
            cache.ensure(req.rid, n)
            plan.work.append(Work(req, 0, n, False))
            budget.spend_portion(n)

    def _room(self, req: Request, n_tokens: int, plan: StepPlan) -> bool:
        """Pages for `req` to hold n_tokens, taken from live requests junior to it if need be, most junior first."""
        if self.cache.can_ensure(req.rid, n_tokens):
            return True
        juniors = {r.rid: r for r in reversed(self.live) if r.order > req.order}
        for rid in self.cache.reclaim(req.rid, n_tokens, juniors):
            self._requeue(juniors[rid])
            plan.evicted.append(juniors[rid])
        return self.cache.can_ensure(req.rid, n_tokens)

    def _most_that_fits(self, req: Request, n: int) -> int:
        """The most tokens (at most n) of req's next portion that the free pages can back."""
        lo, hi = 0, n
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.cache.can_ensure(req.rid, req.cached + mid):
                lo = mid
            else:
                hi = mid - 1
        return lo
