"""Continuous-batching scheduler: which request runs which of its tokens in the next step.

Policy, in the manner of the reference's scheduler (fusezap/serve/scheduler.py:1-19, 235-298): first come, first
served. A request's *pending* tokens are the known tokens that are not in the cache yet (`tokens[num_computed:]`): the
whole prompt of a new request, one token of a request that decodes, everything known of a request that lost its pages.
Each step, under the token budget:
  1. requests with one pending token (decoding) get it, oldest first;
  2. running requests with more pending tokens get their next portion, oldest first, under the prompt budget;
  3. waiting requests are admitted in arrival order while the budget, `max_num_seqs` and the free pages allow; the
     head of the queue is never skipped.
All of a step's rows run as one batch (the reference runs prompt portions and decoded tokens as two forwards).

When pages run out (scheduler.py:120-138, 256-259): the request that needs a page takes it from the *newest* running
request that is newer than itself and not already in this step; that victim gives back all its pages, keeps its output
and goes back to the waiting queue ahead of later arrivals; when it is admitted again everything it knows is pending
and is recomputed in portions (nothing is sampled again). A decoding request with nobody newer to take from steps back
itself. The oldest request therefore always progresses, and since `add` refuses a request that could not fit the pool
alone, every request finishes.
"""
from __future__ import annotations
import enum
from collections import deque
from dataclasses import dataclass, field
from typing import Any

from ..cache import CacheManager


class SeqStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(eq=False)
class Sequence:
    seq_id: int
    prompt: list[int]
    params: Any
    arrival: int
    output: list[int] = field(default_factory=list)
    num_computed: int = 0
    status: SeqStatus = SeqStatus.WAITING
    finish_reason: str | None = None
    sampler: Any = None
    num_preemptions: int = 0
    preempted_at: int = -1
    first_step: int = -1
    finish_step: int = -1

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_at(self, i: int) -> int:
        n = len(self.prompt)
        return self.prompt[i] if i < n else self.output[i - n]

    def tokens_between(self, lo: int, hi: int) -> list[int]:
        n = len(self.prompt)
        if hi <= n:
            return self.prompt[lo:hi]
        if lo >= n:
            return self.output[lo - n: hi - n]
        return self.prompt[lo:] + self.output[: hi - n]

    @property
    def num_pending(self) -> int:
        return self.num_tokens - self.num_computed

    @property
    def decoding(self) -> bool:
        return self.num_pending == 1 and self.num_computed > 0


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 32
    max_prefill_tokens: int = 256
    max_num_batched_tokens: int | None = None
    prefill_first: int = 0

    @property
    def token_budget(self) -> int:
        return self.max_num_batched_tokens or (self.max_num_seqs + self.max_prefill_tokens)


@dataclass
class SchedulerOutput:
    decode: list[Sequence] = field(default_factory=list)                    # one token each
    prefill: list[tuple[Sequence, int, int]] = field(default_factory=list)   # (request, first position, tokens)
    preempted: list[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return len(self.decode) + sum(n for _, _, n in self.prefill)

    @property
    def empty(self) -> bool:
        return not self.decode and not self.prefill


class Scheduler:
    def __init__(self, cfg: SchedulerConfig, cache: CacheManager):
        self.cfg, self.cache = cfg, cache
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self.steps = 0
        self.num_preemptions = 0
        self.pf_streak = 0

    @property
    def capacity(self) -> int:
        return self.cache.capacity_tokens

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- requests in and out
    def add(self, seq: Sequence, max_tokens: int) -> None:
        if not seq.prompt:
            raise ValueError("empty prompt")
        need = len(seq.prompt) + max_tokens
        if need > self.capacity:
            raise ValueError(f"prompt ({len(seq.prompt)}) + max_tokens ({max_tokens}) = {need} exceeds the cache's "
                             f"capacity of {self.capacity} tokens for one request")
        seq.status = SeqStatus.WAITING
        self._enqueue(seq)

    def _enqueue(self, seq: Sequence) -> None:
        i = len(self.waiting)
        while i > 0 and self.waiting[i - 1].arrival > seq.arrival:
            i -= 1
        self.waiting.insert(i, seq)

    def finish(self, seq: Sequence, reason: str) -> None:
        seq.status, seq.finish_reason, seq.finish_step = SeqStatus.FINISHED, reason, self.steps
        self.cache.free(seq.seq_id)
        if seq in self.running:
            self.running.remove(seq)
        if seq in self.waiting:
            self.waiting.remove(seq)

    def preempt(self, seq: Sequence) -> None:
        self.cache.free(seq.seq_id)
        self.running.remove(seq)
        seq.num_computed, seq.status, seq.preempted_at = 0, SeqStatus.WAITING, self.steps
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self._enqueue(seq)

    # ---- one step
    def _make_room(self, seq: Sequence, n_tokens: int, out: SchedulerOutput) -> bool:
        busy = {id(s) for s in out.decode} | {id(s) for s, _, _ in out.prefill}
        while not self.cache.can_ensure(seq.seq_id, n_tokens):
            newer = [s for s in self.running if s.arrival > seq.arrival and id(s) not in busy]
            if not newer:
                return False
            victim = max(newer, key=lambda s: s.arrival)
            self.preempt(victim)
            out.preempted.append(victim)
        return True

    def _prompt_work(self) -> bool:
        return any(not s.decoding for s in self.running) or bool(
            self.waiting and len(self.running) < self.cfg.max_num_seqs and self.waiting[0].preempted_at != self.steps)

    def schedule(self) -> SchedulerOutput:
        self.steps += 1
        cfg, out = self.cfg, SchedulerOutput()
        budget = cfg.token_budget
        self.running.sort(key=lambda s: s.arrival)
        if (cfg.prefill_first and self.pf_streak < cfg.prefill_first and any(s.decoding for s in self.running)
                and self._prompt_work()):
            self._portions(out, min(cfg.max_prefill_tokens, budget))
            if out.prefill:
                self.pf_streak += 1
                return out
        # 1. one token for every request that decodes, oldest first
        for seq in list(self.running):
            if seq not in self.running or not seq.decoding:
                continue
            if budget <= 0:
                break
            if not self._make_room(seq, seq.num_computed + 1, out):
                self.preempt(seq)
                out.preempted.append(seq)
                continue
            self.cache.ensure(seq.seq_id, seq.num_computed + 1)
            out.decode.append(seq)
            budget -= 1
        if out.decode:
            self.pf_streak = 0
        # 2 and 3. portions of pending prompts, then admissions
        self._portions(out, min(cfg.max_prefill_tokens, budget))
        return out

    def _portions(self, out: SchedulerOutput, pbudget: int) -> None:
        cfg, cache = self.cfg, self.cache
        for seq in list(self.running):
            if seq not in self.running or seq.decoding or seq in out.decode:
                continue
            if pbudget <= 0:
                break
            n = min(seq.num_pending, pbudget)
            if not self._make_room(seq, seq.num_computed + n, out):
                n = self._largest_fit(seq, n)
                if n <= 0:
                    continue
            cache.ensure(seq.seq_id, seq.num_computed + n)
            out.prefill.append((seq, seq.num_computed, n))
            pbudget -= n
        while self.waiting and pbudget > 0 and len(self.running) < cfg.max_num_seqs:
            seq = self.waiting[0]
            if seq.preempted_at == self.steps:
                break
            n = min(seq.num_pending, pbudget)
            if not cache.can_ensure(seq.seq_id, n):
                n = self._largest_fit(seq, n) if not self.running else 0
                if n <= 0:
                    break
            self.waiting.popleft()
            seq.status = SeqStatus.RUNNING
            if seq.first_step < 0:
                seq.first_step = self.steps
            self.running.append(seq)
            cache.ensure(seq.seq_id, n)
            out.prefill.append((seq, 0, n))
            pbudget -= n

    def _largest_fit(self, seq: Sequence, n: int) -> int:
        """The most tokens (at most n) of seq's next portion that the free pages can back."""
        lo, hi = 0, n
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.cache.can_ensure(seq.seq_id, seq.num_computed + mid):
                lo = mid
            else:
                hi = mid - 1
        return lo
