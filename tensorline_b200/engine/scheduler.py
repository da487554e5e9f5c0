"""Continuous-batching scheduler: which request runs how many tokens in the next step.

Host logic only; it owns no tensors and calls no kernels, so its decisions are testable without a
GPU.  `schedule()` builds a typed `Plan` in two phases under one token budget of
`max_batched_tokens` (the rules of tzar-beep/Tensorline's `BatchEngine._schedule`,
tensorline/batch_engine.py:314-356):

1. *serve what runs*, in order of admission: a decoding request asks for one token, a request
   whose prompt (or recomputed history) is not through asks for the rest of it, cut to what is
   left of the budget: chunked prefill.  If the cache cannot make room, a victim chosen by the
   *preemption policy* (default: the request admitted last, batch_engine.py:325-334) gives back
   all it holds, goes to the front of the queue and is later recomputed from its first token,
   prompt and generated tokens alike (batch_engine.py:292-298); the budget it had been given in
   this plan is returned.
2. *admit what waits*, in order of arrival, while budget, the sequence limit and pages allow.  A
   request at the head of the queue that cannot get its pages waits and holds nothing meanwhile;
   if nothing is running it will never fit, and fails (batch_engine.py:337-347).

Two decisions are this engine's own.  Before a request would have to give up its *own* pages
(it is the policy's victim, or nothing else runs), its portion is cut to the room the cache still
has: with a window, a long prompt needs pages for window + portion tokens, and a smaller portion
may fit where the whole budget does not.  And a request that could not lie in the empty cache is
failed with `RequestDoesNotFit` (also when it outgrows the pool while decoding alone) instead of
being recomputed for ever.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

from ..cache import CacheManager
from ..sampling.params import GenStats, SamplingParams


@dataclass(eq=False)
class Request:
    rid: int
    prompt_len: int
    tokens: list
    params: SamplingParams
    stops: set
    stats: GenStats = field(default_factory=GenStats)
    t_submit: float = 0.0
    num_computed: int = 0               # tokens whose cache entries are written
    done: bool = False
    admitted_once: bool = False
    error: Exception | None = None
    seed: int = 0                       # seed of this request's sampling draws

    @property
    def num_generated(self) -> int:
        return len(self.tokens) - self.prompt_len

    @property
    def output_tokens(self) -> list:
        return self.tokens[self.prompt_len:]

    @property
    def remaining(self) -> int:
        """Tokens known but not yet in the cache: the rest of a prompt, or the one token to decode."""
        return len(self.tokens) - self.num_computed


class RequestDoesNotFit(RuntimeError):
    pass


@dataclass
class Slice:
    """One request's share of a step: `count` tokens from position `start` on."""
    request: Request
    start: int
    count: int

    @property
    def wants_logits(self) -> bool:
        """Only a slice that ends at the request's last known token samples (batch_engine.py:376)."""
        return self.start + self.count == len(self.request.tokens)

    @property
    def tokens(self) -> list:
        return self.request.tokens[self.start:self.start + self.count]


@dataclass
class Plan:
    """What one call of `schedule()` decided."""
    slices: list = field(default_factory=list)
    admitted: list = field(default_factory=list)        # requests that entered the running set
    preempted: list = field(default_factory=list)       # requests sent back to the queue
    failed: list = field(default_factory=list)          # requests that can never fit

    def __bool__(self) -> bool:
        return bool(self.slices)

    def __len__(self) -> int:
        return len(self.slices)

    def __iter__(self):
        return iter(self.slices)

    @property
    def num_tokens(self) -> int:
        return sum(s.count for s in self.slices)

    def kinds(self) -> tuple:
        """(decoded tokens, prompt-portion tokens) of the step."""
        ones = sum(1 for s in self.slices if s.count == 1 and s.start > 0 and s.wants_logits)
        return ones, self.num_tokens - ones

    def withdraw(self, req: Request) -> int:
        """Take `req` out of the plan; returns the tokens it had been given."""
        back = sum(s.count for s in self.slices if s.request is req)
        self.slices = [s for s in self.slices if s.request is not req]
        return back


def newest_first(running: list) -> Request:
    """The request admitted last gives way (tensorline/batch_engine.py:327)."""
    return running[-1]


def least_computed_first(running: list) -> Request:
    """The request that is cheapest to recompute gives way; among equals the newest."""
    return min(reversed(running), key=lambda r: r.num_computed)


PREEMPTION_POLICIES = {"newest": newest_first, "least_computed": least_computed_first}


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_num_seqs: int, max_batched_tokens: int, max_model_len: int,
                 preemption="newest"):
        """`preemption`: a name from PREEMPTION_POLICIES or a function (running requests in order of
        admission) -> the one that gives way."""
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_batched_tokens = max_batched_tokens
        self.max_model_len = max_model_len
        self.pick_victim = PREEMPTION_POLICIES[preemption] if isinstance(preemption, str) else preemption
        self.waiting: deque = deque()
        self.running: list = []
        self.failed: list = []          # requests failed by the last schedule() call
        # counters (tensorline/batch_engine.py:119-125)
        self.steps = 0
        self.preemptions = 0
        self.max_running_seen = 0
        self.prompt_tokens_total = 0
        self.prefix_hit_tokens = 0
        self.finished = {}              # finish reason -> count

    # ------------------------------------------------------------------ queue
    def add(self, req: Request) -> None:
        if req.prompt_len >= self.max_model_len:          # tensorline/batch_engine.py:173-174
            raise ValueError(f"prompt has {req.prompt_len} tokens; max_model_len is {self.max_model_len}")
        if req.prompt_len < 1:
            raise ValueError("a request needs at least one prompt token")
        req.stats.prompt_tokens = req.prompt_len
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ decisions
    def _give_back(self, req: Request) -> None:
        if self.cache.holds(req.rid):
            self.cache.release(req.rid)

    def preempt(self, req: Request) -> None:
        """Recompute-style preemption: everything is given back, the request waits at the front."""
        self.running.remove(req)
        self._give_back(req)
        req.num_computed = 0
        self.waiting.appendleft(req)
        self.preemptions += 1

    def schedule(self) -> Plan:
        """The next step's plan."""
        plan = Plan()
        left = self._serve_running(plan, self.max_batched_tokens)
        self._admit_waiting(plan, left)
        self.failed = plan.failed
        if plan:
            self.max_running_seen = max(self.max_running_seen, len(self.running))
        return plan

    def _reserve(self, req: Request, ask: int, plan: Plan, left: int) -> tuple:
        """Pages for `ask` more tokens of the running request `req`.  Others give way by the policy;
        when it would be `req` itself, the portion is first cut to the room there is.  Returns
        (tokens granted, budget left); 0 tokens if `req` was preempted or has to sit this step out."""
        while not self.cache.grow(req.rid, req.num_computed, req.num_computed + ask):
            victim = self.pick_victim(self.running)
            if victim is req:
                room = min(ask - 1, self.cache.room_for(req.rid, req.num_computed))
                if room >= 1 and self.cache.grow(req.rid, req.num_computed, req.num_computed + room):
                    return room, left
                self.preempt(req)
                plan.preempted.append(req)
                return 0, left
            self.preempt(victim)
            plan.preempted.append(victim)
            left += plan.withdraw(victim)
        return ask, left

    def _serve_running(self, plan: Plan, left: int) -> int:
        for req in list(self.running):                   # in order of admission
            if req not in self.running:                  # gave way to an older one in this pass
                continue
            ask = min(req.remaining, left)
            if ask <= 0:
                continue
            got, left = self._reserve(req, ask, plan, left)
            if got:
                plan.slices.append(Slice(req, req.num_computed, got))
                left -= got
        return left

    def _admit_waiting(self, plan: Plan, left: int) -> int:
        while self.waiting and left > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            cached = self.cache.admit(req.rid, req.tokens)
            if cached is None:                           # no slot
                break
            req.num_computed = cached
            ask = min(req.remaining, left)
            alone = not self.running
            fits = not (alone and not self.cache.can_ever_hold(len(req.tokens)))
            if fits and not self.cache.grow(req.rid, cached, cached + ask):
                room = min(ask, self.cache.room_for(req.rid, cached)) if alone else 0
                fits = room >= 1 and self.cache.grow(req.rid, cached, cached + room)
                ask = room
            if not fits:
                self._give_back(req)                     # it holds nothing while it waits
                req.num_computed = 0
                if not alone:
                    break                                # room will come when others finish
                self.waiting.popleft()                   # alone and still no room: it never will fit
                req.done = True
                req.error = RequestDoesNotFit("request does not fit in the KV cache")
                plan.failed.append(req)
                continue
            self.waiting.popleft()
            self.running.append(req)
            plan.admitted.append(req)
            if not req.admitted_once:                    # not a re-admission after preemption
                req.admitted_once = True
                req.stats.cached_tokens = cached
                self.prompt_tokens_total += req.prompt_len
                self.prefix_hit_tokens += cached
            plan.slices.append(Slice(req, cached, ask))
            left -= ask
        return left

    # ------------------------------------------------------------------ after a step
    def computed(self, plan) -> None:
        """The step ran: count its tokens as cached and offer full pages for sharing."""
        self.steps += 1
        for s in plan:
            s.request.num_computed += s.count
            self.cache.advance(s.request.rid, s.request.num_computed, s.request.tokens)

    def accept(self, req: Request, tok: int, now: float | None = None) -> bool:
        """Take one sampled token (tensorline/batch_engine.py:395-406).  A stop token ends the
        request and is not kept; returns True if the token was appended."""
        now = time.perf_counter() if now is None else now
        if req.num_generated == 0:
            req.stats.ttft_s = now - req.t_submit
        if tok in req.stops:
            self.finish(req, "stop", now)
            return False
        req.tokens.append(tok)
        if req.num_generated >= req.params.max_tokens or len(req.tokens) >= self.max_model_len:
            self.finish(req, "length", now)
        return True

    def finish(self, req: Request, reason: str, now: float | None = None) -> None:
        now = time.perf_counter() if now is None else now
        req.done = True
        req.stats.finish_reason = reason
        req.stats.completion_tokens = req.num_generated
        req.stats.total_s = now - req.t_submit
        self.finished[reason] = self.finished.get(reason, 0) + 1
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        self._give_back(req)

    def abort(self, req: Request) -> None:
        """Stop a request wherever it is (tensorline/batch_engine.py:300-312)."""
        if not req.done:
            self.finish(req, "abort")

    def fail_all(self, err: Exception) -> list:
        """An error in the step: every request fails and gives back what it holds
        (tensorline/batch_engine.py:568-576)."""
        everyone = self.running + list(self.waiting)
        self.running.clear()
        self.waiting.clear()
        for req in everyone:
            self._give_back(req)
            req.done = True
            req.error = err
        return everyone
