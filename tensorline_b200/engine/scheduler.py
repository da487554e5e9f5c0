"""Continuous-batching scheduler: which request runs how many tokens in the next step.

Host logic only; it owns no tensors and calls no kernels, so its decisions are testable
without a GPU.  The rules are those of tzar-beep/Tensorline's `BatchEngine._schedule`
(tensorline/batch_engine.py:314-356):

* a budget of `max_batched_tokens` tokens per step;
* running requests first, oldest first: a decoding request asks for one token, a request
  whose prompt (or recomputed history) is not through asks for the rest of it, cut to the
  budget: chunked prefill;
* when pages run out the *newest* running request is preempted: all it holds is given back,
  it goes to the front of the waiting queue and is recomputed from its first token later,
  prompt and generated tokens alike (batch_engine.py:292-298, :325-334);
* then waiting requests are admitted in order of arrival while budget, sequence limit and
  pages allow; a request at the head that cannot get its pages waits, unless nothing is
  running, in which case it can never fit and is failed (batch_engine.py:337-347).
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


class RequestDoesNotFit(RuntimeError):
    pass


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_num_seqs: int, max_batched_tokens: int, max_model_len: int):
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_batched_tokens = max_batched_tokens
        self.max_model_len = max_model_len
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
    def _release(self, req: Request) -> None:
        if self.cache.holds(req.rid):
            self.cache.release(req.rid)

    def preempt(self, req: Request) -> None:
        """Recompute-style preemption (tensorline/batch_engine.py:292-298)."""
        self.running.remove(req)
        self._release(req)
        req.num_computed = 0
        self.waiting.appendleft(req)
        self.preemptions += 1

    def schedule(self) -> list:
        """The next step's plan: [(request, number of tokens)]."""
        self.failed = []
        budget = self.max_batched_tokens
        plan: list = []
        for req in list(self.running):                     # oldest first
            if req not in self.running:                    # preempted earlier in this pass
                continue
            n = min(len(req.tokens) - req.num_computed, budget)
            if n <= 0:
                continue
            fits = True
            while not self.cache.grow(req.rid, req.num_computed, req.num_computed + n):
                victim = self.running[-1]                  # the newest
                self.preempt(victim)
                budget += sum(k for r, k in plan if r is victim)
                plan = [(r, k) for r, k in plan if r is not victim]
                if victim is req:
                    fits = False
                    break
            if fits:
                plan.append((req, n))
                budget -= n
        while self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            cached = self.cache.admit(req.rid, req.tokens)
            if cached is None:                             # no slot: wait
                break
            req.num_computed = cached
            n = min(len(req.tokens) - req.num_computed, budget)
            # A request whose tokens can never all lie in the pool would be recomputed for ever.
            hopeless = not self.running and not self.cache.can_ever_hold(len(req.tokens))
            if hopeless or not self.cache.grow(req.rid, req.num_computed, req.num_computed + n):
                self._release(req)                         # drop shared pages while it waits
                req.num_computed = 0
                if not self.running:                       # cannot fit even alone
                    self.waiting.popleft()
                    req.done = True
                    req.error = RequestDoesNotFit("request does not fit in the KV cache")
                    self.failed.append(req)
                    continue
                break
            self.waiting.popleft()
            self.running.append(req)
            if not req.admitted_once:                      # not a re-admission after preemption
                req.admitted_once = True
                req.stats.cached_tokens = req.num_computed
                self.prompt_tokens_total += req.prompt_len
                self.prefix_hit_tokens += req.num_computed
            plan.append((req, n))
            budget -= n
        if plan:
            self.max_running_seen = max(self.max_running_seen, len(self.running))
        return plan

    # ------------------------------------------------------------------ after a step
    def computed(self, plan) -> None:
        """The step ran: count its tokens as cached and publish full pages
        (tensorline/batch_engine.py:387-389)."""
        self.steps += 1
        for req, n in plan:
            req.num_computed += n
            self.cache.advance(req.rid, req.num_computed, req.tokens)

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
        self._release(req)

    def abort(self, req: Request) -> None:
        """Stop a request wherever it is (tensorline/batch_engine.py:300-312)."""
        if not req.done:
            self.finish(req, "abort")

    def fail_all(self, err: Exception) -> list:
        """An error in the step: every request fails and gives back what it holds
        (tensorline/batch_engine.py:568-576)."""
        out = self.running + list(self.waiting)
        for req in out:
            self._release(req)
            req.done = True
            req.error = err
        self.running.clear()
        self.waiting.clear()
        return out
