"""Continuous-batching scheduler over the cache manager.

The reference admits a request only when the pool covers the worst case of every
active request, runs whole-prompt prefills and decode steps as separate forwards
and never preempts (sid/engine/scheduler.py:23-120).  Here one step mixes both:

1. every running request gets tokens first, in admission order: a decoding
   request its one token, a request still in its prompt the next portion, cut
   to what is left of the step's token budget (``max_prefill_tokens``);
2. then waiting requests are admitted first-come first-served while a state
   slot, a place among the ``max_decode_batch`` running requests, budget and
   pages for their first portion are there; the head of the queue blocks the
   rest;
3. pages are reserved as the decisions are made, not for the worst case, so they
   can run out.  When a running request cannot get the pages for its tokens, the
   most recently admitted running request is preempted: its pages and slot go
   back, it returns to the FRONT of the waiting queue with nothing computed, and
   it later recomputes prompt and outputs (the sampled tokens are kept, so the
   text does not change).  The oldest running request is never the victim while
   another one runs; a request that could never fit the pool alone is refused
   when it is added.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass

from ..cache.manager import CacheManager
from .request import Request, RequestState


@dataclass
class Scheduled:
    request: Request
    num_tokens: int


class Scheduler:
    def __init__(self, cache: CacheManager, max_prefill_tokens: int, max_decode_batch: int):
        self.cache = cache
        self.token_budget = int(max_prefill_tokens)
        self.max_running = int(max_decode_batch)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._admitted = 0
        self.num_preemptions = 0

    def add(self, req: Request) -> None:
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- decisions of one step -----------------------------------------------

    def _preempt(self, victim: Request) -> None:
        self.cache.release_slot(victim.slot)
        victim.slot = -1
        victim.num_computed = 0
        victim.state = RequestState.WAITING
        victim.num_preemptions += 1
        self.num_preemptions += 1
        self.running.remove(victim)
        self.waiting.appendleft(victim)

    def schedule(self) -> list[Scheduled]:
        budget = self.token_budget
        out: list[Scheduled] = []
        preempted = False

        # 1. running requests, decoding ones first, each group in admission order
        order = sorted(self.running, key=lambda r: (r.remaining != 1, r.admit_order))
        for req in order:
            if req.state != RequestState.RUNNING or budget <= 0 or req.done_generating:
                continue
            n = min(req.remaining, budget)
            while not self.cache.can_allocate(req.slot, req.num_computed + n):
                victim = max(self.running, key=lambda r: r.admit_order)
                for s in out:
                    if s.request is victim:      # it was given tokens in this step: take them back
                        budget += s.num_tokens
                out = [s for s in out if s.request is not victim]
                self._preempt(victim)
                preempted = True
                if victim is req:
                    break
            if req.state != RequestState.RUNNING:
                continue
            self.cache.allocate(req.slot, req.num_computed + n)
            out.append(Scheduled(req, n))
            budget -= n

        # 2. admissions, first come first served; none in a step that had to preempt
        while not preempted and self.waiting and budget > 0 \
                and len(self.running) < self.max_running and self.cache.num_free_slots > 0:
            req = self.waiting[0]
            n = min(req.remaining, budget)
            if not self.cache.can_allocate(None, req.num_computed + n):
                break
            self.waiting.popleft()
            req.slot = self.cache.allocate_slot()
            req.state = RequestState.RUNNING
            req.admit_order = self._admitted
            self._admitted += 1
            self.running.append(req)
            self.cache.allocate(req.slot, req.num_computed + n)
            out.append(Scheduled(req, n))
            budget -= n
        return out

    # ---- after a step ------------------------------------------------------------

    def release_finished(self) -> list[Request]:
        """Retire every finished request.  A running one gives its pages and slot back.  A
        waiting one can be finished too: it was preempted while its last token was still on
        its way from the device, holds nothing, and must not be admitted again."""
        done = [r for r in self.running if r.finished_reason is not None]
        for r in done:
            self.cache.release_slot(r.slot)
            r.slot = -1
            r.state = RequestState.DONE
            self.running.remove(r)
        late = [r for r in self.waiting if r.finished_reason is not None]
        for r in late:
            r.state = RequestState.DONE
            self.waiting.remove(r)
        return done + late
