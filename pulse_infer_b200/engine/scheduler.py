"""Continuous batching with chunked prefill under a token budget, and a decided answer to "the pages
have run out".

Each call of ``schedule_next_batch`` plans one step:

1. every running request that is decoding contributes its one pending token;
2. running requests that are still feeding known tokens (prompt, or a recomputation) get portions, in
   admission order, while the token budget (``max_tokens_per_step``) lasts - a portion is cut to the
   budget, to ``chunk_size`` and to the pages that are free, so portions have any size;
3. waiting requests are admitted first-come-first-served while ``max_batch_size`` / ``max_sequences``
   slots, the token budget and the pages for their first portion allow.

Pages are reserved here, before the step runs, so a step never starts without its pages.  When a
running request needs a page and none is free, the most recently admitted running request is
preempted: its pages are given back, it returns to the FRONT of the waiting queue and later recomputes
prompt plus generated tokens (greedy choices and the counter-based sampler make the outcome the same
as without the preemption).  A request that cannot fit even alone is finished with reason
``out_of_pages`` instead of stalling the engine.

Reference parity: ``include/pulse/scheduler/continuous_batch_scheduler.hpp:49-73`` (all running requests,
then admission from a FIFO queue while ``max_batch_size`` and ``max_sequences`` allow), ``75-89``
(``update_after_step``), ``124-136`` (``Stats``).  The reference has no token budget (each request takes
``min(chunk_size, remaining)``), never looks at free pages, and aborts the run when allocation fails
(``src/scheduler/continuous_batch_engine.cpp:98-101``).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..sampling.params import SamplingParams
from .request import InferenceRequest, RequestState


@dataclass
class ScheduledBatch:
    entries: list = field(default_factory=list)      # (request, number of tokens) in batch order
    preempted: list = field(default_factory=list)    # requests that lost their pages while planning
    failed: list = field(default_factory=list)       # requests finished because they can never fit

    def batch_size(self) -> int:
        return len(self.entries)

    def empty(self) -> bool:
        return not self.entries

    @property
    def requests(self) -> list:
        return [r for r, _ in self.entries]

    @property
    def num_tokens(self) -> int:
        return sum(n for _, n in self.entries)


@dataclass
class Stats:
    num_running: int = 0
    num_waiting: int = 0
    num_finished: int = 0
    total_requests: int = 0
    num_preemptions: int = 0
    num_steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    free_pages: tuple = ()


class ContinuousBatchScheduler:
    def __init__(self, cache, max_batch_size: int, max_sequences: int = 32, chunk_size: int = 256,
                 max_tokens_per_step: int | None = None):
        """``cache``: the cache manager (slots and pages are opened, reserved and closed through it)."""
        if max_batch_size <= 0 or max_sequences <= 0 or chunk_size <= 0:
            raise ValueError("max_batch_size, max_sequences and chunk_size must be positive")
        self.cache = cache
        self.max_batch_size = max_batch_size
        self.max_sequences = max_sequences
        self.chunk_size = chunk_size
        self.max_tokens_per_step = max_tokens_per_step or max_batch_size * chunk_size
        self.waiting_queue: deque = deque()
        self.running_requests: list = []
        self.request_map: dict = {}
        self._next_request_id = 0
        self._decode_turn = 0
        self.stats_preemptions = 0
        self.stats_steps = 0
        self.stats_prefill_tokens = 0
        self.stats_decode_tokens = 0

    # ---- requests ------------------------------------------------------------------------------------
    def add_request(self, prompt_tokens, max_new_tokens: int, sampling: SamplingParams | None = None,
                    ignore_eos: bool = False) -> int:
        if len(prompt_tokens) == 0:
            raise ValueError("a request needs at least one prompt token")
        rid = self._next_request_id
        self._next_request_id += 1
        req = InferenceRequest(rid, list(prompt_tokens), max_new_tokens, sampling or SamplingParams(), ignore_eos)
        self.waiting_queue.append(req)
        self.request_map[rid] = req
        return rid

    def get_request(self, request_id: int):
        return self.request_map.get(request_id)

    def has_work(self) -> bool:
        return bool(self.running_requests) or bool(self.waiting_queue)

    def num_running(self) -> int:
        return len(self.running_requests)

    def num_waiting(self) -> int:
        return len(self.waiting_queue)

    # ---- planning one step ----------------------------------------------------------------------------
    def _fits(self, req: InferenceRequest, tokens: int) -> bool:
        return self.cache.can_reserve(req.request_id, req.num_computed_tokens + tokens)

    def _largest_fitting(self, req: InferenceRequest, tokens: int) -> int:
        """The longest portion <= tokens whose pages are free right now (0 if not even one token)."""
        if self._fits(req, tokens):
            return tokens
        page = self.cache.page_size
        free = min(self.cache.free_pages()) if self.cache.free_pages() else 0
        # tokens that still fit in the request's last page, plus whole free pages
        reserved_end = ((req.num_computed_tokens + page - 1) // page) * page
        room = max(0, reserved_end - req.num_computed_tokens) + free * page
        n = min(tokens, room)
        if n <= 0 or self._fits(req, n):
            return max(n, 0)
        lo, hi = 0, n              # fits(lo) holds (lo = 0 asks for nothing), fits(hi) does not: bisect
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if self._fits(req, mid):
                lo = mid
            else:
                hi = mid
        return lo

    def _preempt(self, victim: InferenceRequest, batch: ScheduledBatch) -> int:
        """Take ``victim`` out of the running set; returns the tokens it had been given in ``batch`` (they go back
        into the step's budget)."""
        self.cache.close(victim.request_id)
        victim.preempt()
        self.running_requests.remove(victim)
        self.waiting_queue.appendleft(victim)
        batch.preempted.append(victim)
        given_back = sum(n for r, n in batch.entries if r is victim)
        batch.entries = [(r, n) for r, n in batch.entries if r is not victim]
        self.stats_preemptions += 1
        return given_back

    def schedule_next_batch(self) -> ScheduledBatch:
        batch = ScheduledBatch()
        budget = self.max_tokens_per_step
        decode_entries: set = set()

        # 1. decoding requests: one token each; make room by preempting the newest request if need be.  When the
        # budget is smaller than the number of decoding requests, the starting point moves on from step to step, so
        # that the same requests are not left out every time.
        decoding = [r for r in self.running_requests if not r.is_prefill() and r.has_pending_input()]
        if len(decoding) > budget > 0:
            turn = self._decode_turn % len(decoding)
            decoding = decoding[turn:] + decoding[:turn]
            self._decode_turn += budget
        for req in decoding:
            if req not in self.running_requests:
                continue
            while not self._fits(req, 1):
                victim = self.running_requests[-1]
                if victim is req and len(self.running_requests) == 1:
                    self.cache.close(req.request_id)      # alone and still no room: it can never go on
                    self.running_requests.remove(req)
                    req.finish("out_of_pages")
                    batch.failed.append(req)
                    break
                budget += self._preempt(victim, batch)
                if victim is req:
                    break
            if req in self.running_requests and budget > 0:
                self.cache.reserve(req.request_id, req.num_computed_tokens + 1)
                batch.entries.append((req, 1))
                decode_entries.add(req.request_id)
                budget -= 1

        # 2. running requests that still feed known tokens: portions under the budget and the free pages
        for req in list(self.running_requests):
            if not req.is_prefill() or budget <= 0:
                continue
            n = self._largest_fitting(req, min(self.chunk_size, req.pending_tokens(), budget))
            if n > 0:
                self.cache.reserve(req.request_id, req.num_computed_tokens + n)
                batch.entries.append((req, n))
                budget -= n

        # 3. admission, first come first served
        while (self.waiting_queue and budget > 0 and len(self.running_requests) < self.max_batch_size
               and len(self.running_requests) < self.max_sequences and self.cache.num_free_slots > 0):
            req = self.waiting_queue[0]
            want = min(self.chunk_size, req.pending_tokens(), budget)
            need = self.cache.pages_for_new_request(want)
            if any(n > f for n, f in zip(need, self.cache.free_pages())):
                if not self.running_requests and not batch.entries:
                    # nothing is running and the first portion still does not fit: shrink it, or give up
                    fit = min(self.cache.free_pages()) * self.cache.page_size if self.cache.free_pages() else want
                    if fit <= 0:
                        self.waiting_queue.popleft()
                        req.finish("out_of_pages")
                        batch.failed.append(req)
                        continue
                    want = min(want, fit)
                else:
                    break                           # hold admission back until pages come free
            self.waiting_queue.popleft()
            self.cache.open(req.request_id)
            self.cache.reserve(req.request_id, want)
            req.start_running()
            self.running_requests.append(req)
            batch.entries.append((req, want))
            budget -= want

        # a step must make progress: if requests run but nothing was planned, the newest one gives way (unless the
        # running requests only wait for sampled tokens to be read back)
        if not batch.entries and self.running_requests and not any(r.unresolved for r in self.running_requests):
            victim = self.running_requests[-1]
            if len(self.running_requests) == 1:
                self.cache.close(victim.request_id)
                self.running_requests.remove(victim)
                victim.finish("out_of_pages")
                batch.failed.append(victim)
            else:
                self._preempt(victim, batch)
                return self._merge(batch, self.schedule_next_batch())
        for req, n in batch.entries:          # counted from what is really in the step (preemptions took entries out)
            if req.request_id in decode_entries:
                self.stats_decode_tokens += n
            else:
                self.stats_prefill_tokens += n
        return batch

    @staticmethod
    def _merge(first: ScheduledBatch, second: ScheduledBatch) -> ScheduledBatch:
        second.preempted = first.preempted + second.preempted
        second.failed = first.failed + second.failed
        return second

    # ---- after the step ---------------------------------------------------------------------------------
    def update_after_step(self, batch: ScheduledBatch, finished_ids) -> None:
        """Account the step and drop finished requests from the running list (scheduler.hpp:75-89)."""
        self.stats_steps += 1
        for rid in finished_ids:
            req = self.request_map.get(rid)
            if req is None:
                continue
            if req in self.running_requests:
                if not req.is_finished():
                    req.finish()
                self.running_requests.remove(req)
            elif req in self.waiting_queue and req.is_finished():
                # preempted while a sampled id was still in flight, and that id ended it: nothing is left to recompute
                self.waiting_queue.remove(req)

    def abort(self, request_id: int, reason: str = "aborted") -> None:
        """Take a request out wherever it is; its pages and slot are given back."""
        req = self.request_map.get(request_id)
        if req is None or req.is_finished():
            return
        if req in self.running_requests:
            self.running_requests.remove(req)
            self.cache.close(req.request_id)
        elif req in self.waiting_queue:
            self.waiting_queue.remove(req)
        req.finish(reason)

    def get_stats(self) -> Stats:
        finished = sum(1 for r in self.request_map.values() if r.is_finished())
        return Stats(self.num_running(), self.num_waiting(), finished, len(self.request_map), self.stats_preemptions,
                     self.stats_steps, self.stats_prefill_tokens, self.stats_decode_tokens,
                     tuple(self.cache.free_pages()))
