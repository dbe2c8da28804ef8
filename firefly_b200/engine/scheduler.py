"""The iteration-level scheduler: which requests run which tokens in the next step.

Called once per engine iteration, like the reference's ``Scheduler::step``
(src/scheduler.cc:82-163): requests that are already active go first, then
pending requests are admitted first-come-first-served while there is room.  The
names of the reference's limits are kept: ``max_batch_size_limit`` (64 active
requests, src/scheduler.cc:144) and ``max_prefill_chunk_size`` (256 prompt tokens
per request per step, src/engine.cc:240-241).  Differences, all deliberate:

* One step holds portions of prompts *and* decode tokens, under one token budget
  ``max_num_batched_tokens``; the reference runs them as separate calls.
* A request gets all the pages its portion needs before it is scheduled (the
  reference under-allocates later chunks, src/scheduler.cc:88-100,137-149).
* A finished request's pages go straight back to the free list.
* When pages run out the reference skips the starved requests every step and can
  stall forever (src/scheduler.cc:101-106).  Here the most recently admitted
  active request is preempted: its pages are freed, it keeps its tokens and goes
  back to the head of the pending queue, and on readmission recomputes prompt +
  generated tokens.  The oldest active request therefore always makes progress.
  A request that cannot fit in the pool even alone is finished with an error.

Every request is described by ``all tokens = prompt + generated`` and the number
of them already in the cache; a step feeds the next portion, and when the
portion reaches the end of the tokens the logits of its last place are sampled.
Decoding is the case where exactly one token is left.  A preempted request needs
no special path: it simply has zero tokens in the cache again.

Pure host logic: it needs the cache manager's bookkeeping but no device.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Sequence

from ..cache.manager import CacheManager
from .request import GenerationRequest, RequestStatus


@dataclass
class ScheduledItem:
    request: GenerationRequest
    start: int            # index of the first token fed (== tokens in the cache)
    num_tokens: int
    samples: bool         # the portion reaches the last token: its logits give the next token


@dataclass
class SchedulerBatch:
    items: List[ScheduledItem] = field(default_factory=list)
    preempted: List[GenerationRequest] = field(default_factory=list)
    failed: List[GenerationRequest] = field(default_factory=list)

    @property
    def requests(self) -> List[GenerationRequest]:
        return [it.request for it in self.items]

    @property
    def num_tokens(self) -> int:
        return sum(it.num_tokens for it in self.items)


class Scheduler:
    def __init__(self, cache: CacheManager, *, max_batch_size_limit: int = 64,
                 max_prefill_chunk_size: int = 256, max_num_batched_tokens: int = 8192,
                 max_model_len: int = 32768, eos_token_ids: Sequence[int] = (),
                 whole_prompts_when_idle: bool = False):
        """``whole_prompts_when_idle``: while no request is decoding, a portion may be as long as the
        step's token budget allows instead of ``max_prefill_chunk_size``.  Portions exist to bound what
        a prompt adds to the decode steps of the requests that are already running; with none running
        they only cost (eight steps of 256 tokens take 1.7 times as long as one of 2048 at the 8B
        shape).  The reference cuts prompts always (src/engine.cc:240-241)."""
        if max_prefill_chunk_size < 1 or max_num_batched_tokens < 1 or max_batch_size_limit < 1:
            raise ValueError("scheduler limits must be positive")
        self.cache = cache
        self.max_batch_size_limit = max_batch_size_limit
        self.max_prefill_chunk_size = max_prefill_chunk_size
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.eos_token_ids = frozenset(eos_token_ids)
        self.whole_prompts_when_idle = whole_prompts_when_idle
        self._chunk_now = max_prefill_chunk_size
        self.pending_requests: Deque[GenerationRequest] = deque()
        self.active_requests: List[GenerationRequest] = []
        self._arrivals = 0

    # ---- submission -------------------------------------------------------------
    def add_request(self, req: GenerationRequest) -> None:
        if not req.prompt_tokens:
            raise ValueError(f"request {req.id!r}: empty prompt")
        if len(req.prompt_tokens) + 1 > self.max_model_len:
            raise ValueError(f"request {req.id!r}: prompt of {len(req.prompt_tokens)} tokens leaves no "
                             f"room to generate within max_model_len {self.max_model_len}")
        req.status = RequestStatus.PENDING
        req.arrival = self._arrivals
        self._arrivals += 1
        self.pending_requests.append(req)

    def has_unfinished_requests(self) -> bool:
        return bool(self.pending_requests or self.active_requests)

    # ---- one iteration ------------------------------------------------------------
    def _portion(self, req: GenerationRequest, budget: int) -> int:
        left = req.get_total_len() - req.context_len
        return min(left, self._chunk_now, budget)

    def _preempt(self, req: GenerationRequest, batch: SchedulerBatch) -> None:
        self.cache.free(req.cache)
        req.cache = None
        req.status = RequestStatus.PENDING
        req.num_preemptions += 1
        self.active_requests.remove(req)
        self.pending_requests.appendleft(req)
        batch.preempted.append(req)

    def _fail(self, req: GenerationRequest, why: str, batch: SchedulerBatch) -> None:
        if req.cache is not None:
            self.cache.free(req.cache)
            req.cache = None
        if req in self.active_requests:
            self.active_requests.remove(req)
        req.status = RequestStatus.FINISHED
        req.finish_reason = f"error: {why}"
        batch.failed.append(req)

    def step(self) -> SchedulerBatch:
        batch = SchedulerBatch()
        budget = self.max_num_batched_tokens
        # the longest portion of this step: the configured size, or the whole budget while nobody decodes
        decoding = any(r.get_total_len() - r.context_len == 1 and r.generated_tokens for r in self.active_requests)
        self._chunk_now = self.max_prefill_chunk_size if (decoding or not self.whole_prompts_when_idle) \
            else max(self.max_prefill_chunk_size, budget)
        # 1. active requests, oldest first; each gets the pages of its next portion
        i = 0
        while i < len(self.active_requests):
            req = self.active_requests[i]
            n = self._portion(req, budget)
            if n <= 0:
                i += 1
                continue
            while not self.cache.grow(req.cache, req.context_len + n):
                victim = self.active_requests[-1]
                if victim is req:
                    break
                # the victim may already be in this batch: take it out again
                batch.items = [it for it in batch.items if it.request is not victim]
                self._preempt(victim, batch)
            else:
                batch.items.append(ScheduledItem(req, req.context_len, n,
                                                 req.context_len + n == req.get_total_len()))
                budget -= n
                i += 1
                continue
            # req is the youngest left and still does not fit
            if len(self.active_requests) == 1:
                self._fail(req, f"needs more cache pages than the pool holds "
                                f"({req.context_len + n} tokens)", batch)
            else:
                self._preempt(req, batch)
            # do not advance i: the list shrank
        # 2. admission, first come first served; never right after a preemption in this step
        while (self.pending_requests and not batch.preempted and budget > 0
               and len(self.active_requests) < self.max_batch_size_limit and self.cache.can_admit()):
            req = self.pending_requests[0]
            total = req.get_total_len()
            n = min(total, self._chunk_now, budget)
            why = self.cache.why_it_cannot_fit(total, self.max_prefill_chunk_size)
            if why is not None:
                self.pending_requests.popleft()
                self._fail(req, why, batch)
                continue
            rc = self.cache.admit(req.id)
            if not self.cache.grow(rc, n):
                self.cache.free(rc)
                break
            self.pending_requests.popleft()
            req.cache = rc
            req.status = RequestStatus.ACTIVE
            self.active_requests.append(req)
            batch.items.append(ScheduledItem(req, 0, n, n == total))
            budget -= n
        return batch

    # ---- after the step -------------------------------------------------------------
    def append_token(self, req: GenerationRequest, token: int) -> bool:
        """Record a sampled token; returns True when the request is finished."""
        req.generated_tokens.append(int(token))
        if not req.sampling.ignore_eos and int(token) in self.eos_token_ids:
            self.finish_request(req, "eos")
            return True
        if len(req.generated_tokens) >= req.max_tokens or req.get_total_len() >= self.max_model_len:
            self.finish_request(req, "length")
            return True
        return False

    def finish_request(self, req: GenerationRequest, reason: str = "length") -> None:
        req.status = RequestStatus.FINISHED
        req.finish_reason = reason
        if req.cache is not None:
            self.cache.free(req.cache)
            req.cache = None
        if req in self.active_requests:
            self.active_requests.remove(req)
        else:
            try:
                self.pending_requests.remove(req)
            except ValueError:
                pass
