"""The scheduler: which requests run in the next step, and with which tokens.

Host-only decisions over the cache manager's bookkeeping; it launches nothing.  In
mischief/lgml the same decisions are spread over the engine's coroutines
(``lua/lgml/engine.lua``): FIFO admission into at most ``slots`` slots when the pool
can hold the prompt and one more token (``:1248-1262``, ``:3050-3056``, ``room_for``
``:1144-1157``); prompts cut into portions of ``ubatch`` tokens (``:57``,
``prefill_batched`` ``:2213-2255``); all pending portions and decode tokens of a turn
joined into one pass (``flush`` ``:1423-1506``); finish on an end token, the token
limit or the repeat guard (``:3100-3209``, ``:2679-2689``); and, when the pool is full,
preemption: a request gives its cells back, waits, and is prefilled again from its
tokens so far so that "its reply is whole" (``preempt`` ``:1193-1243``); a request
that is alone and still does not fit ends with reason "length" (``:3183-3186``).

Policy here: decode tokens are planned first, then prompt portions in admission
order, under a token budget per step.  When a running request needs a page and none
is free, the most recently admitted running request is preempted: it gives back all
its pages and goes to the head of the waiting queue with prompt + generated tokens as
its new prompt (its sampler keeps its state, so the continuation is what it would
have been).  A request that is alone and cannot get a page ends with "length".
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Hashable, List, Optional, Sequence

from ..cache import CacheManager, NoSlot
from ..sampling import Sampler, SamplingParams

UBATCH = 512          # prompt tokens per request per step (lua/lgml/engine.lua:57)
UNKNOWN_TOKEN = -1    # stands for an id that is still on the device (a step planned ahead)
REPEAT_STOP = 256     # equal tokens in a row that end a reply (lua/lgml/engine.lua:61, :2679-2689)


@dataclass
class GenRequest:
    id: Hashable
    prompt: List[int]
    max_new_tokens: int
    params: SamplingParams = field(default_factory=SamplingParams)
    stop_ids: Sequence[int] = ()
    # state
    generated: List[int] = field(default_factory=list)
    n_cached: int = 0                 # tokens whose keys and values are in the cache
    cache_req: object = None
    sampler: Optional[Sampler] = None
    finish_reason: Optional[str] = None
    admitted_at: int = -1
    preemptions: int = 0
    repeat_run: int = 0

    tokens: List[int] = field(default_factory=list)   # prompt + generated, kept as one list

    def __post_init__(self):
        if self.sampler is None:
            self.sampler = Sampler(self.params)
        self.tokens = list(self.prompt) + list(self.generated)

    @property
    def n_pending(self) -> int:
        return len(self.tokens) - self.n_cached


@dataclass
class PlannedEntry:
    request: GenRequest
    tokens: List[int]
    sample: bool          # the portion ends the known tokens: the next token is sampled from its last logits


class Scheduler:
    def __init__(self, cache: CacheManager, max_position: int, ubatch: int = UBATCH, max_batch_tokens: int = 2048,
                 repeat_stop_tokens: int = REPEAT_STOP):
        if ubatch <= 0 or max_batch_tokens <= 0:
            raise ValueError("ubatch and max_batch_tokens must be positive")
        self.cache = cache
        self.max_position = max_position
        self.ubatch = ubatch
        self.max_batch_tokens = max_batch_tokens
        self.repeat_stop_tokens = repeat_stop_tokens
        self.waiting: Deque[GenRequest] = deque()
        self.running: List[GenRequest] = []
        self.finished: List[GenRequest] = []
        self._admissions = 0
        self._preempted_now: set = set()
        # counters, as the reference's batch_passes / batch_rows / batch_tokens (lua/lgml/engine.lua:1488-1492)
        self.stats = dict(steps=0, rows=0, tokens=0, preemptions=0, admitted=0, prefix_tokens=0)

    # ---- intake --------------------------------------------------------------------------
    def add(self, req: GenRequest) -> None:
        """Queue a request.  A prompt that cannot fit the context or the whole pool is
        refused at once (``lua/lgml/engine.lua:3008-3010``)."""
        if not req.prompt:
            raise ValueError(f"request {req.id!r}: empty prompt")
        if len(req.prompt) >= self.max_position:
            raise ValueError(f"request {req.id!r}: prompt of {len(req.prompt)} tokens does not fit the context of {self.max_position}")
        if self.cache.pages_for(len(req.prompt) + 1) > self.cache.n_pages:
            raise ValueError(f"request {req.id!r}: prompt of {len(req.prompt)} tokens does not fit the cache pool of "
                             f"{self.cache.n_pages * self.cache.page_size} tokens")
        self.waiting.append(req)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- planning ------------------------------------------------------------------------
    def _preempt(self, victim: GenRequest, plan: List[PlannedEntry]) -> int:
        """Take ``victim`` out of the running set (and out of ``plan``, if it is in it already).
        Returns the tokens that leave the plan with it: the caller gives them back to the step's budget."""
        # (with a prefix cache its full pages stay findable: when it is admitted again it takes
        #  up what the pool has not needed meanwhile, lua/lgml/engine.lua:1193-1243)
        self.cache.publish(victim.cache_req, victim.tokens)
        self.cache.close(victim.cache_req)
        victim.cache_req = None
        victim.n_cached = 0
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.running.remove(victim)
        dropped = sum(len(e.tokens) for e in plan if e.request is victim)
        plan[:] = [e for e in plan if e.request is not victim]
        self.waiting.appendleft(victim)
        self._preempted_now.add(id(victim))
        return dropped

    def _finish(self, req: GenRequest, reason: str) -> None:
        req.finish_reason = reason
        if req.cache_req is not None:
            self.cache.publish(req.cache_req, req.tokens)
            self.cache.close(req.cache_req)
            req.cache_req = None
        if req in self.running:
            self.running.remove(req)
        self.finished.append(req)

    def _reserve(self, req: GenRequest, n: int, plan: List[PlannedEntry]):
        """Pages for n more tokens of a running request.  While the pool is short the most
        recently admitted running request is preempted; if that is ``req`` itself it goes
        back to the queue (None), unless it is alone, in which case nothing can help (False).
        Returns (that outcome, the tokens that left the plan with preempted requests)."""
        refund = 0
        while not self.cache.reserve(req.cache_req, n):
            victim = max(self.running, key=lambda r: r.admitted_at)
            if victim is req:
                if len(self.running) == 1:
                    return False, refund
                return None, refund + self._preempt(req, plan)
            refund += self._preempt(victim, plan)
        return True, refund

    def plan(self) -> List[PlannedEntry]:
        """The entries of the next step (it reserves their pages).  Empty when idle."""
        plan: List[PlannedEntry] = []
        budget = self.max_batch_tokens
        self._preempted_now = set()     # requests this call preempts: they wait for a later turn
        # 1. running requests: single decode tokens first, then prompt portions, oldest first
        order = sorted(self.running, key=lambda r: (r.n_pending > 1, r.admitted_at))
        for req in order:
            if req not in self.running or budget <= 0:   # preempted while planning an earlier one
                continue
            n = min(req.n_pending, self.ubatch, budget)
            if n <= 0:
                continue
            got, refund = self._reserve(req, n, plan)
            budget += refund                 # a preempted request's planned tokens do not run
            if got is True and refund:
                more = min(req.n_pending, self.ubatch, budget)
                if more > n and self.cache.reserve(req.cache_req, more):
                    n = more
            if got is None:
                continue
            if got is False:
                # alone and out of pages: the reply ends here (lua/lgml/engine.lua:3183-3186)
                self._finish(req, "length")
                continue
            toks = req.tokens[req.n_cached:req.n_cached + n]
            plan.append(PlannedEntry(req, toks, sample=(n == req.n_pending)))
            budget -= n
        # 2. admission, FIFO: a slot, and room for the prompt and one more token
        while self.waiting and budget > 0 and len(self.cache.live) < self.cache.max_slots:
            req = self.waiting[0]
            if id(req) in self._preempted_now:
                # it gave its pages up in this very call so that an older request could go on: letting
                # it in again at once would only take them back (and prefill it from the start)
                break
            total = len(req.prompt) + len(req.generated)
            # (pages that the prefix cache already holds for its first tokens need not be free:
            #  cached ones count as free and are not taken twice, held ones are shared)
            shared = self.cache.cached_prefix_tokens(req.tokens) // self.cache.page_size
            if self.cache.pages_for(total + 1) - shared > self.cache.n_free_pages - self.cache.cached_pages_in_prefix(req.tokens):
                if not self.running and not plan:
                    # nothing will ever free a page: the request cannot run
                    self.waiting.popleft()
                    self._finish(req, "length")
                    continue
                break
            try:
                req.cache_req = self.cache.open(req.id, req.tokens)
            except NoSlot:
                break
            req.n_cached = req.cache_req.n_tokens        # what the prefix cache held of its tokens
            self.stats["prefix_tokens"] += req.n_cached
            self.waiting.popleft()
            req.admitted_at = self._admissions
            self._admissions += 1
            self.stats["admitted"] += 1
            self.running.append(req)
            n = min(req.n_pending, self.ubatch, budget)
            if not self.cache.reserve(req.cache_req, n):
                raise AssertionError("admission checked the pool, yet the first portion found no pages")
            plan.append(PlannedEntry(req, req.tokens[req.n_cached:req.n_cached + n], sample=(n == req.n_pending)))
            budget -= n
        if plan:
            self.stats["steps"] += 1
            self.stats["rows"] += len(plan)
            self.stats["tokens"] += sum(len(e.tokens) for e in plan)
        return plan

    def plan_ahead(self, inflight: List[PlannedEntry]) -> Optional[List[PlannedEntry]]:
        """The decode step after ``inflight``, planned before the tokens that ``inflight``
        samples are known: the same requests, one token each, the ids still on the device.
        None when the outcome of ``inflight`` could change the plan in any way but an end
        token: a request waits, a token limit or the repeat guard may strike, a portion of a
        prompt is under way, or a page is missing.  A request that ``inflight`` ends with an
        end token runs one token too many; ``complete`` drops it."""
        if self.waiting or not inflight or len(inflight) != len(self.running) or len(inflight) > self.max_batch_tokens:
            return None
        for e in inflight:
            r = e.request
            if not e.sample or r.finish_reason is not None or r.cache_req is None:
                return None
            after = len(r.generated) + 1
            if after >= r.max_new_tokens or len(r.prompt) + after >= self.max_position:
                return None
            if self.repeat_stop_tokens and r.repeat_run + 1 >= self.repeat_stop_tokens:
                return None
        for e in inflight:
            if not self.cache.reserve(e.request.cache_req, 1):
                return None
        plan = [PlannedEntry(e.request, [UNKNOWN_TOKEN], True) for e in inflight]
        self.stats["steps"] += 1
        self.stats["rows"] += len(plan)
        self.stats["tokens"] += len(plan)
        return plan

    # ---- after the step --------------------------------------------------------------------
    def complete(self, plan: List[PlannedEntry], sampled: Dict[Hashable, int]) -> List[GenRequest]:
        """Record that the planned tokens ran; ``sampled`` maps the id of each entry with
        ``sample`` set to its new token.  Returns the requests that finished."""
        done = []
        for e in plan:
            req = e.request
            if req.finish_reason is not None:
                continue                     # planned ahead of the end token that finished it
            req.n_cached += len(e.tokens)
            if not e.sample:
                continue
            tok = int(sampled[req.id])
            req.sampler.accept(tok)
            req.repeat_run = req.repeat_run + 1 if (req.generated and req.generated[-1] == tok) else 1
            req.generated.append(tok)
            req.tokens.append(tok)
            reason = None
            if tok in req.stop_ids:
                reason = "stop"
            elif len(req.generated) >= req.max_new_tokens:
                reason = "length"
            elif len(req.prompt) + len(req.generated) >= self.max_position:
                reason = "length"
            elif self.repeat_stop_tokens and req.repeat_run >= self.repeat_stop_tokens:
                reason = "length"
            if reason:
                self._finish(req, reason)
                done.append(req)
        return done
