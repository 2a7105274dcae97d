"""The scheduler: which requests run in the next step, and with how many tokens.

The reference admits whole prompts first-come-first-served under a 2048-token
budget and a reservation of prompt + max_new tokens against 90 % of the pool,
and runs either a prefill step or a decode step, never both
(serve/run.py:265-293). Here every step is mixed: each decoding request gets
its one token first, what is left of the token budget goes to prompt portions
(of running requests first, then of newly admitted ones, in arrival order), so
a prompt may take several steps.

When pages run out. With ``reserve_full`` admission promises prompt + max_new
tokens to every request, as the reference does, and pages cannot run out.
Without it, a step that cannot get its pages evicts the request admitted last:
its pages and slot are given back, it returns to the head of the waiting queue
and is later recomputed from its prompt plus the tokens it had generated. A
request that could never fit the pool alone is refused when it is added.

This module decides; it runs nothing. ``plan`` returns the step's entries and
``update`` takes the sampled tokens. It needs the cache manager only for
counting pages and slots.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

from .step import FROM_DEVICE


@dataclass(eq=False)      # a request is itself, not its fields: `in` and `remove` on the queues compare identities
class SchedRequest:
    rid: int
    prompt: List[int]
    max_new_tokens: int
    temperature: float = 0.0
    stop_ids: Sequence[int] = ()
    generated: List[Optional[int]] = field(default_factory=list)   # None: sampled on the device, not yet read back
    fed: int = 0                 # tokens of prompt+generated already in the cache
    finished: bool = False
    finish_reason: Optional[str] = None
    preemptions: int = 0
    last_logits: object = None

    @property
    def sequence_length(self) -> int:
        return len(self.prompt) + len(self.generated)

    def pending(self) -> List[int]:
        """Tokens not yet in the cache; a token the host has not read back yet stands as FROM_DEVICE."""
        if self.fed >= len(self.prompt):
            rest = self.generated[self.fed - len(self.prompt):]
        else:
            rest = self.prompt[self.fed:] + self.generated
        return [FROM_DEVICE if t is None else t for t in rest]


@dataclass
class PlannedEntry:
    request: SchedRequest
    tokens: List[int]
    samples: bool                # the portion reaches the end of the sequence: a token is sampled from its last place


@dataclass
class SchedulerStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    max_running: int = 0


class Scheduler:
    def __init__(self, cache, max_tokens_per_step: int, prefill_chunk: Optional[int] = None, reserve_full: bool = False,
                 admission_fraction: float = 0.9, max_context: Optional[int] = None):
        self.cache = cache
        self.budget = max_tokens_per_step
        self.prefill_chunk = prefill_chunk or max_tokens_per_step
        self.reserve_full = reserve_full
        self.admission_fraction = admission_fraction
        self.max_context = max_context or cache.max_context
        self.waiting: Deque[SchedRequest] = deque()
        self.running: List[SchedRequest] = []     # in order of admission
        self.finished: List[SchedRequest] = []
        self.promised = [0] * len(cache.groups)   # reserve_full: pages of each cache group promised to running requests
        self.stats = SchedulerStats()
        self.evicted: List[SchedRequest] = []     # evicted by the last plan(); the caller gives back their cache

    # ---- sizes --------------------------------------------------------------
    # Every count of pages is the cache manager's: it knows its groups, their pools, which of them give pages
    # back behind a window, and what each request holds. The scheduler never turns tokens into pages itself.
    def _promise(self, req: SchedRequest) -> List[int]:
        """Per cache group: the most pages the request can hold at a time (the last generated token is never fed
        back, so the cache holds at most prompt + max_new - 1 tokens)."""
        return self.cache.peak_pages(len(req.prompt) + req.max_new_tokens - 1, min(self.prefill_chunk, self.budget))

    # ---- requests -----------------------------------------------------------
    def add(self, req: SchedRequest) -> None:
        if len(req.prompt) == 0:
            raise ValueError(f"request {req.rid}: empty prompt")
        if req.max_new_tokens < 1:
            raise ValueError(f"request {req.rid}: max_new_tokens must be at least 1")
        most = len(req.prompt) + req.max_new_tokens - 1
        if most > self.max_context:
            raise ValueError(f"request {req.rid}: prompt of {len(req.prompt)} + {req.max_new_tokens} new tokens exceeds the "
                             f"context limit of {self.max_context}")
        for gi, (need, pool) in enumerate(zip(self._promise(req), self.cache.pool_pages())):
            if need > pool:
                raise ValueError(f"request {req.rid}: needs {need} cache pages of group {gi}, the pool has {pool}")
        self.waiting.append(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---- planning -----------------------------------------------------------
    def plan(self) -> List[PlannedEntry]:
        """Entries of the next step. Evicts running requests if their pages cannot be had
        (they are listed in ``self.evicted`` for the caller to close in the cache)."""
        self.evicted = []
        while True:
            entries, at_most = self._plan_running()
            batch = [(e.request.rid, e.request.fed + len(e.tokens)) for e in entries]
            if self.cache.fits(batch, freed=[v.rid for v in self.evicted], at_most=at_most if not self.evicted else None):
                break
            # pages ran out: the request admitted last goes back to the head of the queue
            victim = self.running.pop()
            self._evict(victim)
        used = sum(len(e.tokens) for e in entries)
        entries.extend(self._admit(self.budget - used, batch))
        self.stats.max_running = max(self.stats.max_running, len(self.running))
        return entries

    def _evict(self, victim: SchedRequest) -> None:
        victim.fed = 0
        victim.preemptions += 1
        self.stats.preemptions += 1
        if self.reserve_full:
            self.promised = [a - b for a, b in zip(self.promised, self._promise(victim))]
        self.evicted.append(victim)
        self.waiting.appendleft(victim)

    def _plan_running(self):
        """(entries of the running requests, an upper bound of the pages they want of any cache group)."""
        entries: List[PlannedEntry] = []
        left = self.budget
        ps = self.cache.page_size
        at_most = 0
        portions = []
        # decoding requests first: one token each (this loop runs for every live request in every step)
        for r in self.running:
            gen = r.generated
            n = len(r.prompt) + len(gen) - r.fed
            if n == 1:
                if left > 0:
                    tok = gen[-1] if gen else r.prompt[-1]
                    entries.append(PlannedEntry(r, [FROM_DEVICE if tok is None else tok], True))
                    left -= 1
                    at_most += 1                    # growing by n tokens takes at most ceil(n / page_size) pages
            elif n > 1:
                portions.append((r, n))
        # then portions of prompts already under way
        for r, n in portions:
            if left > 0:
                take = min(n, self.prefill_chunk, left)
                entries.append(PlannedEntry(r, r.pending()[:take], take == n))
                left -= take
                at_most += -(-take // ps)
        return entries, at_most

    def _admit(self, left: int, batch: List) -> List[PlannedEntry]:
        """Waiting requests, in arrival order, while the token budget, the slots and the pages last. ``batch``: what the
        running requests already take in this step, as (request, length after the step) pairs."""
        entries: List[PlannedEntry] = []
        free_slots = self.cache.free_slots + len(self.evicted)
        pools = self.cache.pool_pages()
        free = None           # per group: pages left once the running requests have theirs (asked for at the first candidate)
        while self.waiting and left > 0 and free_slots > 0:
            r = self.waiting[0]
            if r in self.evicted:
                break   # evicted in this very step; it waits for the next
            n = r.sequence_length - r.fed
            take = min(n, self.prefill_chunk, left)
            if self.reserve_full:
                promise = self._promise(r)
                if self.running and any(have + p > self.admission_fraction * pool
                                        for have, p, pool in zip(self.promised, promise, pools)):
                    break
            if free is None:
                free = self.cache.free_after(batch, freed=[v.rid for v in self.evicted])
            want = self.cache.pages_wanted(r.rid, r.fed + take)
            if any(w > f for w, f in zip(want, free)):
                break
            free = [f - w for f, w in zip(free, want)]
            if self.reserve_full:
                self.promised = [a + b for a, b in zip(self.promised, promise)]
            self.waiting.popleft()
            self.running.append(r)
            entries.append(PlannedEntry(r, r.pending()[:take], take == n))
            left -= take
            free_slots -= 1
        return entries

    # ---- after the step -----------------------------------------------------
    def update(self, entries: Sequence[PlannedEntry], sampled: Sequence[int]) -> List[SchedRequest]:
        """Account a launched step. ``sampled``: one token for each entry with ``samples`` set, in order; None for a
        token that is still on the device (``resolve`` fills it in later; stopping by a stop id is then found
        there). Returns the requests that finished (the caller gives back their cache)."""
        self.stats.steps += 1
        done: List[SchedRequest] = []
        it = iter(sampled)
        for e in entries:
            r = e.request
            if r.fed + len(e.tokens) > len(r.prompt) and len(e.tokens) == 1:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += len(e.tokens)
            r.fed += len(e.tokens)
            if not e.samples:
                continue
            tok = next(it)
            tok = int(tok) if tok is not None else None
            r.generated.append(tok)
            if len(r.generated) >= r.max_new_tokens:
                r.finished, r.finish_reason = True, "length"
            elif tok is not None and tok in r.stop_ids:
                r.finished, r.finish_reason = True, "stop"
            if r.finished:
                done.append(r)
        for r in done:
            self.running.remove(r)
            self.finished.append(r)
            if self.reserve_full:
                self.promised = [a - b for a, b in zip(self.promised, self._promise(r))]
        return done

    def resolve(self, request: SchedRequest, index: int, token: int) -> bool:
        """The token generated at ``index`` has reached the host. Returns True if it ends the request (a stop id):
        the request leaves the queues, what was generated past it (a step launched meanwhile) is dropped, and the
        caller gives back its cache."""
        if index >= len(request.generated):
            return False                      # the request was cut short by an earlier stop id
        request.generated[index] = int(token)
        if int(token) in request.stop_ids and (not request.finished or index < len(request.generated) - 1):
            del request.generated[index + 1:]
            newly = not request.finished
            request.finished, request.finish_reason = True, "stop"
            if request in self.running:
                self.running.remove(request)
                if self.reserve_full:
                    self.promised = [a - b for a, b in zip(self.promised, self._promise(request))]
            if request in self.waiting:
                self.waiting.remove(request)
            if newly:
                self.finished.append(request)
            return True
        return False
