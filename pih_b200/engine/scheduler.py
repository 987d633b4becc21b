"""Continuous-batching scheduler: admits, cuts prompts, decodes, finishes, frees.

The reference's controller (plugins/execution-default/controller_runtime.cpp:144-801,
policy in phase_tier_scheduler.cpp:52-185, per-request ledger in
controller_sequence.cpp:72-300) builds plans that are all-prefill or
all-decode, reserves a request's whole lifetime of pages at admission and
answers 429 when they are not there; it never preempts.  This scheduler
keeps the reference's ledger and finishing rules and changes the rest:

* a step mixes single decode tokens with prompt portions under one token
  budget (``max_batch_tokens``; the reference's ``maximum_batch_tokens``)
  and a bound on live requests (``max_batch_sequences``);
* pages are taken step by step, so the pool may be smaller than the sum of
  lifetimes.

Ledger (controller_sequence.cpp:167-173): with P prompt tokens, A accepted
tokens and K computed tokens, ``K = P + A - 1`` between steps once the
prompt is done; the token sampled last is fed at position K.  Here a
request's tokens are ``prompt + outputs``; a step computes the next ``n`` of
them, and logits are wanted exactly when the step reaches their end.

Finishing (controller_runtime.cpp:731-750): ``length`` when A reaches
``max_tokens``; ``stop`` when the sampled token is an end-of-sequence or
stop id and A >= ``minimum_new_tokens``; the stop token is part of the
output.

When pages run out
------------------
Order of service is order of arrival.  Running requests are served first,
oldest first.  If the pool cannot hold the next tokens of a running
request, the *youngest* running request is preempted: its pages go back,
its computed length returns to 0 and it moves to the head of the waiting
queue; all its tokens (prompt and outputs so far) are computed again when
it is next admitted, and because sampling is keyed by (seed, ordinal) the
tokens it goes on to produce are the same.  This repeats until the request
fits.  If a request is alone and still does not fit, it can never fit: it
finishes with reason ``"capacity"``.  A waiting request is admitted only
while a state slot is free, the budget has room, and the pool can hold the
first portion it would be given; admission stops at the first request that
does not fit (no overtaking).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Hashable, List, Optional, Sequence

from ..sampling.params import SamplingParams


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    eos_token_ids: Sequence[int] = ()
    outputs: List[int] = field(default_factory=list)
    output_logprobs: List[float] = field(default_factory=list)     # one per output, when the request asked for them
    output_top_logprobs: List[list] = field(default_factory=list)   # per output [(id, log-probability), ...], best first
    num_computed: int = 0
    status: str = "waiting"              # waiting | running | finished
    finish_reason: Optional[str] = None  # stop | length | capacity | cancelled | error
    arrival: int = 0
    preemptions: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.outputs

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.outputs)


@dataclass
class Scheduled:
    request: Request
    tokens: List[int]
    samples: bool                        # the step reaches the end of the request's tokens


@dataclass
class SchedulerOutput:
    scheduled: List[Scheduled]
    preempted: List[Request]
    failed: List[Request]

    @property
    def num_tokens(self) -> int:
        return sum(len(s.tokens) for s in self.scheduled)


class _Granted:
    """Pages granted so far in one scheduling decision, per cache group."""

    def __init__(self, cache):
        self.cache = cache
        self.taken = [0] * len(cache.groups)

    def fits(self, rid, n: int) -> bool:
        need = self.cache.pages_needed(rid, n)
        free = self.cache.num_free_pages()
        return all(self.taken[g] + need[g] <= free[g] for g in range(len(need)))

    def grant(self, rid, n: int) -> None:
        for g, c in enumerate(self.cache.pages_needed(rid, n)):
            self.taken[g] += c


class Scheduler:
    def __init__(self, cache, max_batch_sequences: int = 32, max_batch_tokens: int = 4096,
                 max_context: Optional[int] = None):
        if max_batch_sequences < 1 or max_batch_tokens < 1:
            raise ValueError("max_batch_sequences and max_batch_tokens must be >= 1")
        self.cache = cache
        self.max_batch_sequences = max_batch_sequences
        self.max_batch_tokens = max_batch_tokens
        self.max_context = max_context
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self._arrivals = 0

    # -- admission ----------------------------------------------------------
    def add(self, request: Request) -> None:
        if not request.prompt:
            raise ValueError("a request needs at least one prompt token")
        if self.max_context is not None and len(request.prompt) + request.params.max_tokens > self.max_context:
            raise ValueError(f"prompt ({len(request.prompt)}) + max_tokens ({request.params.max_tokens}) "
                             f"exceeds the context limit of {self.max_context}")
        request.arrival = self._arrivals
        self._arrivals += 1
        request.status = "waiting"
        self.waiting.append(request)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one scheduling decision ----------------------------------------------
    def _preempt(self, victim: Request, out: SchedulerOutput) -> None:
        self.running.remove(victim)
        self.cache.release(victim.rid)
        victim.num_computed = 0
        victim.status = "waiting"
        victim.preemptions += 1
        self.waiting.appendleft(victim)
        out.preempted.append(victim)

    def schedule(self) -> SchedulerOutput:
        out = SchedulerOutput([], [], [])
        budget = self.max_batch_tokens
        asks = _Granted(self.cache)                         # pages already granted this step, per group
        # running requests, oldest first
        for req in sorted(self.running, key=lambda r: r.arrival):
            if req.status != "running" or budget == 0:
                continue
            n = min(req.num_tokens - req.num_computed, budget)
            while not asks.fits(req.rid, n):
                victims = [r for r in self.running if r.status == "running" and r is not req
                           and all(s.request is not r for s in out.scheduled)]
                if not victims:
                    break
                self._preempt(max(victims, key=lambda r: r.arrival), out)
            if not asks.fits(req.rid, n):
                others = [s for s in out.scheduled]
                if others:
                    continue                                  # wait for a later step: others will finish
                # alone and it does not fit: it never will
                self.running.remove(req)
                self.cache.release(req.rid)
                req.status, req.finish_reason = "finished", "capacity"
                out.failed.append(req)
                continue
            asks.grant(req.rid, n)
            start = req.num_computed
            out.scheduled.append(Scheduled(req, self._next_tokens(req, start, n), start + n == req.num_tokens))
            budget -= n
        # admit waiting requests in order, no overtaking; not in a step that preempted
        while self.waiting and budget > 0 and len(self.running) < self.max_batch_sequences \
                and self.cache.slots.num_free > 0 and not out.preempted:
            req = self.waiting[0]
            n = min(req.num_tokens - req.num_computed, budget)
            self.cache.add_request(req.rid)
            if not asks.fits(req.rid, n):
                self.cache.release(req.rid)
                if not self.running and not out.scheduled:
                    # nothing else holds pages: even an empty pool is too small for this portion;
                    # try the largest portion that fits, else it can never run
                    n = self._largest_fit(req, n, asks)
                    if n == 0:
                        self.waiting.popleft()
                        req.status, req.finish_reason = "finished", "capacity"
                        out.failed.append(req)
                        continue
                    self.cache.add_request(req.rid)
                else:
                    break
            self.waiting.popleft()
            req.status = "running"
            self.running.append(req)
            asks.grant(req.rid, n)
            start = req.num_computed
            out.scheduled.append(Scheduled(req, self._next_tokens(req, start, n), start + n == req.num_tokens))
            budget -= n
        return out

    def plan_ahead(self, prev: SchedulerOutput) -> Optional[SchedulerOutput]:
        """The step after ``prev``, planned while ``prev`` is still running on the device and its sampled
        tokens are not known yet: every request of ``prev`` decodes one more token, which the device feeds
        from ``prev``'s samples (the entries carry a placeholder id, in ``prev``'s order).  Returns None
        whenever the plain path has a decision to make, and then nothing has changed: a request waits, a
        request of ``prev`` did not sample or ends with ``prev``'s token by length, a running request was
        left out of ``prev``, or the pool cannot hold one more token of each.  A request that ``prev``'s
        token turns out to stop is only found out afterwards: the token this step computes for it is then
        dropped by ``update``, and its pages are back in the pool before any later step can use them."""
        if self.waiting or prev.preempted or prev.failed or not prev.scheduled:
            return None
        if len(prev.scheduled) != len(self.running) or len(prev.scheduled) > self.max_batch_tokens:
            return None
        asks = _Granted(self.cache)
        scheduled = []
        for s in prev.scheduled:
            req = s.request
            if not s.samples or req.status != "running":
                return None
            if len(req.outputs) + 1 >= req.params.max_tokens:     # prev's token is its last
                return None
            if not asks.fits(req.rid, 1):
                return None
            asks.grant(req.rid, 1)
            scheduled.append(Scheduled(req, [0], True))
        return SchedulerOutput(scheduled, [], [])

    @staticmethod
    def _next_tokens(req: Request, start: int, n: int) -> List[int]:
        """Tokens start..start+n-1 of prompt + outputs, without building the whole list."""
        p = len(req.prompt)
        if start >= p:
            return req.outputs[start - p:start - p + n]
        if start + n <= p:
            return req.prompt[start:start + n]
        return req.prompt[start:] + req.outputs[:start + n - p]

    def _largest_fit(self, req: Request, n: int, asks) -> int:
        self.cache.add_request(req.rid)
        try:
            while n > 0 and not asks.fits(req.rid, n):
                n -= 1
            return n
        finally:
            self.cache.release(req.rid)

    # -- after the step ----------------------------------------------------------
    def update(self, out: SchedulerOutput, sampled: Sequence[Optional[int]],
               logprobs: Optional[Sequence[Optional[float]]] = None,
               top_logprobs: Optional[Sequence[Optional[list]]] = None) -> List[Request]:
        """``sampled[i]`` is the token sampled for ``out.scheduled[i]`` (None
        when that entry did not sample), ``logprobs[i]`` its log-probability where it was asked for,
        ``top_logprobs[i]`` the step's most probable ids with theirs (the request keeps as many as it asked for).
        Returns the requests that finished."""
        finished = []
        for i, (s, tok) in enumerate(zip(out.scheduled, sampled)):
            req = s.request
            if req.status == "finished":
                continue                   # it ended while this step was in flight (planned ahead): dropped
            req.num_computed += len(s.tokens)
            if not s.samples:
                continue
            if tok is None:
                raise ValueError(f"request {req.rid!r} reached its end but no token was sampled")
            req.outputs.append(int(tok))
            if req.params.logprobs and logprobs is not None and logprobs[i] is not None:
                req.output_logprobs.append(float(logprobs[i]))
            if req.params.top_logprobs and top_logprobs is not None and top_logprobs[i] is not None:
                req.output_top_logprobs.append(list(top_logprobs[i][:req.params.top_logprobs]))
            accepted = len(req.outputs)
            stops = set(req.params.stop_token_ids)
            if not req.params.ignore_eos:
                stops.update(req.eos_token_ids)
            if int(tok) in stops and accepted >= req.params.minimum_new_tokens:
                req.finish_reason = "stop"
            elif accepted >= req.params.max_tokens:
                req.finish_reason = "length"
            if req.finish_reason is not None:
                req.status = "finished"
                self.running.remove(req)
                self.cache.release(req.rid)
                finished.append(req)
        return finished

    def cancel(self, rid: Hashable, reason: str = "cancelled") -> Optional[Request]:
        """Cooperative cancel at a step boundary (controller_runtime.cpp: cancel -> draining).  ``reason``
        "error": a step that the request took part in failed."""
        for req in list(self.running):
            if req.rid == rid:
                self.running.remove(req)
                self.cache.release(rid)
                req.status, req.finish_reason = "finished", reason
                return req
        for req in list(self.waiting):
            if req.rid == rid:
                self.waiting.remove(req)
                req.status, req.finish_reason = "finished", reason
                return req
        return None

    def suppressed_ids(self, req: Request, pending: int = 0) -> List[int]:
        """Stop ids may not be sampled before ``minimum_new_tokens`` tokens exist
        (plugins/model-qwen3/controller_packed_driver.cpp:114-143).  ``pending``: tokens sampled on the
        device that are not in ``outputs`` yet."""
        if len(req.outputs) + pending >= req.params.minimum_new_tokens:
            return []
        ids = set(req.params.stop_token_ids)
        if not req.params.ignore_eos:
            ids.update(req.eos_token_ids)
        return sorted(ids)
