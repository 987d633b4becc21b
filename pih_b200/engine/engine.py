"""The Python entry point: token ids in, token ids out, in-process.

The reference's Python package is an HTTP client for a running worker
(python/pih_client/client.py:145-288): ``Client(base_url).ready()``,
``.models()``, ``.complete(prompt, model=..., max_tokens=128, **params)`` and
``.stream_complete(...)``; it always sends ``temperature=0, top_p=1`` unless
overridden and insists on ``n == 1``.  This engine keeps those names,
defaults and meanings but works on token ids inside the process (servers and
tokenizers are out of its scope): ``Engine(model_dir).complete(token_ids,
max_tokens=128, temperature=0, top_p=1, seed=0)`` returns the reference's
token-generation result (src/worker/worker_bootstrap.cpp:584-591):
``{"schema": "pih.token-generation-result.v1", "token_ids": [...],
"finish_reason": "stop" | "length", "prompt_tokens": n, "completion_tokens": m}``.

Underneath: ``submit`` queues a request, ``step`` lets the scheduler build
one mixed batch, runs the step function, samples and books the tokens — the
loop that the reference's owner thread runs (plugins/model-qwen3/batch_generation.h:98-203).
"""
from __future__ import annotations

import itertools
import os
from collections import deque
from typing import Deque, Dict, Hashable, Iterator, List, Optional, Sequence

import torch

from ..kernels.ops import KernelError, error_text
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..cache import DEFAULT_PAGE_SIZE, OutOfPages
from .batch import StepEntry
from ..kernels import get_ops
from .factory import runner_for
from .scheduler import Request, Scheduler

RESULT_SCHEMA = "pih.token-generation-result.v1"


MAX_TOP_LOGPROBS = 20


class _Landing:
    """Pinned host memory for what one step reports back: the ids it sampled, their log-probabilities where a
    request asked for them, and, behind them, the device's error word as it stood after the step; with the
    event that says all have arrived."""

    def __init__(self, rows: int):
        self.rows = rows
        # ids [rows], log-probabilities [rows], top ids and top log-probabilities [rows, up to 20] each, the error word
        self.buffer = torch.empty((2 + 2 * MAX_TOP_LOGPROBS) * rows + 1, dtype=torch.int32, pin_memory=True)
        self.event = torch.cuda.Event()


class _InFlight:
    """A step that has been queued on the device: its plan, the ids it samples, and the error word after it —
    both copied to pinned host memory right behind the step, before any later step."""

    def __init__(self, out, tokens, error_word=None, landing: Optional[_Landing] = None, logprobs=None, top=None):
        self.out = out
        self.tokens = tokens
        self.logprobs = logprobs            # fp32 on the device, one per sampled id, or None
        self.top = top                      # (ids [rows, n], log-probabilities [rows, n]) on the device, or None
        self.landing = landing
        self.error_word = error_word
        self.rows = 0 if tokens is None else int(tokens.shape[0])
        self.holders = []                   # (request id, its cache record) of the step's requests
        # kernels that run on the host have finished by now: the word is read as it stands
        self._code = int(error_word) if landing is None and error_word is not None else None
        if landing is not None:
            if tokens is not None:
                landing.buffer[:self.rows].copy_(tokens, non_blocking=True)
            if logprobs is not None:
                landing.buffer[landing.rows:landing.rows + self.rows].copy_(logprobs.view(torch.int32), non_blocking=True)
            if top is not None:
                n = int(top[0].shape[1])
                base = 2 * landing.rows
                landing.buffer[base:base + self.rows * n].copy_(top[0].reshape(-1), non_blocking=True)
                base += MAX_TOP_LOGPROBS * landing.rows
                landing.buffer[base:base + self.rows * n].copy_(top[1].reshape(-1).view(torch.int32), non_blocking=True)
            landing.buffer[-1:].copy_(error_word, non_blocking=True)
            landing.event.record()

    def done(self) -> bool:
        return self.landing is None or self.landing.event.query()

    def wait(self) -> None:
        if self.landing is not None:
            self.landing.event.synchronize()

    def error_code(self) -> int:
        """The error word after this step (call after ``wait`` or a true ``done``)."""
        if self.landing is not None:
            return int(self.landing.buffer[-1])
        return self._code or 0

    def token_list(self) -> List[int]:
        """The sampled ids; waits for this step only, not for steps queued after it."""
        if self.tokens is None:
            return []
        if self.landing is None:
            return self.tokens.tolist()
        self.wait()
        return self.landing.buffer[:self.rows].tolist()

    def logprob_list(self) -> Optional[List[float]]:
        if self.logprobs is None:
            return None
        if self.landing is None:
            return self.logprobs.tolist()
        self.wait()
        return self.landing.buffer[self.landing.rows:self.landing.rows + self.rows].view(torch.float32).tolist()

    def top_list(self) -> Optional[List[List[tuple]]]:
        """Per sampled row its most probable ids with their log-probabilities, best first."""
        if self.top is None:
            return None
        n = int(self.top[0].shape[1])
        if self.landing is None:
            ids, lps = self.top[0].tolist(), self.top[1].tolist()
        else:
            self.wait()
            base = 2 * self.landing.rows
            ids = self.landing.buffer[base:base + self.rows * n].view(self.rows, n).tolist()
            base += MAX_TOP_LOGPROBS * self.landing.rows
            lps = self.landing.buffer[base:base + self.rows * n].view(torch.float32).view(self.rows, n).tolist()
        return [list(zip(i, l)) for i, l in zip(ids, lps)]


class Engine:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", *, device: str = "cuda:0",
                 page_size: int = DEFAULT_PAGE_SIZE, max_cache_tokens: Optional[int] = None, memory_fraction: float = 0.9,
                 maximum_batch_sequences: int = 32, maximum_batch_tokens: int = 4096,
                 maximum_context_tokens: Optional[int] = None, cuda_graphs: bool = True,
                 run_ahead: bool = True, ops: Optional[object] = None, model: Optional[tuple] = None,
                 capture_decode_after: int = 8):
        """``model_dir``: a folder with config.json and model.safetensors.  ``model``: instead of loading that
        folder, a ``(configuration, model)`` pair that is already built on its device (``model_dir`` is then
        only a name; ``dtype`` and ``device`` are the model's own).

        ``max_cache_tokens``: the size of every cache group's pool.  None (the default): what the device has
        left once the weights are on it, so that at most ``memory_fraction`` of its memory is in use — but no
        more than ``maximum_batch_sequences`` requests of ``maximum_context_tokens`` need (see
        ``factory.cache_tokens_for_memory``; the chosen size is ``engine.cache_tokens``).

        ``capture_decode_after``: with CUDA graphs, a decode step's shape is captured into a graph once it has been
        run this many times as it is (a capture costs about ten such steps; with requests that end one after the
        other a shape lasts a few steps only: measured on 32 requests of the 1.7B shape, 8 gave 6.1 thousand
        generated tokens a second against 5.6 with captures at first sight)."""
        from ..models import load_model
        from ..parts.registry import Runtime
        from .factory import DTYPES, cache_tokens_for_memory
        self.model_dir = model_dir
        if model is not None:
            self.config, self.model = model
        else:
            if dtype not in DTYPES:
                raise ValueError(f"dtype must be one of {sorted(DTYPES)}, got {dtype!r}")
            dev = torch.device(device)
            rt = Runtime(device=dev, dtype=DTYPES[dtype], ops=ops if ops is not None else get_ops(dev))
            self.config, self.model = load_model(model_dir, rt)
        self.device = self.model.rt.device
        max_positions = self.model.spec.max_positions
        self.max_context = min(maximum_context_tokens or max_positions, max_positions)
        if max_cache_tokens is None:
            if self.device.type == "cuda":
                max_cache_tokens = cache_tokens_for_memory(
                    self.model, page_size=page_size, max_requests=maximum_batch_sequences,
                    max_batch_tokens=maximum_batch_tokens, max_context=self.max_context,
                    memory_fraction=memory_fraction)
            else:
                max_cache_tokens = min(maximum_batch_sequences * self.max_context, 1 << 16)
        self.cache_tokens = max_cache_tokens
        self.cache, self.runner = runner_for(self.model, page_size=page_size, max_cache_tokens=max_cache_tokens,
                                             max_requests=maximum_batch_sequences, cuda_graphs=cuda_graphs,
                                             capture_decode_after=capture_decode_after)
        self.rt = self.model.rt
        spec = self.model.spec
        self.scheduler = Scheduler(self.cache, max_batch_sequences=maximum_batch_sequences,
                                   max_batch_tokens=maximum_batch_tokens, max_context=self.max_context)
        self.sampler = Sampler(self.rt.ops, spec.vocab, self.device)
        self._ids = itertools.count()
        self._live: Dict[Hashable, Request] = {}
        self.run_ahead = run_ahead       # plan and queue the next decode step before this one's ids are read
        self._inflight: Optional[_InFlight] = None
        self.steps_planned_ahead = 0
        self._unconfirmed: Deque[_InFlight] = deque()   # queued steps whose error word has not been seen, oldest first
        self._free_landings: List[_Landing] = []

    # -- the reference client's small calls ---------------------------------------
    def ready(self) -> bool:
        return True

    def models(self) -> dict:
        return {"object": "list", "data": [{"id": os.path.basename(os.path.normpath(self.model_dir)),
                                             "object": "model", "architecture": self.config.architecture}]}

    # -- requests -------------------------------------------------------------------
    def submit(self, prompt_token_ids: Sequence[int], params: Optional[SamplingParams] = None,
               rid: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt_token_ids]
        vocab = self.model.spec.vocab
        for t in prompt:
            if not 0 <= t < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        # as many ids as are asked for must be left beside the suppressed ones (plugins/model-qwen3/qwen3_sampler.cpp:46-49)
        stops = len(set(params.stop_token_ids) | set(self.model.spec.eos_token_ids))
        if params.top_logprobs > vocab - stops:
            raise ValueError(f"top_logprobs of {params.top_logprobs} is more than a vocabulary of {vocab} leaves "
                             f"beside {stops} ids that may be suppressed")
        rid = next(self._ids) if rid is None else rid
        if rid in self._live:
            raise ValueError(f"request {rid!r} is already live")
        req = Request(rid, prompt, params, eos_token_ids=tuple(self.model.spec.eos_token_ids))
        self.scheduler.add(req)
        self._live[rid] = req
        return rid

    def cancel(self, rid: Hashable) -> None:
        if self.scheduler.cancel(rid) is not None:
            self._live.pop(rid, None)

    def has_work(self) -> bool:
        return self._inflight is not None or self.scheduler.has_work()

    def drain(self) -> None:
        """Wait for every queued step and see its error word (raises ``KernelError`` as ``step`` does)."""
        if self._unconfirmed:
            self._settle(self._unconfirmed[-1])

    def warm_up(self, decode_batches: Optional[Sequence[int]] = None, rows: Optional[Sequence[int]] = None) -> dict:
        """Run — and, with CUDA graphs, capture — the step shapes that serving under this engine's limits
        meets most, before the first request: decode steps of every batch size that has a graph of its own,
        steps of the token budget's rows with every bucket of requests, with and without wanted rows, and a
        prompt alone in its step at every smaller bucket of rows (the first token of a short prompt on an idle
        engine: 13 to 16 ms at the first sight of its bucket, 2 to 4 ms from its graph).
        What a process pays once (library handles and kernels loaded at their first launch, work areas,
        captures) is then not paid between requests.  Stand-in requests hold a few pages for the duration of
        the call; nothing of them remains.  Only with an engine that holds no request.  ``decode_batches`` /
        ``rows``: other batch sizes / row counts than the default choice.  Returns what it did."""
        import time
        from .runner import _requests_bucket, _rows_bucket
        if self._live or self._inflight is not None:
            raise RuntimeError("warm_up needs an engine without requests")
        runner, cache, ops = self.runner, self.cache, self.rt.ops
        t0 = time.perf_counter()
        limit = self.scheduler.max_batch_sequences
        if decode_batches is None:
            decode_batches = [n for n in range(1, limit + 1) if runner._graph_key_of_decode(n)[1] == n]
        lone = []
        if rows is None:
            rows = [min(self.scheduler.max_batch_tokens, self.max_context - 1)]
            lone = sorted({_rows_bucket(n) for n in range(2, rows[0])} - {_rows_bucket(rows[0])})
        tag = ("warm-up", next(self._ids))
        standing: List[Hashable] = []
        done = {"decode_batches": [], "steps": [], "graphs_before": len(runner._graphs)}

        def decoders(n):
            while len(standing) < n:
                rid = (tag, "d", len(standing))
                runner.step([StepEntry(rid, [0], [])])
                standing.append(rid)
            return standing[:n]

        try:
            for n in sorted(set(int(b) for b in decode_batches if 1 <= int(b) <= limit)):
                ids = decoders(n)
                for _ in range(runner.capture_decode_after + 1):
                    runner.step([StepEntry(r, [0], [0]) for r in ids])
                done["decode_batches"].append(n)
            while len(standing) > limit - 1:                       # (a slot for the request that brings the portion)
                runner.finish(standing.pop())
            for t in sorted(set(int(r) for r in rows if int(r) >= 2)):
                buckets = sorted({_requests_bucket(n) for n in range(1, limit + 1)})
                for requests in buckets:
                    beside = min(requests, limit) - 1             # decode tokens beside one portion
                    if t - beside < 2:
                        continue
                    for wanted in (True, False):
                        ids = decoders(beside)
                        rid = (tag, "p", t, requests, wanted)
                        for _ in range(runner.CAPTURE_AFTER_STEP + 1):
                            entries = [StepEntry(r, [0], [0] if wanted else []) for r in ids]
                            entries.append(StepEntry(rid, [0] * (t - beside), [t - beside - 1] if wanted else []))
                            runner.step(entries)
                        runner.finish(rid)
                        done["steps"].append((_rows_bucket(t), requests, wanted))
            for t in lone:                                         # a prompt alone, whole, wanting its last row
                rid = (tag, "l", t)
                for turn in range(runner.CAPTURE_AFTER_STEP + 1):
                    runner.step([StepEntry((rid, turn), [0] * t, [t - 1])])
                    runner.finish((rid, turn))
                done["steps"].append((t, 1, True))
        except OutOfPages:
            done["stopped"] = "out of pages"
        finally:
            for rid in standing:
                runner.finish(rid)
            for rid in [r for r in cache.requests if isinstance(r, tuple) and r and r[0] == tag]:
                runner.finish(rid)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        ops.check_errors()
        done["graphs"] = len(runner._graphs)
        done["seconds"] = round(time.perf_counter() - t0, 3)
        return done

    # -- one step ---------------------------------------------------------------------
    # A step's sampled ids are needed on the host only to book them and to see who stops.  So while
    # step N runs, step N + 1 is planned (Scheduler.plan_ahead: every request decodes one more token),
    # its batch is built and it is queued behind N with its input ids fed on the device from N's
    # samples; only then does the host wait for N's ids.  The device never waits for the scheduler, the
    # batch builder or the copy of the ids.  A request that N's token stops has one token too many
    # computed in N + 1; it is dropped.  Whenever the plain path has a decision to make (admission, a
    # request at its length limit, pages that run out) nothing is planned ahead.
    #
    # What a step did counts only once it has been seen to succeed (the reference advances its block tables
    # only after the step completed without an error, qwen3_bf16_packed_batch_transaction.cpp:118-167).  The
    # kernels never trap: they record the first fault in one word on the device.  A copy of that word travels
    # to pinned host memory behind every step, with the sampled ids and under the same event, so seeing it
    # costs no wait of its own.  Until then the cache holds the step's tokens as queued, not confirmed.  A
    # non-zero word fails every request that took part in a step not yet confirmed: no token of such a step
    # is booked, the requests go back to their confirmed state, end with reason "error" and free what they
    # hold, the word is cleared, and ``step`` raises ``KernelError``; requests outside those steps go on.
    def _launch(self, out, feed=None) -> "_InFlight":
        pending = 1 if feed is not None else 0
        entries = [StepEntry(s.request.rid, s.tokens, [len(s.tokens) - 1] if s.samples else [])
                   for s in out.scheduled]
        logits = self.runner.step(entries, token_feed=feed, confirm=False)
        sampling = [s.request for s in out.scheduled if s.samples]
        tokens = logprobs = top = None
        if sampling:
            wanted = any(r.params.logprobs for r in sampling)
            top_n = max(r.params.top_logprobs for r in sampling)
            extra = {"logprobs": True} if wanted else {}
            if top_n:
                extra["top_logprobs"] = top_n
            tokens = self.sampler.sample_on_device(
                logits, [r.params for r in sampling], [len(r.outputs) + pending for r in sampling],
                [self.scheduler.suppressed_ids(r, pending) for r in sampling], **extra)
            if top_n:
                tokens, logprobs, top = tokens
            elif wanted:
                tokens, logprobs = tokens
        word = getattr(self.rt.ops, "error_word", None)
        on_gpu = self.device.type == "cuda" and word is not None
        flight = _InFlight(out, tokens, word, self._landing() if on_gpu else None, logprobs, top)
        flight.holders = [(s.request.rid, self.cache.requests[s.request.rid]) for s in out.scheduled]
        self._unconfirmed.append(flight)
        return flight

    def _landing(self) -> _Landing:
        if self._free_landings:
            return self._free_landings.pop()
        return _Landing(self.scheduler.max_batch_sequences)

    def _settle(self, upto: Optional["_InFlight"]) -> None:
        """See the error words of queued steps, oldest first: those up to ``upto`` (waiting for it), or, with
        None, those that the device has finished.  A step seen to succeed is confirmed in the cache."""
        while self._unconfirmed:
            flight = self._unconfirmed[0]
            if upto is None and not flight.done():
                return
            flight.wait()
            code = flight.error_code()
            if code:
                self._fail(code)
            self._unconfirmed.popleft()
            for rid, held in flight.holders:
                if self.cache.requests.get(rid) is held and held.unconfirmed:
                    self.cache.confirm(rid)
            if flight.landing is not None:
                self._free_landings.append(flight.landing)
            if flight is upto:
                return

    def _fail(self, code: int) -> None:
        flights = list(self._unconfirmed)
        self._unconfirmed.clear()
        self._inflight = None                       # a step planned ahead is among the flights: dropped with them
        affected: Dict[int, Request] = {}
        for flight in flights:
            for (rid, held), s in zip(flight.holders, flight.out.scheduled):
                if self.cache.requests.get(rid) is held:
                    self.cache.rollback(rid, unconfirmed=True)
                if s.request.status != "finished":
                    affected[id(s.request)] = s.request
            if flight.landing is not None:
                self._free_landings.append(flight.landing)
        for req in affected.values():
            self.scheduler.cancel(req.rid, reason="error")
            self._live.pop(req.rid, None)
        clear = getattr(self.rt.ops, "clear_errors", None)
        if clear is not None:
            clear()                                 # queued behind every step in flight
        raise KernelError(f"a kernel reported: {error_text(code)}; the requests of the steps not yet seen to "
                          f"succeed were ended with reason 'error': {[r.rid for r in affected.values()]}")

    def _collect(self, flight: "_InFlight") -> List[Request]:
        self._settle(flight if flight.tokens is not None else None)
        out = flight.out
        sampled: List[Optional[int]] = [None] * len(out.scheduled)
        logprobs: List[Optional[float]] = [None] * len(out.scheduled)
        tops: List[Optional[list]] = [None] * len(out.scheduled)
        if flight.tokens is not None:
            it = iter(flight.token_list())
            lp = flight.logprob_list()
            lp_it = iter(lp) if lp is not None else None
            top = flight.top_list()
            top_it = iter(top) if top is not None else None
            for i, s in enumerate(out.scheduled):
                if s.samples:
                    sampled[i] = next(it)
                    if lp_it is not None:
                        logprobs[i] = next(lp_it)
                    if top_it is not None:
                        tops[i] = next(top_it)
        live = [s.request for s in out.scheduled if s.samples and s.request.status != "finished"]
        self.scheduler.update(out, sampled, logprobs, tops)
        progressed = live + list(out.failed)
        for req in progressed:
            if req.status == "finished":
                self._live.pop(req.rid, None)
        return progressed

    def step(self) -> List[Request]:
        """One scheduler turn and one model step; returns the requests that
        produced a token in it (finished ones have ``status == 'finished'``).  Raises ``KernelError`` when a
        kernel of a queued step reported a fault (see above)."""
        flight = self._inflight
        self._inflight = None
        if flight is None:
            self._settle(None)
            out = self.scheduler.schedule()
            for req in out.failed:
                self._live.pop(req.rid, None)
            if not out.scheduled:
                if self._unconfirmed:
                    self._settle(self._unconfirmed[-1])
                return list(out.failed)
            flight = self._launch(out)
        ahead_failed = None
        if self.run_ahead and flight.tokens is not None:
            plan = self.scheduler.plan_ahead(flight.out)
            if plan is not None:
                try:
                    self._inflight = self._launch(plan, feed=flight.tokens)
                    self.steps_planned_ahead += 1
                except OutOfPages:
                    pass                            # nothing was queued or kept: the plain path decides next turn
                except Exception as error:          # the step that already ran is still collected, then this is raised
                    ahead_failed = error
        done = self._collect(flight)
        if ahead_failed is not None:
            raise ahead_failed
        return done

    # -- whole generations ------------------------------------------------------------
    @staticmethod
    def _result(req: Request) -> dict:
        result = {"schema": RESULT_SCHEMA, "token_ids": list(req.outputs), "finish_reason": req.finish_reason,
                  "prompt_tokens": len(req.prompt), "completion_tokens": len(req.outputs)}
        if req.params.logprobs:
            result["logprobs"] = list(req.output_logprobs)     # log-probability of each token under its scaled logits
            if req.params.top_logprobs:
                # per token the most probable ids, best first (plugins/surface-openai-http/entrypoint.cpp:367-382)
                result["top_logprobs"] = [[{"token_id": int(i), "logprob": float(l)} for i, l in step]
                                          for step in req.output_top_logprobs]
        return result

    @staticmethod
    def _params(max_tokens: int, parameters: dict) -> SamplingParams:
        if "n" in parameters and (type(parameters["n"]) is not int or parameters["n"] != 1):
            raise ValueError("native engine supports exactly n=1")
        merged = {"temperature": 0.0, "top_p": 1.0}
        merged.update(parameters)
        return SamplingParams(max_tokens=max_tokens, **merged)

    def complete(self, prompt_token_ids: Sequence[int], *, max_tokens: int = 128, **parameters) -> dict:
        return self.complete_batch([prompt_token_ids], max_tokens=max_tokens, **parameters)[0]

    def complete_batch(self, prompts: Sequence[Sequence[int]], *, max_tokens: int = 128,
                       parameters_per_prompt: Optional[Sequence[dict]] = None, **parameters) -> List[dict]:
        reqs = []
        for i, p in enumerate(prompts):
            extra = dict(parameters)
            if parameters_per_prompt is not None:
                extra.update(parameters_per_prompt[i])
            mt = extra.pop("max_tokens", max_tokens)
            rid = self.submit(p, self._params(mt, extra))
            reqs.append(self._live[rid])
        try:
            while any(r.status != "finished" for r in reqs):
                self.step()
        except Exception:
            for r in reqs:                           # nothing of this call stays behind in the engine
                if r.status != "finished":
                    self.cancel(r.rid)
            raise
        return [self._result(r) for r in reqs]

    def stream_complete(self, prompt_token_ids: Sequence[int], *, max_tokens: int = 128,
                        **parameters) -> Iterator[int]:
        """Yields token ids as they are produced; the request's result is in
        ``engine.last_result`` when the iterator ends."""
        rid = self.submit(prompt_token_ids, self._params(max_tokens, parameters))
        req = self._live[rid]
        sent = 0
        try:
            while req.status != "finished":
                self.step()
                while sent < len(req.outputs):
                    yield req.outputs[sent]
                    sent += 1
        finally:
            if req.status != "finished":
                self.cancel(rid)
        self.last_result = self._result(req)
