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
from typing import Dict, Hashable, Iterator, List, Optional, Sequence

import torch

from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .batch import StepEntry
from .factory import create_runner, runner_for
from .scheduler import Request, Scheduler

RESULT_SCHEMA = "pih.token-generation-result.v1"


class _InFlight:
    """A step that has been queued on the device: its plan and the ids it samples, on the device and — by a
    copy queued right behind the sampler, before any later step — in pinned host memory."""

    def __init__(self, out, tokens, landing=None):
        self.out = out
        self.tokens = tokens
        self.host = self.copied = None
        if tokens is not None and tokens.device.type == "cuda":
            # `landing`: a pinned buffer and its event, owned by the engine and free again (two steps at most
            # are in flight, the engine rotates three)
            buffer, self.copied = landing
            self.host = buffer[:tokens.shape[0]]
            self.host.copy_(tokens, non_blocking=True)
            self.copied.record()

    def token_list(self) -> List[int]:
        """The sampled ids; waits for this step only, not for steps queued after it."""
        if self.host is None:
            return self.tokens.tolist()
        self.copied.synchronize()
        return self.host.tolist()


class Engine:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", *, device: str = "cuda:0",
                 page_size: int = 16, max_cache_tokens: Optional[int] = None,
                 maximum_batch_sequences: int = 32, maximum_batch_tokens: int = 4096,
                 maximum_context_tokens: Optional[int] = None, cuda_graphs: bool = True,
                 run_ahead: bool = True, ops: Optional[object] = None, model: Optional[tuple] = None,
                 decode_batch_multiple: int = 1):
        """``model_dir``: a folder with config.json and model.safetensors.  ``model``: instead of loading that
        folder, a ``(configuration, model)`` pair that is already built on its device (``model_dir`` is then
        only a name; ``dtype`` and ``device`` are the model's own).  ``decode_batch_multiple``: with CUDA graphs,
        decode steps are brought to a multiple of this many requests by stand-in requests, so that a few graphs
        serve every batch size (1, the default: never — the stand-ins are tested with the stand-in kernels on the
        CPU and have not yet run on a GPU)."""
        from ..config.registry import load_config
        self.model_dir = model_dir
        if model is not None:
            self.config, self.model = model
            self.device = self.model.rt.device
            max_positions = self.model.spec.max_positions
        else:
            self.device = torch.device(device)
            max_positions = load_config(model_dir).model_spec().max_positions
        self.max_context = min(maximum_context_tokens or max_positions, max_positions)
        if max_cache_tokens is None:
            max_cache_tokens = min(maximum_batch_sequences * self.max_context, 1 << 20)
        pad = decode_batch_multiple if cuda_graphs else 1
        if model is not None:
            self.cache, self.runner = runner_for(self.model, page_size=page_size, max_cache_tokens=max_cache_tokens,
                                                 max_requests=maximum_batch_sequences, cuda_graphs=cuda_graphs,
                                                 pad_decode_to=pad)
        else:
            self.config, self.model, self.cache, self.runner = create_runner(
                model_dir, dtype, device=device, page_size=page_size, max_cache_tokens=max_cache_tokens,
                max_requests=maximum_batch_sequences, cuda_graphs=cuda_graphs, ops=ops, pad_decode_to=pad)
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
        self._landings = None            # pinned buffers for the sampled ids, made at the first step on a GPU
        self._landing_turn = 0

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

    # -- one step ---------------------------------------------------------------------
    # A step's sampled ids are needed on the host only to book them and to see who stops.  So while
    # step N runs, step N + 1 is planned (Scheduler.plan_ahead: every request decodes one more token),
    # its batch is built and it is queued behind N with its input ids fed on the device from N's
    # samples; only then does the host wait for N's ids.  The device never waits for the scheduler, the
    # batch builder or the copy of the ids.  A request that N's token stops has one token too many
    # computed in N + 1; it is dropped.  Whenever the plain path has a decision to make (admission, a
    # request at its length limit, pages that run out) nothing is planned ahead.
    def _launch(self, out, feed=None) -> "_InFlight":
        pending = 1 if feed is not None else 0
        entries = [StepEntry(s.request.rid, s.tokens, [len(s.tokens) - 1] if s.samples else [])
                   for s in out.scheduled]
        logits = self.runner.step(entries, token_feed=feed)
        sampling = [s.request for s in out.scheduled if s.samples]
        tokens = None
        if sampling:
            tokens = self.sampler.sample_on_device(
                logits, [r.params for r in sampling], [len(r.outputs) + pending for r in sampling],
                [self.scheduler.suppressed_ids(r, pending) for r in sampling])
        return _InFlight(out, tokens, self._landing() if tokens is not None and tokens.device.type == "cuda" else None)

    def _landing(self):
        if self._landings is None:
            rows = self.scheduler.max_batch_sequences
            self._landings = [(torch.empty(rows, dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                              for _ in range(3)]
        self._landing_turn = (self._landing_turn + 1) % len(self._landings)
        return self._landings[self._landing_turn]

    def _collect(self, flight: "_InFlight") -> List[Request]:
        out = flight.out
        sampled: List[Optional[int]] = [None] * len(out.scheduled)
        if flight.tokens is not None:
            it = iter(flight.token_list())             # waits for this step
            for i, s in enumerate(out.scheduled):
                if s.samples:
                    sampled[i] = next(it)
        live = [s.request for s in out.scheduled if s.samples and s.request.status != "finished"]
        self.scheduler.update(out, sampled)
        progressed = live + list(out.failed)
        for req in progressed:
            if req.status == "finished":
                self._live.pop(req.rid, None)
        return progressed

    def step(self) -> List[Request]:
        """One scheduler turn and one model step; returns the requests that
        produced a token in it (finished ones have ``status == 'finished'``)."""
        flight = self._inflight
        self._inflight = None
        if flight is None:
            out = self.scheduler.schedule()
            for req in out.failed:
                self._live.pop(req.rid, None)
            if not out.scheduled:
                return list(out.failed)
            flight = self._launch(out)
        if self.run_ahead and flight.tokens is not None:
            plan = self.scheduler.plan_ahead(flight.out)
            if plan is not None:
                self._inflight = self._launch(plan, feed=flight.tokens)
                self.steps_planned_ahead += 1
        return self._collect(flight)

    # -- whole generations ------------------------------------------------------------
    @staticmethod
    def _result(req: Request) -> dict:
        return {"schema": RESULT_SCHEMA, "token_ids": list(req.outputs), "finish_reason": req.finish_reason,
                "prompt_tokens": len(req.prompt), "completion_tokens": len(req.outputs)}

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
        while any(r.status != "finished" for r in reqs):
            self.step()
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
