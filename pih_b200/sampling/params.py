"""Sampling options of a request, with the reference's names, ranges and defaults.

plugins/model-qwen3/request_sampling.h:9-44: ``temperature`` 0..2 (0 means
greedy and then ``top_p`` must be 1), ``top_p`` in (0,1], ``seed`` >= 0 with
an omitted seed meaning 0 ("deliberately zero, not hidden host RNG state"),
``n`` must be 1.  ``top_k`` and ``minimum_new_tokens`` exist in the
reference's descriptor (include/pih/model/qwen3_sampler.h:23;
include/pih/scheduler/controller_request_arena.h:28-30) without an HTTP key;
here they are plain options.  ``max_tokens`` defaults to 128
(plugins/model-qwen3/entrypoint.cpp:252-254).  ``logprobs`` asks for what the
reference's sampler returns with every token, ``selected_logprob``
(plugins/model-qwen3/qwen3_sampler.cpp:143-149); ``top_logprobs`` = n (at most
20, qwen3_sampler.cpp:23, and only with ``logprobs``:
plugins/model-qwen3/controller_packed_driver.cpp:125-126) adds the n most
probable ids of every step with their log-probabilities
(qwen3_sampler.cpp:132-143).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple


@dataclass(frozen=True)
class SamplingParams:
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: Optional[int] = None
    seed: int = 0
    max_tokens: int = 128
    stop_token_ids: Tuple[int, ...] = ()
    minimum_new_tokens: int = 0
    ignore_eos: bool = False
    n: int = 1
    logprobs: bool = False             # return the log-probability of every sampled token (the reference's selected_logprob)
    top_logprobs: int = 0              # ... and the ids and log-probabilities of this many most probable tokens (at most 20)

    def __post_init__(self):
        if self.n != 1:
            raise ValueError("n must be 1")
        for name in ("temperature", "top_p"):
            v = getattr(self, name)
            if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
                raise ValueError("sampling parameter must be a finite number")
        if not (0.0 <= self.temperature <= 2.0) or not (0.0 < self.top_p <= 1.0):
            raise ValueError("temperature must be 0..2 and top_p must be (0,1]")
        if self.temperature == 0.0 and self.top_p != 1.0:
            raise ValueError("greedy temperature=0 requires top_p=1")
        if self.temperature == 0.0 and self.top_k is not None:
            raise ValueError("greedy temperature=0 takes no top_k")
        if self.top_k is not None and (isinstance(self.top_k, bool) or not isinstance(self.top_k, int)
                                       or self.top_k < 1):
            raise ValueError("top_k must be an integer >= 1")
        if isinstance(self.seed, bool) or not isinstance(self.seed, int) or not 0 <= self.seed < 2 ** 63:
            raise ValueError("seed must be an integer in 0..INT64_MAX")
        if isinstance(self.max_tokens, bool) or not isinstance(self.max_tokens, int) or self.max_tokens < 1:
            raise ValueError("max_tokens must be a positive integer")
        if isinstance(self.top_logprobs, bool) or not isinstance(self.top_logprobs, int) \
                or not 0 <= self.top_logprobs <= 20:
            raise ValueError("top_logprobs must be an integer in 0..20")
        if self.top_logprobs and not self.logprobs:
            raise ValueError("top_logprobs needs logprobs")
        if self.minimum_new_tokens < 0:
            raise ValueError("minimum_new_tokens must be >= 0")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0.0
