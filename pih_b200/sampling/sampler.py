"""Sampling of one token per row of logits, on the device.

Definition from the reference (plugins/model-qwen3/qwen3_sampler.cpp:106-185,
its single-thread CUDA twin kernels/cuda/qwen_bf16_primitives.cu:894-999):
``scaled = logit / temperature`` (1 when greedy); suppressed ids are left
out; order by scaled descending with ties to the lower id; greedy takes the
first; otherwise keep the first ``top_k``, weights ``exp(scaled - scaled[0])``,
the shortest prefix whose share reaches ``top_p``, and pick by inverse CDF
with ``u = (word + 0.5) / 2^32`` where ``word`` is a Philox4x32-10 word keyed
by (seed, ordinal of the sampled token) (qwen3_sampler.cpp:85-104).  The
draw therefore depends on the request alone, not on what else is in the
batch or how often the request was recomputed.

The device kernel finds the same prefixes by radix selection over the whole
row instead of sorting it; its sums are formed in a different order than
the reference's sequential float sums, so a draw that lands within rounding
of a boundary may pick the neighbouring token.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from .params import SamplingParams

MAX_SUPPRESSED = 17          # include/pih/model/qwen3_sampler.h:18


class Sampler:
    def __init__(self, ops, vocab: int, device: torch.device):
        self.ops = ops
        self.vocab = vocab
        self.device = device

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], ordinals: Sequence[int],
               suppressed: Sequence[Sequence[int]]) -> List[int]:
        return self.sample_on_device(logits, params, ordinals, suppressed).tolist()

    def sample_on_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], ordinals: Sequence[int],
                         suppressed: Sequence[Sequence[int]]) -> torch.Tensor:
        """The sampled ids as an int32 tensor on the device, without waiting for them."""
        S = logits.shape[0]
        if not (len(params) == len(ordinals) == len(suppressed) == S):
            raise ValueError("one set of sampling parameters per row of logits is needed")
        if all(p.greedy for p in params) and not any(suppressed):
            return self.ops.argmax(logits)
        fl = torch.empty(S, 2, dtype=torch.float32)
        it = torch.empty(S, 6 + MAX_SUPPRESSED, dtype=torch.int32)
        for i, (p, o, sup) in enumerate(zip(params, ordinals, suppressed)):
            if len(sup) > MAX_SUPPRESSED or len(sup) >= self.vocab:
                raise ValueError("too many suppressed token ids")
            fl[i, 0] = p.temperature
            fl[i, 1] = p.top_p
            k = 0 if p.top_k is None or p.top_k >= self.vocab else p.top_k
            row = [k, p.seed & 0xFFFFFFFF, (p.seed >> 32) & 0xFFFFFFFF, o & 0xFFFFFFFF, (o >> 32) & 0xFFFFFFFF,
                   len(sup)] + list(sup) + [-1] * (MAX_SUPPRESSED - len(sup))
            it[i] = torch.tensor([v - (1 << 32) if v >= (1 << 31) else v for v in row], dtype=torch.int32)
        return self.ops.sample(logits, fl.to(self.device), it.to(self.device))
