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
row instead of sorting it, and adds the masses exactly (fixed point) where
the reference adds them one after the other in float32.  Over a few
thousand terms the two agree to the last places, and a draw picks another
token only when it lands within rounding of a boundary.  Over a vocabulary
of 150 000 the sequential float32 sum drops every term below half an ulp of
the running total, a few thousandths of the mass in all, so there the
reference's own boundaries sit that far from the exact ones and a draw may
fall on a token some places further along the sorted order.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch

from .params import SamplingParams

MAX_SUPPRESSED = 17          # include/pih/model/qwen3_sampler.h:18
_INT_COLUMNS = 6 + MAX_SUPPRESSED


class Sampler:
    """Per-row parameters reach the device in one copy from pinned memory that does not wait (a copy from
    pageable memory would stall the host until the device has caught up, in every step)."""

    STAGES = 4                # pinned buffers in rotation: a buffer is reused only after its copy has left it

    def __init__(self, ops, vocab: int, device: torch.device):
        self.ops = ops
        self.vocab = vocab
        self.device = device
        self._stages = []
        self._turn = 0

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], ordinals: Sequence[int],
               suppressed: Sequence[Sequence[int]]) -> List[int]:
        return self.sample_on_device(logits, params, ordinals, suppressed).tolist()

    def _stage(self, rows: int):
        """(host int32 buffer, event or None) with room for ``rows`` rows of parameters."""
        need = rows * (2 + _INT_COLUMNS)
        pin = self.device.type == "cuda"
        if len(self._stages) < self.STAGES:
            self._stages.append([torch.empty(max(need, 64 * (2 + _INT_COLUMNS)), dtype=torch.int32, pin_memory=pin),
                                 torch.cuda.Event() if pin else None, False])
        self._turn = (self._turn + 1) % len(self._stages)
        stage = self._stages[self._turn]
        if stage[2]:
            stage[1].synchronize()
            stage[2] = False
        if stage[0].numel() < need:
            stage[0] = torch.empty(2 * need, dtype=torch.int32, pin_memory=pin)
        return stage

    def sample_on_device(self, logits: torch.Tensor, params: Sequence[SamplingParams], ordinals: Sequence[int],
                         suppressed: Sequence[Sequence[int]], logprobs: bool = False, top_logprobs: int = 0):
        """The sampled ids as an int32 tensor on the device, without waiting for them; with ``logprobs`` a pair
        of the ids and the log-probability of each (fp32, on the device); with ``top_logprobs`` = n > 0 a triple
        whose third member is ``(ids [rows, n], log-probabilities [rows, n])`` of every row's n most probable ids."""
        S = logits.shape[0]
        if not (len(params) == len(ordinals) == len(suppressed) == S):
            raise ValueError("one set of sampling parameters per row of logits is needed")
        if all(p.greedy for p in params) and not any(suppressed):
            ids = self.ops.argmax(logits)
            if top_logprobs > 0:
                return ids, self.ops.selected_logprob(logits, ids), self.ops.top_logprobs(logits, top_logprobs)
            return (ids, self.ops.selected_logprob(logits, ids)) if logprobs else ids
        stage = self._stage(S)
        host = stage[0][:S * (2 + _INT_COLUMNS)]
        view = host.numpy()
        fl = view[:2 * S].view(np.float32).reshape(S, 2)
        it = view[2 * S:].view(np.uint32).reshape(S, _INT_COLUMNS)
        # whole columns at a time (a row at a time cost the host 8 us a row, every step)
        fl[:, 0] = [p.temperature for p in params]
        fl[:, 1] = [p.top_p for p in params]
        it[:, 0] = [0 if p.top_k is None or p.top_k >= self.vocab else p.top_k for p in params]
        it[:, 1] = [p.seed & 0xFFFFFFFF for p in params]
        it[:, 2] = [(p.seed >> 32) & 0xFFFFFFFF for p in params]
        it[:, 3] = [o & 0xFFFFFFFF for o in ordinals]
        it[:, 4] = [(o >> 32) & 0xFFFFFFFF for o in ordinals]
        it[:, 5] = [len(sup) for sup in suppressed]
        it[:, 6:] = 0xFFFFFFFF
        for i, sup in enumerate(suppressed):
            if sup:
                if len(sup) > MAX_SUPPRESSED or len(sup) >= self.vocab:
                    raise ValueError("too many suppressed token ids")
                it[i, 6:6 + len(sup)] = list(sup)
        dev = torch.empty(host.numel(), dtype=torch.int32, device=self.device)
        dev.copy_(host, non_blocking=True)
        if stage[1] is not None:
            stage[1].record()
            stage[2] = True
        fparams, iparams = dev[:2 * S].view(torch.float32).view(S, 2), dev[2 * S:].view(S, _INT_COLUMNS)
        ids = self.ops.sample(logits, fparams, iparams)
        if top_logprobs > 0:
            return (ids, self.ops.selected_logprob(logits, ids, fparams, iparams),
                    self.ops.top_logprobs(logits, top_logprobs, fparams, iparams))
        return (ids, self.ops.selected_logprob(logits, ids, fparams, iparams)) if logprobs else ids
