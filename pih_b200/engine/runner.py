"""The step function: run the tokens of one packed batch from the cache.

Counterpart of the reference's
``QwenBf16PackedSynchronousBackend::execute_packed``
(plugins/model-qwen3/qwen3_bf16_packed_synchronous_backend.cpp:79-182) with
the batch transaction around it
(qwen3_bf16_packed_batch_transaction.cpp:18-169): prepare the cache append
for every sequence, run the step, and advance the block tables only after
it.  Differences: a step may mix prompt portions and decode tokens; it
returns logits at the rows that were asked for (the reference returns
sampled ids and keeps logits on the device); rows are never padded to a
fixed bucket.
"""
from __future__ import annotations

from typing import Hashable, Optional, Sequence

import torch

from ..cache import CacheManager, OutOfPages
from .batch import BatchBuilder, StepBatch, StepEntry


class ModelRunner:
    def __init__(self, model, cache: CacheManager, cuda_graphs: bool = False):
        self.cuda_graphs = cuda_graphs
        self.model = model
        self.cache = cache
        self.device = model.rt.device
        self.builder = BatchBuilder(self.device)
        self.num_entries = len(model.spec.schedule)
        self.steps_run = 0

    def prepare(self, entries: Sequence[StepEntry]) -> StepBatch:
        """Allocate cache room for every entry (all or none) and pack the batch."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if len(e.tokens) < 1:
                raise ValueError(f"request {e.rid!r} brings no tokens")
            if not self.cache.has_request(e.rid):
                self.cache.add_request(e.rid)
        done = []
        try:
            for e in entries:
                self.cache.append(e.rid, len(e.tokens))
                done.append(e.rid)
        except OutOfPages:
            for rid in done:
                self.cache.rollback(rid)
            raise
        return self.builder.build(entries, self.cache)

    def run(self, batch: StepBatch) -> Optional[torch.Tensor]:
        caches = [self.cache.view(i, batch.block_tables, batch.slot_mappings)
                  for i in range(self.num_entries)]
        return self.model.forward(batch, caches)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run ``entries`` as one batch; returns fp32 logits ``[wanted, vocab]``
        in the order of the entries and of their ``want`` lists, or None."""
        batch = self.prepare(entries)
        try:
            logits = self.run(batch)
        except Exception:
            for e in entries:
                self.cache.rollback(e.rid)
            raise
        for e in entries:
            self.cache.commit(e.rid)
        self.steps_run += 1
        return logits

    def finish(self, rid: Hashable) -> None:
        """The request has ended: everything it holds goes back to the pools."""
        if self.cache.has_request(rid):
            self.cache.release(rid)
