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


class _FixedPlans(dict):
    """Attention plans of a captured step: the same for every group size."""

    def __init__(self, plan):
        super().__init__()
        self._plan = plan

    def __contains__(self, key):
        return True

    def __getitem__(self, key):
        return self._plan


class _BoundedPlans(dict):
    """Attention plans of a captured step of several requests: computed per group size from the rows that
    each request brings (the step's key fixes them), with the longest context that the step's block tables
    can hold in place of the contexts themselves."""

    def __init__(self, counts, max_ctx: int):
        super().__init__()
        self._counts, self._max_ctx = list(counts), max_ctx

    def __contains__(self, key):
        return True

    def __getitem__(self, group):
        tile_max_q = dec_cap = 0
        for n in self._counts:
            if n * group <= 16:
                dec_cap = max(dec_cap, n)
            else:
                tile_max_q = max(tile_max_q, n)
        return tile_max_q, dec_cap, self._max_ctx if dec_cap else 0


class ModelRunner:
    def __init__(self, model, cache: CacheManager, cuda_graphs: bool = False, capture_decode_after: int = 0):
        self.cuda_graphs = cuda_graphs
        self.model = model
        self.cache = cache
        self.device = model.rt.device
        self.builder = BatchBuilder(self.device)
        self.num_entries = len(model.spec.schedule)
        self.steps_run = 0
        # A decode step is captured when its shape (requests, table width) has been run this many times uncaptured.
        # A capture costs about as much as ten uncaptured steps; a batch whose requests end one after the other
        # shows a shape for a few steps only.
        self.capture_decode_after = capture_decode_after
        self._graphs = {}
        self._sightings = {}               # shapes seen once and not captured yet; bounded like the graphs
        self._graph_pool = None
        self._confirm = True

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

    def step(self, entries: Sequence[StepEntry], token_feed: Optional[torch.Tensor] = None,
             confirm: bool = True) -> Optional[torch.Tensor]:
        """Run ``entries`` as one batch; returns fp32 logits ``[wanted, vocab]``
        in the order of the entries and of their ``want`` lists, or None.

        ``token_feed``: an int32 tensor on the device with one id per row of the step, which replaces the
        entries' token ids on the device — the ids that an earlier step sampled and that the host has not
        read yet.

        ``confirm``: the step's tokens count as soon as its kernels are queued (for a caller that reads the
        device's error word itself before it goes on, as the replay program does).  With False the cache
        only notes them as queued: the caller calls ``confirm(rids)`` once it has seen the step's error
        word as zero, or ``discard(rids)`` when it was not.

        The returned tensor may be reused by the next step: use it (or queue the kernel that does) before
        calling ``step`` again."""
        self._confirm = confirm
        return self._step(entries, token_feed)

    def confirm(self, rids) -> None:
        """The oldest queued step of each of these requests was seen to succeed."""
        for rid in rids:
            if self.cache.has_request(rid):
                self.cache.confirm(rid)

    def discard(self, rids) -> None:
        """A queued step of these requests failed: they return to their confirmed length, pages and state."""
        for rid in rids:
            if self.cache.has_request(rid):
                self.cache.rollback(rid, unconfirmed=True)

    def _commit(self, rid) -> None:
        self.cache.commit(rid, confirmed=self._confirm)

    def _step(self, entries: Sequence[StepEntry], token_feed: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        if self._graphable(entries):
            return self._graph_step(entries, token_feed)
        batch = self.prepare(entries)
        try:
            self._feed(batch, token_feed)
            logits = self.run(batch)
        except Exception:
            for e in entries:
                self.cache.rollback(e.rid)
            raise
        for e in entries:
            self._commit(e.rid)
        self.steps_run += 1
        return logits

    # -- steps replayed from CUDA graphs --------------------------------------------------
    # A step is ~7-10 launches per layer; for few rows the launches, not the kernels, bound it.  The
    # launch geometry of every kernel depends only on (rows, requests, wanted rows, block-table width,
    # the attention plan); which request owns which row is data in the step's device buffer.  So a step
    # can be captured once per such key and replayed with fresh data written into the same buffer:
    #   * decode steps (every request one token that wants its logits): captured at first sight;
    #   * any other step of at least GRAPH_MIN_ROWS rows — a prompt portion, or portions beside decode
    #     tokens — whose requests each want nothing or their last row: keyed by the rows that each
    #     request brings, in order, and captured when that key is seen the second time (chunked prefill
    #     under a token budget repeats its shapes: the same decode rows beside the same portion).  The
    #     GRAPH_LIMIT most recently used of these are kept.
    GRAPH_WIDTH_STEP = 64           # block-table widths are rounded up to a multiple of this many pages
    GRAPH_MIN_ROWS = 128
    GRAPH_LIMIT = 48
    CAPTURE_AFTER_STEP = 1          # a mixed step is captured when its shape is seen the second time

    def _graphable(self, entries) -> bool:
        return self._graph_key(entries) is not None

    def _graph_key(self, entries):
        if not (self.cuda_graphs and self.device.type == "cuda"):
            return None
        if all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return ("decode", len(entries))
        counts = tuple(len(e.tokens) for e in entries)
        if sum(counts) >= self.GRAPH_MIN_ROWS and all(list(e.want) in ([], [len(e.tokens) - 1]) for e in entries):
            return ("step", counts, tuple(len(e.want) for e in entries))
        return None

    @staticmethod
    def _feed(batch: StepBatch, token_feed: Optional[torch.Tensor]) -> None:
        if token_feed is not None:
            if (token_feed.dim() != 1 or token_feed.shape[0] != batch.token_ids.shape[0]
                    or token_feed.dtype != batch.token_ids.dtype):
                raise ValueError("token_feed needs one int32 id per row of the step")
            batch.token_ids.copy_(token_feed)                # queued behind the batch's own copy to the device

    def _graph_step(self, entries, token_feed=None) -> Optional[torch.Tensor]:
        kind = self._graph_key(entries)
        for e in entries:
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
        rids = [e.rid for e in entries]
        step_w = self.GRAPH_WIDTH_STEP
        width = -(-self.cache.table_width(rids) // step_w) * step_w
        key = kind + (width,)
        state = self._graphs.get(key)
        try:
            seen = self._sightings.get(key, 0)
            if state is None and seen < (self.CAPTURE_AFTER_STEP if kind[0] == "step" else self.capture_decode_after):
                # this shape has not been seen often enough to be worth a capture: run it as it is
                self._sightings[key] = seen + 1
                if len(self._sightings) > 4 * self.GRAPH_LIMIT:           # dicts keep insertion order: oldest out
                    del self._sightings[next(iter(self._sightings))]
                batch = self.builder.build(entries, self.cache)
                self._feed(batch, token_feed)
                logits = self.run(batch)
            elif state is None:
                self._sightings.pop(key, None)
                logits = self._capture(entries, key, width, token_feed)
            else:
                batch = self.builder.build(entries, self.cache, width=width, device_buffer=state["buffer"])
                self._feed(batch, token_feed)
                if key[0] == "step":
                    self._graphs[key] = self._graphs.pop(key)     # most recently used last
                state["graph"].replay()
                self._count_launches(state["launches"])
                logits = state["logits"]
        except Exception:
            for rid in rids:
                self.cache.rollback(rid)
            raise
        for rid in rids:
            self._commit(rid)
        self.steps_run += 1
        return logits

    def _count_launches(self, n: int) -> None:
        ops = self.model.rt.ops
        if hasattr(ops, "launches"):
            ops.launches += n

    def _capture(self, entries, key, width, token_feed=None):
        G = len(self.cache.groups)
        T = sum(len(e.tokens) for e in entries)
        B = len(entries)
        S = sum(len(e.want) for e in entries)
        buffer = torch.empty(self.builder.buffer_size(T, B, S, G, width), dtype=torch.int32, device=self.device)
        batch = self.builder.build(entries, self.cache, width=width, device_buffer=buffer)
        self._feed(batch, token_feed)
        max_ctx = width * self.cache.page_size
        ops = self.model.rt.ops
        # the attention plans of the graph cover every context that fits the table width
        if key[0] == "decode":
            batch.attention_plans = _FixedPlans((0, 1, max_ctx))
        else:
            batch.attention_plans = _BoundedPlans(key[1], max_ctx)
        caches = [self.cache.view(i, batch.block_tables, batch.slot_mappings) for i in range(self.num_entries)]
        # This step itself runs eagerly, on a side stream, from the buffer and with the plans that the graph
        # will have: whatever a kernel or a part sets up or allocates at its first call with these shapes (shared
        # memory limits, tensor maps, scratch sized by the plans, library handles) happens here and not under
        # capture.  The capture that follows records the same launches and executes nothing, so the step's
        # work — a mixer's update of its state slot included — is done exactly once.
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            eager_logits = self.model.forward(batch, caches)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        before = getattr(ops, "launches", 0)
        with torch.cuda.graph(graph, pool=self._graph_pool):
            logits = self.model.forward(batch, caches)
        launches = getattr(ops, "launches", 0) - before        # the pack's kernels inside the graph
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        state = {"graph": graph, "buffer": buffer, "logits": logits, "batch": batch, "launches": launches}
        self._graphs[key] = state
        steps = [k for k in self._graphs if k[0] == "step"]
        if len(steps) > self.GRAPH_LIMIT:                 # dicts keep insertion order; a replay re-inserts its key
            del self._graphs[steps[0]]
        return eager_logits

    def finish(self, rid: Hashable) -> None:
        """The request has ended: everything it holds goes back to the pools."""
        if self.cache.has_request(rid):
            self.cache.release(rid)
