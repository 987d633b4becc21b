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


class _PaddedPlans(dict):
    """Attention plans of a step padded to ``rows`` rows: whatever its requests bring.  Any request may be a
    portion of up to all the rows, or decode-like with as many rows as 16 packed rows hold — unless the step's
    key says that it has no request of one of the two kinds (then that kind's kernel is not launched)."""

    def __init__(self, rows: int, max_ctx: int, small: bool = True, large: bool = True):
        super().__init__()
        self._rows, self._max_ctx, self._small, self._large = rows, max_ctx, small, large

    def __contains__(self, key):
        return True

    def __getitem__(self, group):
        tile_max_q = self._rows if (self._large and self._rows * group > 16) else 0
        dec_cap = max(1, min(self._rows, 16 // group)) if (self._small or tile_max_q == 0) else 0
        return tile_max_q, dec_cap, self._max_ctx if dec_cap else 0


def _rows_bucket(n: int) -> int:
    """Rows of a padded step: 16, 32, 64, then steps of a quarter to a half of the count."""
    for b in (16, 32, 64, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 3072, 4096):
        if n <= b:
            return b
    return -(-n // 2048) * 2048


def _requests_bucket(n: int) -> int:
    return 1 << max(0, n - 1).bit_length()


class ModelRunner:
    def __init__(self, model, cache: CacheManager, cuda_graphs: bool = False, capture_decode_after: int = 0,
                 pad_steps: bool = True):
        self.cuda_graphs = cuda_graphs
        # Steps of different make-up are padded to common shapes (see engine/batch.py), so that a serving run meets
        # a handful of shapes and replays them from graphs, if every part of the model leaves padding alone.
        self.pad_steps = pad_steps and cuda_graphs and bool(getattr(model, "pad_safe", False))
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
    #   * decode steps (every request one token that wants its logits): keyed by the number of requests — beyond
    #     PAD_DECODE_ABOVE of them, padded to a multiple of 8 — and captured when the key has been seen
    #     ``capture_decode_after`` times;
    #   * any other step — a prompt portion, or portions beside decode tokens — whose requests each want
    #     nothing or their last row: padded to (rows bucket, requests bucket, wanted rows: none or one a request)
    #     and captured when that shape is seen the second time.  What the kernels need to know about the step's
    #     make-up is in its device buffer; the attention plans cover every make-up.  Without padding (a model
    #     with a part that does not allow it): keyed by the rows that each request brings, in order, from
    #     GRAPH_MIN_ROWS rows on.  The GRAPH_LIMIT most recently used of these are kept.
    GRAPH_WIDTH_STEP = 64           # block-table widths are rounded up to a multiple of this many pages
    GRAPH_MIN_ROWS = 128
    GRAPH_LIMIT = 48
    CAPTURE_AFTER_STEP = 1          # a mixed step is captured when its shape is seen the second time
    PAD_DECODE_ABOVE = 16           # up to here every batch size of a decode step has a graph of its own

    def _graphable(self, entries) -> bool:
        return self._graph_key(entries) is not None

    def _graph_key(self, entries):
        if not (self.cuda_graphs and self.device.type == "cuda"):
            return None
        n = len(entries)
        if all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._graph_key_of_decode(n)
        counts = tuple(len(e.tokens) for e in entries)
        if not all(list(e.want) in ([], [len(e.tokens) - 1]) for e in entries):
            return None
        if self.pad_steps:
            requests = _requests_bucket(n)
            # whether a request may be decode-like (at most 16 packed rows) / a portion, for any group size of a mixer
            small, large = any(c <= 16 for c in counts), any(c >= 2 for c in counts)
            return ("padded", _rows_bucket(sum(counts)), requests, requests if any(e.want for e in entries) else 0,
                    small, large)
        if sum(counts) >= self.GRAPH_MIN_ROWS:
            return ("step", counts, tuple(len(e.want) for e in entries))
        return None

    def _graph_key_of_decode(self, n: int):
        if self.pad_steps and n > self.PAD_DECODE_ABOVE:
            return ("decode", -(-n // 8) * 8)
        return ("decode", n)

    @staticmethod
    def _padding(kind, entries):
        """(rows, requests, wanted rows) that a step of this key is padded to; None: as it is."""
        if kind[0] == "padded":
            return kind[1], kind[2], kind[3]
        if kind[0] == "decode" and kind[1] != len(entries):
            return kind[1], kind[1], kind[1]
        return None

    def _plans(self, kind, max_ctx: int):
        if kind[0] == "decode":
            return _FixedPlans((0, 1, max_ctx))
        if kind[0] == "padded":
            return _PaddedPlans(kind[1], max_ctx, kind[4], kind[5])
        return _BoundedPlans(kind[1], max_ctx)

    @staticmethod
    def _feed(batch: StepBatch, token_feed: Optional[torch.Tensor]) -> None:
        if token_feed is not None:
            rows = batch.real_rows
            if token_feed.dim() != 1 or token_feed.shape[0] != rows or token_feed.dtype != batch.token_ids.dtype:
                raise ValueError("token_feed needs one int32 id per row of the step")
            batch.token_ids[:rows].copy_(token_feed)         # queued behind the batch's own copy to the device

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
        pad = self._padding(kind, entries)
        wanted = sum(len(e.want) for e in entries)
        try:
            seen = self._sightings.get(key, 0)
            if state is None and seen < (self.capture_decode_after if kind[0] == "decode" else self.CAPTURE_AFTER_STEP):
                # this shape has not been seen often enough to be worth a capture: run it uncaptured (padded as
                # its graph will be and with the graph's plans: the same kernels on the same shapes give the
                # same logits whether replayed or not)
                self._sightings[key] = seen + 1
                if len(self._sightings) > 4 * self.GRAPH_LIMIT:           # dicts keep insertion order: oldest out
                    del self._sightings[next(iter(self._sightings))]
                if pad is None:
                    batch = self.builder.build(entries, self.cache)
                else:
                    batch = self.builder.build(entries, self.cache, width=width, pad=pad)
                    batch.attention_plans = self._plans(kind, width * self.cache.page_size)
                batch.padded = True                               # (a shape that comes again, padded or not)
                self._feed(batch, token_feed)
                logits = self.run(batch)
            elif state is None:
                self._sightings.pop(key, None)
                logits = self._capture(entries, key, width, token_feed)
            else:
                batch = self.builder.build(entries, self.cache, width=width, device_buffer=state["buffer"], pad=pad)
                self._feed(batch, token_feed)
                if key[0] != "decode":
                    self._graphs[key] = self._graphs.pop(key)     # most recently used last
                state["graph"].replay()
                self._count_launches(state["launches"])
                logits = state["logits"]
            if pad is not None and logits is not None:
                logits = logits[:wanted] if wanted else None
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
        pad = self._padding(key, entries)
        if pad is None:
            T, B, S = sum(len(e.tokens) for e in entries), len(entries), sum(len(e.want) for e in entries)
        else:
            T, B, S = pad
        buffer = torch.empty(self.builder.buffer_size(T, B, S, G, width), dtype=torch.int32, device=self.device)
        batch = self.builder.build(entries, self.cache, width=width, device_buffer=buffer, pad=pad)
        batch.padded = True
        self._feed(batch, token_feed)
        ops = self.model.rt.ops
        # the attention plans of the graph cover every context that fits the table width
        batch.attention_plans = self._plans(key, width * self.cache.page_size)
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
        steps = [k for k in self._graphs if k[0] != "decode"]
        if len(steps) > self.GRAPH_LIMIT:                 # dicts keep insertion order; a replay re-inserts its key
            del self._graphs[steps[0]]
        return eager_logits

    def finish(self, rid: Hashable) -> None:
        """The request has ended: everything it holds goes back to the pools."""
        if self.cache.has_request(rid):
            self.cache.release(rid)
