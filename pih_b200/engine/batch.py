"""The packed batch of one step: rows of several requests side by side.

The reference packs a step into 14 host arrays and uploads each with its own
copy (plugins/model-qwen3/qwen3_bf16_packed_step_staging_layout.cpp:60-97;
arrays listed in plugins/execution-default/packed_token_metadata_arena.cpp:58-116:
token ids, positions, request index per row, query start offsets, sample
rows).  Its plans hold prompt portions or single decode tokens, never both
(include/pih/model/packed_token_plan.h:36-37).  Here one step holds any mix:
each request contributes ``n >= 1`` consecutive tokens that start at its
committed length.  All integer arrays are laid out in ONE pinned host buffer
and reach the device with one copy.

Arrays (int32, on the device):
  token_ids[T], positions[T], request_of_row[T], logit_rows[S],
  cu_q[R+1] (row range of request r is cu_q[r]..cu_q[r+1]),
  q_start[R] (length before this step), ctx_len[R] (length after it),
  state_slots[R], and per cache group block_table[R, width] and
  slot_mapping[T].
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import torch


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are wanted


@dataclass
class StepBatch:
    num_rows: int
    num_requests: int
    num_logit_rows: int
    max_q: int                         # most rows of one request
    max_ctx: int                       # longest context after the step
    token_ids: torch.Tensor
    positions: torch.Tensor
    request_of_row: torch.Tensor
    logit_rows: torch.Tensor
    cu_q: torch.Tensor
    q_start: torch.Tensor
    ctx_len: torch.Tensor
    state_slots: torch.Tensor
    block_tables: List[torch.Tensor] = field(default_factory=list)
    slot_mappings: List[torch.Tensor] = field(default_factory=list)
    # host copies for planning kernel launches
    host_cu_q: List[int] = field(default_factory=list)
    host_q_start: List[int] = field(default_factory=list)
    attention_plans: dict = field(default_factory=dict)     # filled by the attention op, per group size


def _align(n: int, a: int = 4) -> int:
    return -(-n // a) * a


class BatchBuilder:
    """Builds StepBatch objects through one reusable pinned buffer."""

    def __init__(self, device: torch.device):
        self.device = device
        self._pinned = None
        self._capacity = 0
        self.last_bytes = 0

    def _host(self, n: int) -> torch.Tensor:
        if n > self._capacity:
            self._capacity = max(2 * n, 4096)
            pin = self.device.type == "cuda"
            self._pinned = torch.empty(self._capacity, dtype=torch.int32, pin_memory=pin)
        return self._pinned[:n]

    def build(self, entries: Sequence[StepEntry], cache, width: Optional[int] = None,
              device_buffer: Optional[torch.Tensor] = None) -> StepBatch:
        """``cache``: the CacheManager, after ``append`` was called for every entry.

        ``width`` fixes the block tables' row length (default: the longest table of the batch);
        ``device_buffer`` is an int32 device tensor to fill instead of a fresh one.  The layout is a
        function of (rows, requests, wanted rows, groups, width) alone, so a step of the same shape
        written into the same buffer puts every array at the same address — what a captured CUDA
        graph needs.
        """
        R = len(entries)
        rids = [e.rid for e in entries]
        counts = [len(e.tokens) for e in entries]
        T = sum(counts)
        starts = [cache.requests[r].num_tokens for r in rids]
        G = len(cache.groups)
        if width is None:
            width = cache.table_width(rids)
        token_ids, positions, req_of_row, logit_rows, cu_q = [], [], [], [], [0]
        for r, e in enumerate(entries):
            token_ids.extend(e.tokens)
            positions.extend(range(starts[r], starts[r] + counts[r]))
            req_of_row.extend([r] * counts[r])
            for w in e.want:
                if not 0 <= w < counts[r]:
                    raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {counts[r]} tokens")
                logit_rows.append(cu_q[-1] + int(w))
            cu_q.append(cu_q[-1] + counts[r])
        S = len(logit_rows)
        fields = [token_ids, positions, req_of_row, logit_rows, cu_q, starts,
                  [starts[r] + counts[r] for r in range(R)],
                  [cache.requests[r].slot for r in rids]]
        for g in range(G):
            fields.append([p for row in cache.block_table_rows(g, rids, width) for p in row])
            sm = []
            for r, rid in enumerate(rids):
                sm.extend(cache.slot_mapping(g, rid, starts[r], counts[r]))
            fields.append(sm)
        offsets, total = [], 0
        for f in fields:
            offsets.append(total)
            total += _align(max(len(f), 1))
        self.wait_copy()
        host = self._host(total)
        view = host.numpy()
        for off, f in zip(offsets, fields):
            if f:
                view[off:off + len(f)] = f
        self.last_bytes = total * 4
        if device_buffer is None:
            dev = torch.empty(total, dtype=torch.int32, device=self.device)
        else:
            if device_buffer.numel() < total:
                raise ValueError("the device buffer is too small for this batch")
            dev = device_buffer[:total]
        dev.copy_(host, non_blocking=True)
        # the pinned buffer is reused by the next build: the copy must have left it
        if self.device.type == "cuda":
            self._copy_done = torch.cuda.Event()
            self._copy_done.record()

        def part(i, n):
            return dev[offsets[i]:offsets[i] + n]

        batch = StepBatch(
            num_rows=T, num_requests=R, num_logit_rows=S, max_q=max(counts),
            max_ctx=max(starts[r] + counts[r] for r in range(R)),
            token_ids=part(0, T), positions=part(1, T), request_of_row=part(2, T),
            logit_rows=part(3, S), cu_q=part(4, R + 1), q_start=part(5, R), ctx_len=part(6, R),
            state_slots=part(7, R), host_cu_q=cu_q, host_q_start=starts)
        for g in range(G):
            batch.block_tables.append(part(8 + 2 * g, R * width).view(R, width))
            batch.slot_mappings.append(part(9 + 2 * g, T))
        return batch

    @staticmethod
    def buffer_size(rows: int, requests: int, wanted: int, groups: int, width: int) -> int:
        """int32 elements that ``build`` needs for a step of this shape."""
        sizes = [rows, rows, rows, wanted, requests + 1, requests, requests, requests]
        for _ in range(groups):
            sizes += [requests * width, rows]
        return sum(_align(max(n, 1)) for n in sizes)

    def wait_copy(self) -> None:
        ev = getattr(self, "_copy_done", None)
        if ev is not None:
            ev.synchronize()
            self._copy_done = None
