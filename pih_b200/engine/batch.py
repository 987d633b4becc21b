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

A step may be PADDED to larger counts of rows, requests and wanted rows, so that steps of different make-up have
one shape (one set of launch geometries, one captured graph).  What is padding is marked in the data, and every
kernel that reads it leaves padding alone: a padding row has token 0, position 0, request -1 and cache slot
``PAD_SLOT`` (nothing is written for it); a padding request has no rows (cu_q stays at the number of real rows),
length 0, state slot -1 and a block table of -1; a padding wanted row repeats row 0.  The rows of padding run
through the row-wise kernels and the products like any other and are never read.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, List, Optional, Sequence

import numpy as np
import torch


PAD_SLOT = -2          # slot_mapping of a row that belongs to no request (a negative slot otherwise is an error)


@dataclass
class StepEntry:
    rid: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()          # places among ``tokens`` whose logits are wanted


@dataclass
class StepBatch:
    num_rows: int                      # with padding: the tensors' sizes, which the kernels' launches follow
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
    meta: torch.Tensor = None              # int32 [4] on the device: (longest context after the step, rows, requests, wanted)
    block_tables: List[torch.Tensor] = field(default_factory=list)
    slot_mappings: List[torch.Tensor] = field(default_factory=list)
    # host copies for planning kernel launches
    host_cu_q: List[int] = field(default_factory=list)
    host_q_start: List[int] = field(default_factory=list)
    attention_plans: dict = field(default_factory=dict)     # filled by the attention op, per group size
    padded: bool = False               # of a shape that other steps share (by padding, or by its nature)
    real_rows: int = 0                 # without padding
    real_requests: int = 0
    real_logit_rows: int = 0


def _align(n: int, a: int = 4) -> int:
    return -(-n // a) * a


class BatchBuilder:
    """Builds StepBatch objects through one reusable pinned buffer."""

    def __init__(self, device: torch.device):
        self.device = device
        self._pinned = None
        self._capacity = 0
        self.last_bytes = 0
        self._copy_done = None
        self._copy_pending = False

    def _host(self, n: int) -> torch.Tensor:
        if n > self._capacity:
            self._capacity = max(2 * n, 4096)
            pin = self.device.type == "cuda"
            self._pinned = torch.empty(self._capacity, dtype=torch.int32, pin_memory=pin)
        return self._pinned[:n]

    def build(self, entries: Sequence[StepEntry], cache, width: Optional[int] = None,
              device_buffer: Optional[torch.Tensor] = None, pad=None) -> StepBatch:
        """``cache``: the CacheManager, after ``append`` was called for every entry.

        ``width`` fixes the block tables' row length (default: the longest table of the batch);
        ``device_buffer`` is an int32 device tensor to fill instead of a fresh one.  The layout is a
        function of (rows, requests, wanted rows, groups, width) alone, so a step of the same shape
        written into the same buffer puts every array at the same address — what a captured CUDA
        graph needs.  ``pad``: (rows, requests, wanted rows) to pad the step to (each at least the real count).
        """
        R = len(entries)
        rids = [e.rid for e in entries]
        reqs = [cache.requests[r] for r in rids]
        counts = [len(e.tokens) for e in entries]
        T = sum(counts)
        starts = [rc.num_tokens for rc in reqs]
        G = len(cache.groups)
        ps = cache.page_size
        if width is None:
            width = cache.table_width(rids)
        cu_q = [0]
        for n in counts:
            cu_q.append(cu_q[-1] + n)
        logit_rows = []
        for r, e in enumerate(entries):
            for w in e.want:
                if not 0 <= w < counts[r]:
                    raise ValueError(f"request {e.rid!r}: wanted place {w} is outside its {counts[r]} tokens")
                logit_rows.append(cu_q[r] + int(w))
        S = len(logit_rows)
        Tp, Rp, Sp = (T, R, S) if pad is None else pad
        if Tp < T or Rp < R or Sp < S:
            raise ValueError("a step cannot be padded to less than it holds")
        sizes = self._sizes(Tp, Rp, Sp, G, width)
        offsets, total = [], 0
        for n in sizes:
            offsets.append(total)
            total += _align(max(n, 1))
        self.wait_copy()
        host = self._host(total)
        v = host.numpy()
        o = offsets
        if T == R:                                   # one token each: no per-request loops over rows
            v[o[0]:o[0] + T] = [e.tokens[0] for e in entries]
            v[o[1]:o[1] + T] = starts
            v[o[2]:o[2] + T] = np.arange(R, dtype=np.int32)
        else:
            for r, e in enumerate(entries):
                lo, hi = cu_q[r], cu_q[r + 1]
                v[o[0] + lo:o[0] + hi] = e.tokens
                v[o[1] + lo:o[1] + hi] = np.arange(starts[r], starts[r] + counts[r], dtype=np.int32)
                v[o[2] + lo:o[2] + hi] = r
        if pad is not None:
            v[o[0] + T:o[0] + Tp] = 0
            v[o[1] + T:o[1] + Tp] = 0
            v[o[2] + T:o[2] + Tp] = -1
            v[o[3] + S:o[3] + Sp] = 0
            v[o[4] + R + 1:o[4] + Rp + 1] = T
            v[o[5] + R:o[5] + Rp] = 0
            v[o[6] + R:o[6] + Rp] = 0
            v[o[7] + R:o[7] + Rp] = -1
        if S:
            v[o[3]:o[3] + S] = logit_rows
        v[o[4]:o[4] + R + 1] = cu_q
        v[o[5]:o[5] + R] = starts
        v[o[6]:o[6] + R] = [starts[r] + counts[r] for r in range(R)]
        v[o[7]:o[7] + R] = [rc.slot for rc in reqs]
        v[o[8]:o[8] + 4] = [max(starts[r] + counts[r] for r in range(R)), T, R, S]
        for g in range(G):
            table = v[o[9 + 2 * g]:o[9 + 2 * g] + R * width].reshape(R, width)
            cache.fill_block_table(g, rids, table)
            if pad is not None:
                v[o[9 + 2 * g] + R * width:o[9 + 2 * g] + Rp * width] = -1
                v[o[10 + 2 * g] + T:o[10 + 2 * g] + Tp] = PAD_SLOT
            sm = v[o[10 + 2 * g]:o[10 + 2 * g] + T]
            for r, rc in enumerate(reqs):
                pages = rc.pages[g].arr
                lo, n, st = cu_q[r], counts[r], starts[r]
                if n == 1:
                    page = pages[st // ps]
                    sm[lo] = page * ps + st % ps if page >= 0 else -1
                else:
                    pos = np.arange(st, st + n, dtype=np.int64)
                    page = pages[pos // ps].astype(np.int64)
                    sm[lo:lo + n] = np.where(page >= 0, page * ps + pos % ps, -1)
            if (sm < 0).any():
                raise AssertionError("a row of this step lies in a page that was given back")
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
            if self._copy_done is None:
                self._copy_done = torch.cuda.Event()
            self._copy_done.record()
            self._copy_pending = True

        def part(i, n):
            return dev[offsets[i]:offsets[i] + n]

        batch = StepBatch(
            num_rows=Tp, num_requests=Rp, num_logit_rows=Sp, max_q=max(counts),
            max_ctx=max(starts[r] + counts[r] for r in range(R)),
            token_ids=part(0, Tp), positions=part(1, Tp), request_of_row=part(2, Tp),
            logit_rows=part(3, Sp), cu_q=part(4, Rp + 1), q_start=part(5, Rp), ctx_len=part(6, Rp),
            state_slots=part(7, Rp), meta=part(8, 4), host_cu_q=cu_q + [T] * (Rp - R),
            host_q_start=starts + [0] * (Rp - R), real_rows=T, real_requests=R, real_logit_rows=S,
            padded=pad is not None)
        for g in range(G):
            batch.block_tables.append(part(9 + 2 * g, Rp * width).view(Rp, width))
            batch.slot_mappings.append(part(10 + 2 * g, Tp))
        return batch

    @staticmethod
    def _sizes(rows: int, requests: int, wanted: int, groups: int, width: int):
        sizes = [rows, rows, rows, wanted, requests + 1, requests, requests, requests, 4]
        for _ in range(groups):
            sizes += [requests * width, rows]
        return sizes

    @staticmethod
    def buffer_size(rows: int, requests: int, wanted: int, groups: int, width: int) -> int:
        """int32 elements that ``build`` needs for a step of this shape."""
        return sum(_align(max(n, 1)) for n in BatchBuilder._sizes(rows, requests, wanted, groups, width))

    def wait_copy(self) -> None:
        if self._copy_pending:
            self._copy_done.synchronize()
            self._copy_pending = False
