"""The cache manager: paged keys and values by cache group, and state slots.

What the reference has (include/pih/model/qwen3_kv_slot_pool.h:11-58,
qwen3_kv_block_table.h:13-33, qwen_kv_admission_coordinator.cpp:49-58): one
kind of page holding 16 tokens of all 28 layers, a block table per request,
the whole lifetime ``ceil((prompt + max_new) / 16)`` reserved at admission
and given back when the request has drained.

What is here instead:

* **Cache groups.**  Every schedule entry whose mixer asks for ``PagedKVNeed``
  joins the group of entries with the same (kv_heads, head_dim, window).  A
  group has a page pool of its own and one tensor
  ``[entries, pages, 2 (K,V), kv_heads, page_size, head_dim]``; a page id is
  valid for every entry of its group.  A request has one block table per
  group.
* **Pages on demand.**  ``append`` allocates the pages that the tokens of the
  coming step need, in all groups or in none; ``commit`` advances the
  request's length after the step has run (the reference's two-phase
  ``prepare_append`` / ``commit_append``, qwen3_kv_block_table.cpp:52-108)
  and gives back the pages of a windowed group that every later query has
  moved past.  ``release`` gives back everything a request holds.
* **State slots.**  Every live request holds one slot; mixers that ask for
  ``StateNeed`` get a tensor ``[slots, *shape]`` per entry, zeroed for the
  slot when a request takes it.  Qwen3 has no such mixer; the slots exist so
  that one can be added.  ``append`` keeps a copy of the request's slot as it
  is before the step, and ``rollback`` puts it back: a step that did not run
  to its end leaves no half-advanced state.
* **Lengths that count only once the step was seen to succeed.**  The
  reference advances a block table only after the step has completed without
  an error (qwen3_bf16_packed_batch_transaction.cpp:118-167).  A caller that
  queues steps on the device without waiting for them commits with
  ``confirmed=False``: the next step starts behind the queued tokens, but
  ``confirmed_tokens`` — and with it what a windowed group gives back —
  advances only at ``confirm``, after the step's error word has been read as
  zero.  ``rollback`` then returns the request to its confirmed length, pages
  and state.

Page ids in a block table are indexed by ``position // page_size``; an entry
of a windowed group that was given back reads -1.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.registry import PagedKVNeed, StateNeed
from .pools import OutOfPages, PagePool, StateSlotPool


@dataclass
class CacheGroup:
    need: PagedKVNeed
    entries: List[int]                 # schedule-entry indices, in order
    pool: PagePool
    kv: Optional[torch.Tensor] = None  # [entries, pages, 2, kv_heads, page_size, head_dim]


class PageList:
    """A request's page ids of one group, by page index, in an int32 array that grows by doubling
    (the batch builder copies slices of it straight into the step's block table).  -1 marks a page
    that was given back."""

    __slots__ = ("arr", "n")

    def __init__(self):
        self.arr = np.empty(16, dtype=np.int32)
        self.n = 0

    def __len__(self) -> int:
        return self.n

    def __getitem__(self, i):
        if isinstance(i, slice):
            return self.arr[:self.n][i].tolist()
        if not -self.n <= i < self.n:
            raise IndexError(i)
        return int(self.arr[i if i >= 0 else self.n + i])

    def __iter__(self):
        return iter(self.arr[:self.n].tolist())

    def __eq__(self, other):
        return list(self) == list(other)

    def extend(self, pages) -> None:
        k = len(pages)
        if self.n + k > self.arr.shape[0]:
            grown = np.empty(max(2 * self.arr.shape[0], self.n + k), dtype=np.int32)
            grown[:self.n] = self.arr[:self.n]
            self.arr = grown
        self.arr[self.n:self.n + k] = pages
        self.n += k

    def truncate(self, keep: int):
        """Drop the entries from index ``keep`` on and return them."""
        gone = self.arr[keep:self.n].tolist()
        self.n = min(self.n, keep)
        return gone

    def give_back(self, lo: int, hi: int):
        """Mark entries lo..hi-1 as given back and return the page ids they held."""
        gone = [p for p in self.arr[lo:hi].tolist() if p >= 0]
        self.arr[lo:hi] = -1
        return gone

    def held(self):
        a = self.arr[:self.n]
        return a[a >= 0].tolist()

    def view(self) -> np.ndarray:
        return self.arr[:self.n]


@dataclass
class RequestCache:
    rid: Hashable
    slot: int
    num_tokens: int = 0                               # committed length: where the next step starts
    pending: int = 0                                  # tokens appended, not yet committed
    confirmed_tokens: int = 0                         # length whose steps were seen to succeed (<= num_tokens)
    unconfirmed: List[int] = field(default_factory=list)   # token counts of committed steps not yet confirmed, oldest first
    state_before: List[Dict[int, torch.Tensor]] = field(default_factory=list)   # state slot before each of those steps
    state_pending: Optional[Dict[int, torch.Tensor]] = None   # ... and before the step being appended
    pages: List[PageList] = field(default_factory=list)    # per group: page id per page index, -1 = given back
    first_live: List[int] = field(default_factory=list)    # per group: first page index still held


@dataclass
class PagedCacheView:
    """What a mixer sees of the paged cache in one step."""
    kv: torch.Tensor                   # [pages, 2, kv_heads, page_size, head_dim] of one entry
    block_table: torch.Tensor          # int32 [R, width] of the entry's group, for this step
    slot_mapping: torch.Tensor         # int32 [T]: page * page_size + offset where each row's K/V goes
    page_size: int
    writable: bool                     # False: the entry reads another entry's cache
    window: Optional[int]


@dataclass
class StateCacheView:
    """What a mixer with per-request state sees: ``state[step.state_slots[r]]``."""
    state: torch.Tensor                # [slots, *shape]


class CacheManager:
    def __init__(self, needs: Sequence[Optional[object]], reads_cache_of: Sequence[Optional[int]],
                 page_size: int, num_pages: int, max_requests: int,
                 device: torch.device, dtype: torch.dtype, allocate_tensors: bool = True):
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.device = device
        self.dtype = dtype
        self.reads_cache_of = list(reads_cache_of)
        self.groups: List[CacheGroup] = []
        self.entry_group: Dict[int, Tuple[int, int]] = {}     # entry -> (group, index within the group)
        self.state_tensors: Dict[int, torch.Tensor] = {}
        by_key: Dict[Tuple, int] = {}
        for e, need in enumerate(needs):
            if isinstance(need, PagedKVNeed):
                key = (need.kv_heads, need.head_dim, need.window)
                if key not in by_key:
                    by_key[key] = len(self.groups)
                    self.groups.append(CacheGroup(need, [], PagePool(num_pages)))
                g = by_key[key]
                self.entry_group[e] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(e)
            elif isinstance(need, StateNeed):
                if allocate_tensors:
                    self.state_tensors[e] = torch.zeros((max_requests,) + tuple(need.shape),
                                                        dtype=need.dtype, device=device)
            elif need is not None:
                raise TypeError(f"schedule entry {e}: unknown cache need {need!r}")
        for e, src in enumerate(self.reads_cache_of):
            if src is not None:
                if src not in self.entry_group:
                    raise ValueError(f"schedule entry {e} reads the cache of entry {src}, which keeps no paged cache")
                self.entry_group[e] = self.entry_group[src]
        if allocate_tensors:
            for grp in self.groups:
                n = grp.need
                grp.kv = torch.zeros((len(grp.entries), num_pages, 2, n.kv_heads, page_size, n.head_dim),
                                     dtype=dtype, device=device)
        self.slots = StateSlotPool(max_requests)
        self.requests: Dict[Hashable, RequestCache] = {}

    # -- sizes ----------------------------------------------------------------
    def bytes_per_token(self) -> int:
        esize = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.entries) * 2 * g.need.kv_heads * g.need.head_dim * esize for g in self.groups)

    # -- requests -------------------------------------------------------------
    def add_request(self, rid: Hashable) -> RequestCache:
        if rid in self.requests:
            raise ValueError(f"request {rid!r} is already live")
        slot = self.slots.acquire(rid)
        rc = RequestCache(rid, slot, pages=[PageList() for _ in self.groups], first_live=[0 for _ in self.groups])
        self.requests[rid] = rc
        for t in self.state_tensors.values():
            t[slot].zero_()
        return rc

    def has_request(self, rid: Hashable) -> bool:
        return rid in self.requests

    def _first_needed_page(self, grp: CacheGroup, length: int) -> int:
        """Index of the first page that a query at position >= ``length`` can still read."""
        if grp.need.window is None:
            return 0
        return max(0, length - grp.need.window + 1) // self.page_size

    def pages_needed(self, rid: Hashable, n_new: int) -> List[int]:
        """Pages per group that ``append(rid, n_new)`` would allocate."""
        rc = self.requests[rid]
        end = rc.num_tokens + rc.pending + n_new
        want = -(-end // self.page_size)
        return [max(0, want - len(rc.pages[g])) for g in range(len(self.groups))]

    def can_append(self, asks: Sequence[Tuple[Hashable, int]]) -> bool:
        total = [0] * len(self.groups)
        for rid, n in asks:
            for g, c in enumerate(self.pages_needed(rid, n)):
                total[g] += c
        return all(total[g] <= self.groups[g].pool.num_free for g in range(len(self.groups)))

    def append(self, rid: Hashable, n_new: int) -> None:
        """Make room for the next ``n_new`` tokens of ``rid`` in every group, or in none."""
        if n_new < 1:
            raise ValueError("append needs at least one token")
        rc = self.requests[rid]
        need = self.pages_needed(rid, n_new)
        for g, c in enumerate(need):
            if c > self.groups[g].pool.num_free:
                raise OutOfPages(f"request {rid!r}: group {g} needs {c} pages, "
                                 f"{self.groups[g].pool.num_free} free")
        for g, c in enumerate(need):
            rc.pages[g].extend(self.groups[g].pool.allocate(c, rid))
        if rc.pending == 0 and self.state_tensors:
            # the state as it is before this step (copies queued on the current stream, ahead of the step)
            rc.state_pending = {e: t[rc.slot].clone() for e, t in self.state_tensors.items()}
        rc.pending += n_new

    def rollback(self, rid: Hashable, unconfirmed: bool = False) -> None:
        """Undo appends that were not committed (the step did not run): their pages go back, and the state
        slot is as it was before the step.  With ``unconfirmed`` also the committed steps that were not
        confirmed: the request returns to its confirmed length, pages and state."""
        rc = self.requests[rid]
        saved = rc.state_pending
        if unconfirmed:
            if rc.state_before:
                saved = rc.state_before[0]
            rc.num_tokens = rc.confirmed_tokens
            rc.unconfirmed.clear()
            rc.state_before.clear()
        keep = -(-rc.num_tokens // self.page_size)
        for g, grp in enumerate(self.groups):
            grp.pool.free([p for p in rc.pages[g].truncate(keep) if p >= 0], rid)
        if saved is not None:
            for e, t in saved.items():
                self.state_tensors[e][rc.slot].copy_(t)
        rc.pending = 0
        rc.state_pending = None

    def commit(self, rid: Hashable, confirmed: bool = True) -> None:
        """The step was run (``confirmed``) or queued on the device (not ``confirmed``): the appended tokens
        count for where the next step starts.  Once confirmed, pages that no later query can reach (windowed
        groups) go back to their pool."""
        rc = self.requests[rid]
        if confirmed and rc.unconfirmed:
            raise ValueError(f"request {rid!r} has queued steps to confirm before a confirmed commit")
        rc.num_tokens += rc.pending
        if confirmed:
            rc.confirmed_tokens = rc.num_tokens
            self._give_back(rc)
        else:
            rc.unconfirmed.append(rc.pending)
            if self.state_tensors:
                rc.state_before.append(rc.state_pending)
        rc.state_pending = None
        rc.pending = 0

    def confirm(self, rid: Hashable) -> None:
        """The oldest queued step of ``rid`` was seen to succeed."""
        rc = self.requests[rid]
        if not rc.unconfirmed:
            raise ValueError(f"request {rid!r} has no queued step to confirm")
        rc.confirmed_tokens += rc.unconfirmed.pop(0)
        if rc.state_before:
            rc.state_before.pop(0)
        self._give_back(rc)

    def _give_back(self, rc: RequestCache) -> None:
        for g, grp in enumerate(self.groups):
            first = self._first_needed_page(grp, rc.confirmed_tokens)
            if first > rc.first_live[g]:
                grp.pool.free(rc.pages[g].give_back(rc.first_live[g], first), rc.rid)
                rc.first_live[g] = first

    def release(self, rid: Hashable) -> None:
        rc = self.requests.pop(rid)
        for g, grp in enumerate(self.groups):
            grp.pool.free(rc.pages[g].held(), rid)
        self.slots.release(rc.slot, rid)

    def reset(self, rid: Hashable) -> None:
        """Give back a request's pages but keep it live with length 0
        (preemption: its tokens will be computed again)."""
        rc = self.requests[rid]
        for g, grp in enumerate(self.groups):
            grp.pool.free(rc.pages[g].held(), rid)
            rc.pages[g] = PageList()
            rc.first_live[g] = 0
        rc.num_tokens = rc.confirmed_tokens = 0
        rc.pending = 0
        rc.unconfirmed.clear()
        rc.state_before.clear()
        rc.state_pending = None
        for t in self.state_tensors.values():
            t[rc.slot].zero_()

    def num_free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def check(self) -> None:
        """Every page is free or held by exactly one live request's table."""
        self.slots.check()
        for g, grp in enumerate(self.groups):
            grp.pool.check()
            held = {}
            for rc in self.requests.values():
                for p in rc.pages[g]:
                    if p < 0:
                        continue
                    if p in held:
                        raise AssertionError(f"group {g}: page {p} is held by {held[p]!r} and {rc.rid!r}")
                    held[p] = rc.rid
                    if grp.pool.owner_of(p) != rc.rid:
                        raise AssertionError(f"group {g}: page {p} in {rc.rid!r}'s table is owned by "
                                             f"{grp.pool.owner_of(p)!r}")
            if len(held) + grp.pool.num_free != grp.pool.num_pages:
                raise AssertionError(f"group {g}: {grp.pool.num_pages - len(held) - grp.pool.num_free} pages are lost")

    # -- what a step needs -------------------------------------------------------
    def table_width(self, rids: Sequence[Hashable]) -> int:
        return max(1, max(len(self.requests[r].pages[g]) for r in rids for g in range(len(self.groups)))
                   if self.groups else 1)

    def block_table_rows(self, g: int, rids: Sequence[Hashable], width: int) -> List[List[int]]:
        rows = []
        for r in rids:
            pages = list(self.requests[r].pages[g])
            rows.append(pages + [-1] * (width - len(pages)))
        return rows

    def fill_block_table(self, g: int, rids: Sequence[Hashable], out: np.ndarray) -> None:
        """Write the block-table rows of ``rids`` (group g) into ``out`` [len(rids), width]."""
        for i, r in enumerate(rids):
            pages = self.requests[r].pages[g]
            n = pages.n
            out[i, :n] = pages.arr[:n]
            out[i, n:] = -1

    def slot_mapping(self, g: int, rid: Hashable, start: int, n: int) -> List[int]:
        pages = self.requests[rid].pages[g]
        ps = self.page_size
        out = []
        for pos in range(start, start + n):
            p = pages[pos // ps]
            if p < 0:
                raise AssertionError(f"request {rid!r}: position {pos} lies in a page that was given back")
            out.append(p * ps + pos % ps)
        return out

    def view(self, entry: int, block_tables: List[torch.Tensor], slot_mappings: List[torch.Tensor]):
        """The cache view of schedule entry ``entry`` for a step whose per-group
        block tables and slot mappings are given."""
        if entry in self.state_tensors:
            return StateCacheView(self.state_tensors[entry])
        if entry not in self.entry_group:
            return None
        g, idx = self.entry_group[entry]
        grp = self.groups[g]
        return PagedCacheView(kv=grp.kv[idx], block_table=block_tables[g], slot_mapping=slot_mappings[g],
                              page_size=self.page_size, writable=self.reads_cache_of[entry] is None,
                              window=grp.need.window)
