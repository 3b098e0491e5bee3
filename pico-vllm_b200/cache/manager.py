"""The cache manager: keys and values in pages with a block table per request, groups of
layers with pages of their own, and slots for per-request state of fixed size.

Cache entries (one per layer call that keeps a cache) with the same paged needs (for keys and
values: heads, head size, window) form a *group*.  A group has its own page pool, its own block
tables and, for every tensor its spec names, one device tensor [entries, num_pages, *page shape]
(keys and values: [entries, num_pages, kv_heads, page_size, head_dim] each); a page number means
the same page in every entry of the group, as one block id spans all layers in the reference
(pico_vllm/blockmanager.py:39-42).  Which spec classes are paged and which are fixed-size state is
looked up in ``cache/kinds.py``.  A request holds a *slot* (0..max_num_seqs-1) from admission
to its end; the slot indexes the block tables and the fixed-size state tensors.

Pages are taken when tokens are appended (``append``), given back when the request ends
(``release``) and, in a group with a window W, as soon as every position of a page is older than
the last W (``commit``): the next query, at position L, reads keys L-W+1 .. L only.
The reference frees only at the end of a request (pico_vllm/cache.py:158-167) and raises when
the pool is empty (pico_vllm/blockmanager.py:77-78); here the scheduler asks ``can_append``
first.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..errors import OutOfPages, PicoError, ScheduleError
from ..parts.base import CacheView
from .kinds import kind_of
from .pages import PagePool


@dataclass
class KVGroup:
    spec: object                       # a paged spec: page_tensors(page_size), window
    entries: List[int]                 # cache entry ids served by this group, in order
    pool: PagePool
    tables: np.ndarray                 # int32 [max_num_seqs, max_blocks]; -1 = no page
    first_block: np.ndarray            # int32 [max_num_seqs]; blocks below were given back
    end_block: np.ndarray              # int32 [max_num_seqs]; blocks first_block .. end_block-1 hold pages
    tensors: Dict[str, torch.Tensor] = field(default_factory=dict)   # name -> [len(entries), num_pages, *page shape]

    @property
    def k(self) -> Optional[torch.Tensor]:
        return self.tensors.get("k")

    @property
    def v(self) -> Optional[torch.Tensor]:
        return self.tensors.get("v")


class CacheManager:
    def __init__(self, cache_entries: Sequence, page_size: int, num_pages: int, max_num_seqs: int,
                 max_seq_len: int, dtype: torch.dtype = torch.bfloat16, device="cpu", allocate: bool = True,
                 poison_freed: bool = False):
        self.page_size, self.num_pages, self.max_num_seqs = page_size, num_pages, max_num_seqs
        self.max_seq_len = max_seq_len
        self.max_blocks = -(-max_seq_len // page_size)
        self.dtype, self.device = dtype, torch.device(device)
        self.poison_freed = poison_freed
        self.groups: List[KVGroup] = []
        self.entry_group: Dict[int, tuple] = {}     # entry id -> (group index, index inside the group)
        self.states: Dict[int, torch.Tensor] = {}   # entry id -> [max_num_seqs, *shape]
        self.state_specs: Dict[int, object] = {}
        for eid, spec in enumerate(cache_entries):
            kind = kind_of(spec)
            if kind == "paged":
                for gi, g in enumerate(self.groups):
                    if g.spec == spec:
                        self.entry_group[eid] = (gi, len(g.entries))
                        g.entries.append(eid)
                        break
                else:
                    self.entry_group[eid] = (len(self.groups), 0)
                    self.groups.append(KVGroup(spec, [eid], PagePool(num_pages),
                                               np.full((max_num_seqs, self.max_blocks), -1, np.int32),
                                               np.zeros(max_num_seqs, np.int32), np.zeros(max_num_seqs, np.int32)))
            else:
                self.state_specs[eid] = spec
        if allocate:
            for g in self.groups:
                for name, page_shape in g.spec.page_tensors(page_size).items():
                    g.tensors[name] = torch.zeros((len(g.entries), num_pages) + tuple(page_shape), dtype=dtype,
                                                  device=self.device)
            for eid, spec in self.state_specs.items():
                self.states[eid] = torch.zeros((max_num_seqs,) + tuple(spec.shape),
                                               dtype=getattr(torch, spec.dtype), device=self.device)
        self._free_slots = list(range(max_num_seqs - 1, -1, -1))
        self.seq_len = np.zeros(max_num_seqs, np.int64)   # tokens committed per slot
        self.pending = np.zeros(max_num_seqs, np.int64)   # tokens appended, not yet committed
        self.owner: List[Optional[object]] = [None] * max_num_seqs

    # ------------------------------------------------------------------ sizes
    def bytes_per_page(self) -> int:
        item = torch.empty((), dtype=self.dtype).element_size()
        return sum(len(g.entries) * int(np.prod(shape)) * item
                   for g in self.groups for shape in g.spec.page_tensors(self.page_size).values())

    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    # ------------------------------------------------------------------ requests
    def acquire(self, owner=None) -> int:
        """A slot for a new request: empty block tables, zeroed state."""
        if not self._free_slots:
            raise ScheduleError("no request slot is free")
        slot = self._free_slots.pop()
        self.owner[slot] = owner if owner is not None else True
        self.seq_len[slot] = 0
        self.pending[slot] = 0
        for g in self.groups:
            g.first_block[slot] = 0
            g.end_block[slot] = 0
        for st in self.states.values():
            st[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        """The request is over (or pre-empted): all its pages and its slot come back."""
        if self.owner[slot] is None:
            raise PicoError(f"slot {slot} is released but not held")
        for g in self.groups:
            row = g.tables[slot]
            held = row[row >= 0].tolist()
            self._give_back(g, held)
            row[:] = -1
            g.end_block[slot] = 0
        self.owner[slot] = None
        self.seq_len[slot] = 0
        self.pending[slot] = 0
        self._free_slots.append(slot)

    def _give_back(self, g: KVGroup, pages: List[int]) -> None:
        freed = g.pool.release(pages)
        if self.poison_freed and freed and g.tensors:
            idx = torch.tensor(freed, dtype=torch.long, device=self.device)
            for t in g.tensors.values():
                t[:, idx] = float("nan")

    # ------------------------------------------------------------------ pages for new tokens
    def _blocks_missing(self, g: KVGroup, slot: int, new_len: int) -> int:
        # pages are taken block after block, so the blocks that hold pages are first_block .. end_block - 1
        return max(0, -(-new_len // self.page_size) - int(g.end_block[slot]))

    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        """Pages each group would have to take to hold n_new more tokens of this request."""
        new_len = int(self.seq_len[slot] + self.pending[slot]) + n_new
        return [self._blocks_missing(g, slot, new_len) for g in self.groups]

    def can_append(self, slot: int, n_new: int, reserve: Optional[List[int]] = None) -> bool:
        """True if every group has the pages (beyond ``reserve``, pages promised to others)."""
        new_len = int(self.seq_len[slot] + self.pending[slot]) + n_new
        if new_len > self.max_seq_len:
            return False
        need = self.pages_needed(slot, n_new)
        return all(n <= g.pool.available - (reserve[i] if reserve else 0)
                   for i, (n, g) in enumerate(zip(need, self.groups)))

    def append(self, slot: int, n_new: int) -> int:
        """Takes pages for positions [len, len + n_new) in every group; all or nothing.
        Returns the position of the first new token."""
        start = int(self.seq_len[slot] + self.pending[slot])
        new_len = start + n_new
        if self.owner[slot] is None:
            raise PicoError(f"slot {slot} is not held")
        if new_len > self.max_seq_len:
            raise ScheduleError(f"request would reach {new_len} tokens, the cache holds {self.max_seq_len} per request")
        need = self.pages_needed(slot, n_new)
        for n, g in zip(need, self.groups):
            if n > g.pool.available:
                raise OutOfPages(f"{n} pages wanted for {n_new} tokens, {g.pool.available} of {g.pool.num_pages} free")
        for n, g in zip(need, self.groups):
            if n:
                end = int(g.end_block[slot])
                g.tables[slot, end:end + n] = g.pool.allocate(n)
                g.end_block[slot] = end + n
        self.pending[slot] += n_new
        return start

    def rollback(self, slot: int) -> None:
        """Forgets appended-but-uncommitted tokens (their pages stay with the request)."""
        self.pending[slot] = 0

    def commit(self, slot: int) -> None:
        """The appended tokens are in the cache now.  Gives back pages that a window has passed."""
        self.seq_len[slot] += self.pending[slot]
        self.pending[slot] = 0
        L = int(self.seq_len[slot])
        for g in self.groups:
            W = g.spec.window
            if W is None:
                continue
            dead_blocks = max(0, (L - W + 1)) // self.page_size  # blocks wholly below position L-W+1
            fb = int(g.first_block[slot])
            if dead_blocks > fb:
                row = g.tables[slot]
                held = [int(p) for p in row[fb:dead_blocks] if p >= 0]
                self._give_back(g, held)
                row[fb:dead_blocks] = -1
                g.first_block[slot] = dead_blocks

    # ------------------------------------------------------------------ what kernels read
    def slot_mapping(self, group: int, slot: int, start: int, n: int) -> np.ndarray:
        """Cache row (page * page_size + offset) of positions start .. start+n-1
        (pico_vllm/cache.py:132-156)."""
        pos = np.arange(start, start + n, dtype=np.int64)
        pages = self.groups[group].tables[slot][pos // self.page_size].astype(np.int64)
        if (pages < 0).any():
            raise PicoError(f"slot {slot}: positions {start}..{start + n - 1} have no page")
        return (pages * self.page_size + pos % self.page_size).astype(np.int32)

    def slot_mapping_single(self, group: int, slots: np.ndarray, positions: np.ndarray) -> np.ndarray:
        """The same for one position of each of many requests (a decode step), without a loop."""
        pages = self.groups[group].tables[slots, positions // self.page_size].astype(np.int64)
        if (pages < 0).any():
            bad = int(slots[np.argmax(pages < 0)])
            raise PicoError(f"slot {bad}: its next position has no page")
        return (pages * self.page_size + positions % self.page_size).astype(np.int32)

    def table_row(self, group: int, slot: int) -> np.ndarray:
        return self.groups[group].tables[slot]

    def views(self) -> List[CacheView]:
        """One CacheView per cache entry, in entry order."""
        out: List[CacheView] = []
        n = len(self.entry_group) + len(self.state_specs)
        for eid in range(n):
            if eid in self.entry_group:
                gi, idx = self.entry_group[eid]
                g = self.groups[gi]
                mine = {name: t[idx] for name, t in g.tensors.items()}
                view = CacheView(group=gi, k=mine.get("k"), v=mine.get("v"), page_size=self.page_size, tensors=mine)
                if view.k is not None and view.v is not None and view.k.is_cuda and view.k.dtype == torch.bfloat16 \
                        and view.k.dim() == 4 and view.k.shape == view.v.shape:
                    from .. import ops
                    view.k_map, view.v_map = ops.make_kv_tensor_map(view.k), ops.make_kv_tensor_map(view.v)
                    view.k_map2d, view.v_map2d = ops.make_kv_tensor_map_2d(view.k), ops.make_kv_tensor_map_2d(view.v, values=True)
                out.append(view)
            else:
                out.append(CacheView(state=self.states.get(eid)))
        return out

    # ------------------------------------------------------------------ checks (tests, debugging)
    def check(self) -> None:
        """No page lost, held twice or free while held."""
        for gi, g in enumerate(self.groups):
            held: Dict[int, int] = {}
            for slot in range(self.max_num_seqs):
                row = g.tables[slot]
                pages = row[row >= 0].tolist()
                if self.owner[slot] is None and pages:
                    raise PicoError(f"group {gi}: free slot {slot} still lists pages {pages}")
                for p in pages:
                    held[p] = held.get(p, 0) + 1
            for p, c in held.items():
                if g.pool.refcount(p) != c:
                    raise PicoError(f"group {gi}: page {p} listed {c} times, count {g.pool.refcount(p)}")
            free = list(g.pool._free)
            if len(set(free)) != len(free):
                raise PicoError(f"group {gi}: a page is twice in the free list")
            if set(free) & set(held):
                raise PicoError(f"group {gi}: pages {sorted(set(free) & set(held))} are free and held")
            if len(free) + len(held) != g.pool.num_pages:
                raise PicoError(f"group {gi}: {g.pool.num_pages - len(free) - len(held)} pages lost")
