"""The cache manager: pages of keys and values with a block table per request,
groups of layers with different needs, and slots for per-request state of fixed size.

* A **page** holds ``page_size`` consecutive positions of one request for one layer:
  K and V tensors of shape [n_pages, n_kv_heads, page_size, head_dim] per cache
  index.  A page *id* is valid in every layer of its **group**: the layers of a
  group share one id space, one free list and one block table per request.
* **Groups** are formed by what the layers need: all earlier keys (window None) or
  the last W positions.  A windowed group gives pages back as soon as every
  position in them has fallen out of the window of the request's next query; the
  group of full layers keeps them until the request ends.
* A request holds a **slot**: the row of its block tables and the index of its
  state in every :class:`StateSpec` tensor ([max_slots, *shape], zeroed at
  admission).  Freed pages and slots are used again, most recently freed first.
* ``reserve`` either gets every page the request needs up to a new length, in every
  group, or changes nothing and returns False; what to do then is the scheduler's
  decision.

Reference: ``PagedKvStore`` / ``PagedKvCache`` (crates/ferrox-core/src/cache.rs:
331-405, 427-488: shared physical pages, LIFO free list, per-sequence block table,
new block when seq_len % block_size == 0, exhaustion returned as a value with the
state unchanged :452-476).  The reference keeps one store per layer and never
evicts for windowed layers (attention.rs:506 only *reads* the tail); groups and
window release are this engine's own.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .specs import CacheSpec


class CacheError(RuntimeError):
    pass


class PagePool:
    """Page ids 0..n-1 with a LIFO free list.  ``alloc`` is all-or-nothing."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._free: List[int] = list(range(self.n_pages - 1, -1, -1))  # pop() hands out ascending ids first
        self._held = bytearray(self.n_pages)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = 1
        return out

    def free(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.n_pages or not self._held[p]:
                raise CacheError(f"page {p} freed but not held")
            self._held[p] = 0
            self._free.append(p)

    def held(self) -> int:
        return self.n_pages - len(self._free)


@dataclass
class LayerCache:
    """What a mixer sees of the cache while one schedule entry runs."""

    k: Optional[torch.Tensor]
    v: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]  # device int32 [max_slots, table_width]; -1 = no page
    page_size: int
    state: Optional[torch.Tensor]  # [max_slots, *shape]
    writes: bool = True
    window: Optional[int] = None


class _Group:
    def __init__(self, window, n_pages, max_slots, width, device):
        self.window = window
        self.caches: List[int] = []
        self.pool = PagePool(n_pages)
        self.table = np.full((max_slots, width), -1, dtype=np.int32)
        self.table_dev = torch.full((max_slots, width), -1, dtype=torch.int32, device=device)
        self.first_page = [0] * max_slots  # first logical page still held
        self.n_logical = [0] * max_slots  # logical pages ever mapped (held or given back)
        self.dirty = set()


class CacheManager:
    def __init__(
        self,
        cache_specs: Sequence[Optional[CacheSpec]],
        *,
        page_size: int,
        n_pages,
        max_slots: int,
        max_positions: int,
        device,
        dtype: torch.dtype,
    ):
        """``n_pages``: pages per group (an int for all groups, or {window: n})."""
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        self.page_size = int(page_size)
        self.max_slots = int(max_slots)
        self.max_positions = int(max_positions)
        self.device = torch.device(device)
        self.dtype = dtype
        self.table_width = (self.max_positions + self.page_size - 1) // self.page_size
        self.groups: Dict[object, _Group] = {}
        self._group_of: List[Optional[_Group]] = []
        self._k: List[Optional[torch.Tensor]] = []
        self._v: List[Optional[torch.Tensor]] = []
        self._state: List[Optional[torch.Tensor]] = []
        for idx, cs in enumerate(cache_specs):
            g = None
            k = v = st = None
            if cs is not None and cs.kv is not None:
                key = cs.kv.window
                if key not in self.groups:
                    n = n_pages[key] if isinstance(n_pages, dict) else int(n_pages)
                    self.groups[key] = _Group(key, n, self.max_slots, self.table_width, self.device)
                g = self.groups[key]
                g.caches.append(idx)
                shape = (g.pool.n_pages, cs.kv.n_kv_heads, self.page_size, cs.kv.head_dim)
                k = torch.zeros(shape, dtype=dtype, device=self.device)
                v = torch.zeros(shape, dtype=dtype, device=self.device)
            if cs is not None and cs.state is not None:
                st = torch.zeros((self.max_slots, *cs.state.shape), dtype=cs.state.dtype, device=self.device)
            self._group_of.append(g)
            self._k.append(k)
            self._v.append(v)
            self._state.append(st)
        self._free_slots: List[int] = list(range(self.max_slots - 1, -1, -1))
        self._live = bytearray(self.max_slots)
        self.seq_len = [0] * self.max_slots
        self.peak_pages = {key: 0 for key in self.groups}

    # ---- requests -------------------------------------------------------------
    @property
    def n_free_slots(self) -> int:
        return len(self._free_slots)

    def open_request(self) -> Optional[int]:
        """A slot for a new request (its state zeroed), or None when all are taken."""
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self._live[slot] = 1
        self.seq_len[slot] = 0
        for st in self._state:
            if st is not None:
                st[slot].zero_()
        return slot

    def close_request(self, slot: int) -> None:
        """Give back everything the request holds."""
        self._check_live(slot)
        for g in self.groups.values():
            held = [int(p) for p in g.table[slot, g.first_page[slot]:g.n_logical[slot]] if p >= 0]
            g.pool.free(held)
            if g.n_logical[slot]:
                g.table[slot, :g.n_logical[slot]] = -1
                g.dirty.add(slot)
            g.first_page[slot] = 0
            g.n_logical[slot] = 0
        self.seq_len[slot] = 0
        self._live[slot] = 0
        self._free_slots.append(slot)

    def _check_live(self, slot: int) -> None:
        if not 0 <= slot < self.max_slots or not self._live[slot]:
            raise CacheError(f"slot {slot} is not held by a request")

    # ---- pages ----------------------------------------------------------------
    def _pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def pages_needed(self, slot: int, new_len: int) -> Dict[object, int]:
        """Pages each group still has to get so that positions < new_len are mapped."""
        need = self._pages_for(new_len)
        return {key: max(0, need - g.n_logical[slot]) for key, g in self.groups.items()}

    def free_pages(self) -> Dict[object, int]:
        return {key: g.pool.n_free for key, g in self.groups.items()}

    def can_reserve(self, wanted: Dict[object, int]) -> bool:
        return all(self.groups[key].pool.n_free >= n for key, n in wanted.items())

    def reserve(self, slot: int, new_len: int) -> bool:
        """Map pages for every position < new_len in every group, or change nothing."""
        self._check_live(slot)
        if new_len > self.max_positions:
            raise CacheError(f"length {new_len} exceeds max_positions {self.max_positions}")
        wanted = self.pages_needed(slot, new_len)
        if not self.can_reserve(wanted):
            return False
        for key, n in wanted.items():
            if n == 0:
                continue
            g = self.groups[key]
            pages = g.pool.alloc(n)
            a = g.n_logical[slot]
            g.table[slot, a:a + n] = pages
            g.n_logical[slot] = a + n
            g.dirty.add(slot)
            self.peak_pages[key] = max(self.peak_pages[key], g.pool.held())
        return True

    def commit(self, slot: int, new_len: int) -> None:
        """The request now holds ``new_len`` positions.  Windowed groups give back the
        pages that no later query can read: the next query, at position new_len,
        reads from new_len - W + 1 on."""
        self._check_live(slot)
        if new_len < self.seq_len[slot]:
            raise CacheError("a request's length cannot shrink")
        self.seq_len[slot] = new_len
        for g in self.groups.values():
            if g.window is None:
                continue
            first_needed = max(0, new_len - g.window + 1)
            upto = min(first_needed // self.page_size, g.n_logical[slot])
            a = g.first_page[slot]
            if upto > a:
                g.pool.free([int(p) for p in g.table[slot, a:upto]])
                g.table[slot, a:upto] = -1
                g.first_page[slot] = upto
                g.dirty.add(slot)

    def held_pages(self, slot: int) -> Dict[object, List[int]]:
        return {
            key: [int(p) for p in g.table[slot, g.first_page[slot]:g.n_logical[slot]]]
            for key, g in self.groups.items()
        }

    # ---- device side ----------------------------------------------------------
    def sync_tables(self) -> None:
        """Bring the device copies of the changed block-table rows up to date."""
        for g in self.groups.values():
            if not g.dirty:
                continue
            rows = sorted(g.dirty)
            g.dirty.clear()
            if len(rows) == 1:
                r = rows[0]
                g.table_dev[r].copy_(torch.from_numpy(g.table[r]), non_blocking=False)
            else:
                idx = torch.tensor(rows, dtype=torch.long)
                g.table_dev[idx.to(self.device)] = torch.from_numpy(g.table[rows]).to(self.device)

    def layer_cache(self, cache_index: int, writes: bool = True) -> LayerCache:
        g = self._group_of[cache_index]
        return LayerCache(
            k=self._k[cache_index],
            v=self._v[cache_index],
            block_table=g.table_dev if g is not None else None,
            page_size=self.page_size,
            state=self._state[cache_index],
            writes=writes,
            window=g.window if g is not None else None,
        )

    def kv_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._k + self._v if t is not None)

    # ---- invariants (tests) -----------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or free while mapped."""
        for key, g in self.groups.items():
            mapped = []
            for slot in range(self.max_slots):
                row = g.table[slot]
                if not self._live[slot]:
                    if (row >= 0).any():
                        raise CacheError(f"group {key}: free slot {slot} still maps pages")
                    continue
                mapped += [int(p) for p in row if p >= 0]
                if (row[:g.first_page[slot]] >= 0).any() or (row[g.n_logical[slot]:] >= 0).any():
                    raise CacheError(f"group {key}: slot {slot} maps pages outside its held range")
                if (row[g.first_page[slot]:g.n_logical[slot]] < 0).any():
                    raise CacheError(f"group {key}: slot {slot} has a hole in its held range")
            if len(mapped) != len(set(mapped)):
                raise CacheError(f"group {key}: a page is held twice")
            free = list(g.pool._free)
            if len(free) != len(set(free)):
                raise CacheError(f"group {key}: a page is on the free list twice")
            if set(free) & set(mapped):
                raise CacheError(f"group {key}: a mapped page is on the free list")
            if len(free) + len(mapped) != g.pool.n_pages:
                raise CacheError(f"group {key}: {g.pool.n_pages - len(free) - len(mapped)} pages lost")
