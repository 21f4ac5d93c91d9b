"""The cache manager: pages of keys and values with a block table per request,
groups of layers with different needs, and slots for per-request state of fixed size.

* A **page** holds ``page_size`` consecutive positions of one request for one layer.
  What a position stores is the mixer's own affair: it names its tensors and the
  shape of one position's entry (``cache.specs.PagedSpec``; keys and values, each
  [n_pages, n_kv_heads, page_size, head_dim], are the built-in case).  A page *id*
  is valid in every layer of its **group**: the layers of a group share one id
  space, one free list and one block table per request, whatever they store.
* **Groups** are formed by what the layers need: all earlier keys (window None) or
  the last W positions.  A windowed group gives pages back as soon as every
  position in them has fallen out of the window of the request's next query; the
  group of full layers keeps them until the request ends.
* A request holds a **slot**: the row of its block tables and the index of its
  state in every :class:`StateSpec` tensor ([max_slots, *shape], zeroed at
  admission).  Freed pages and slots are used again, most recently freed first.
* The bookkeeping (free lists, tables, held ranges, window release, invariants) is
  native code (``csrc/host/cache_core.cpp``); this module owns the device tensors and
  the copies of changed table rows to the device.
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

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .specs import CacheSpec


class CacheError(RuntimeError):
    pass


@dataclass
class LayerCache:
    """What a mixer sees of the cache while one schedule entry runs."""

    pages: Dict[str, torch.Tensor]  # the mixer's paged tensors by the names of its PagedSpec
    block_table: Optional[torch.Tensor]  # device int32 [max_slots, table_width]; -1 = no page
    page_size: int
    state: Optional[torch.Tensor]  # [max_slots, *shape]
    writes: bool = True
    window: Optional[int] = None

    @property
    def k(self) -> Optional[torch.Tensor]:
        return self.pages.get("k")

    @property
    def v(self) -> Optional[torch.Tensor]:
        return self.pages.get("v")


_CHECKS = {
    1: "a page is mapped outside a live request's held range", 2: "a hole in a request's held range",
    3: "a page is held twice", 4: "a mapped page is not marked held", 5: "a page is on the free list twice",
    6: "a mapped page is on the free list", 7: "a page is lost",
}


class _PoolView:
    """Numbers of one group's page pool (the pool itself lives in the native library)."""

    def __init__(self, mgr, index, n_pages):
        self._mgr, self._index, self.n_pages = mgr, index, n_pages

    @property
    def n_free(self) -> int:
        return self._mgr._lib.fxh_free_pages(self._mgr._h, self._index)

    def held(self) -> int:
        return self.n_pages - self.n_free


class _Group:
    def __init__(self, mgr, index, window, n_pages, max_slots, width, device):
        self.index = index
        self.window = window
        self.caches: List[int] = []
        self.pool = _PoolView(mgr, index, n_pages)
        self.table_dev = torch.full((max_slots, width), -1, dtype=torch.int32, device=device)
        self.table: np.ndarray = None  # view of the native table, set once the native object exists


class _SeqLens:
    def __init__(self, mgr):
        self._mgr = mgr

    def __getitem__(self, slot: int) -> int:
        return self._mgr._lib.fxh_seq_len(self._mgr._h, int(slot))


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
        from ..kernels import hostlib

        if page_size <= 0:
            raise CacheError("page_size must be positive")
        self._lib = hostlib.load()
        self.page_size = int(page_size)
        self.max_slots = int(max_slots)
        self.max_positions = int(max_positions)
        self.device = torch.device(device)
        self.dtype = dtype
        self.table_width = (self.max_positions + self.page_size - 1) // self.page_size
        self.groups: Dict[object, _Group] = {}
        self._group_of: List[Optional[_Group]] = []
        self._pages: List[Dict[str, torch.Tensor]] = []
        self._state: List[Optional[torch.Tensor]] = []
        for idx, cs in enumerate(cache_specs):
            g = None
            st = None
            pages: Dict[str, torch.Tensor] = {}
            if cs is not None and cs.paged is not None:
                key = cs.paged.window
                if key not in self.groups:
                    n = n_pages[key] if isinstance(n_pages, dict) else int(n_pages)
                    self.groups[key] = _Group(self, len(self.groups), key, n, self.max_slots, self.table_width, self.device)
                g = self.groups[key]
                g.caches.append(idx)
                for ts in cs.paged.tensors:
                    if ts.name in pages:
                        raise CacheError(f"cache {idx}: two paged tensors are named {ts.name!r}")
                    pages[ts.name] = torch.zeros((g.pool.n_pages, *ts.page_shape(self.page_size)),
                                                 dtype=ts.dtype or dtype, device=self.device)
            if cs is not None and cs.state is not None:
                st = torch.zeros((self.max_slots, *cs.state.shape), dtype=cs.state.dtype, device=self.device)
            self._group_of.append(g)
            self._pages.append(pages)
            self._state.append(st)
        order = sorted(self.groups.values(), key=lambda g: g.index)
        windows = (ctypes.c_int * max(1, len(order)))(*[-1 if g.window is None else int(g.window) for g in order])
        pages = (ctypes.c_int * max(1, len(order)))(*[g.pool.n_pages for g in order])
        self._h = self._lib.fxh_cache_create(len(order), windows, pages, self.page_size, self.max_slots, self.table_width,
                                            self.max_positions)
        if not self._h:
            raise CacheError("the native cache object could not be made")
        for g in order:
            g.table = np.ctypeslib.as_array(self._lib.fxh_table(self._h, g.index), shape=(self.max_slots, self.table_width))
        self._order = order
        self._need = (ctypes.c_int * max(1, len(order)))()
        self._dirty = (ctypes.c_int * self.max_slots)()
        self.seq_len = _SeqLens(self)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            for g in getattr(self, "_order", []):
                g.table = None
            self._lib.fxh_cache_destroy(h)

    # ---- requests -------------------------------------------------------------
    @property
    def n_free_slots(self) -> int:
        return self._lib.fxh_free_slots(self._h)

    def open_request(self) -> Optional[int]:
        """A slot for a new request (its state zeroed), or None when all are taken."""
        slot = self._lib.fxh_open(self._h)
        if slot < 0:
            return None
        for st in self._state:
            if st is not None:
                st[slot].zero_()
        return slot

    def close_request(self, slot: int) -> None:
        """Give back everything the request holds."""
        self._ok(self._lib.fxh_close(self._h, int(slot)), slot)

    def _ok(self, rc: int, slot=None) -> int:
        if rc >= 0:
            return rc
        if rc == -1:
            raise CacheError(f"slot {slot} is not held by a request")
        if rc == -2:
            raise CacheError(f"length exceeds max_positions {self.max_positions}")
        if rc == -3:
            raise CacheError("a request's length cannot shrink")
        raise CacheError("the page bookkeeping is corrupt (a page freed but not held)")

    # ---- pages ----------------------------------------------------------------
    def pages_needed(self, slot: int, new_len: int) -> Dict[object, int]:
        """Pages each group still has to get so that positions < new_len are mapped."""
        self._ok(self._lib.fxh_pages_needed(self._h, int(slot), int(new_len), self._need), slot)
        return {g.window: self._need[g.index] for g in self._order}

    def free_pages(self) -> Dict[object, int]:
        return {key: g.pool.n_free for key, g in self.groups.items()}

    def can_reserve(self, wanted: Dict[object, int]) -> bool:
        return all(self.groups[key].pool.n_free >= n for key, n in wanted.items())

    def reserve(self, slot: int, new_len: int) -> bool:
        """Map pages for every position < new_len in every group, or change nothing."""
        return self._ok(self._lib.fxh_reserve(self._h, int(slot), int(new_len)), slot) == 0

    def commit(self, slot: int, new_len: int) -> None:
        """The request now holds ``new_len`` positions.  Windowed groups give back the
        pages that no later query can read: the next query, at position new_len,
        reads from new_len - W + 1 on."""
        self._ok(self._lib.fxh_commit(self._h, int(slot), int(new_len)), slot)

    def reserve_step(self, slots: Sequence[int], counts: Sequence[int]) -> Optional[List[int]]:
        """A whole step in one call: request ``slots[i]`` is to grow by ``counts[i]`` positions.  Pages are mapped for
        every request or for none.  Returns the requests' lengths before the step, or None when the pages do not
        suffice (nothing has been changed)."""
        n = len(slots)
        arr = (ctypes.c_int * (3 * n))(*slots, *counts)
        ip = ctypes.cast(arr, ctypes.POINTER(ctypes.c_int))
        rc = self._lib.fxh_reserve_step(self._h, n, ip, ctypes.cast(ctypes.addressof(arr) + 4 * n, type(ip)),
                                        ctypes.cast(ctypes.addressof(arr) + 8 * n, type(ip)))
        if rc == 1:
            return None
        self._ok(rc, list(slots))
        return list(arr[2 * n:3 * n])

    def commit_step(self, slots: Sequence[int], counts: Sequence[int]) -> None:
        """The step has run: every request holds ``counts[i]`` positions more."""
        n = len(slots)
        arr = (ctypes.c_int * (2 * n))(*slots, *counts)
        ip = ctypes.cast(arr, ctypes.POINTER(ctypes.c_int))
        self._ok(self._lib.fxh_commit_step(self._h, n, ip, ctypes.cast(ctypes.addressof(arr) + 4 * n, type(ip))),
                 list(slots))

    def held_pages(self, slot: int) -> Dict[object, List[int]]:
        out = {}
        for g in self._order:
            a, b = self._lib.fxh_first_page(self._h, g.index, slot), self._lib.fxh_n_logical(self._h, g.index, slot)
            out[g.window] = [int(p) for p in g.table[slot, a:b]]
        return out

    @property
    def peak_pages(self) -> Dict[object, int]:
        return {g.window: self._lib.fxh_peak_pages(self._h, g.index) for g in self._order}

    # ---- device side ----------------------------------------------------------
    def sync_tables(self) -> None:
        """Bring the device copies of the changed block-table rows up to date."""
        for g in self._order:
            n = self._lib.fxh_take_dirty(self._h, g.index, self._dirty, self.max_slots)
            if n == 0:
                continue
            rows = [self._dirty[i] for i in range(n)]
            if n == 1:
                r = rows[0]
                g.table_dev[r].copy_(torch.from_numpy(g.table[r].copy()), non_blocking=False)
            else:
                idx = torch.tensor(rows, dtype=torch.long)
                g.table_dev[idx.to(self.device)] = torch.from_numpy(g.table[rows]).to(self.device)

    def layer_cache(self, cache_index: int, writes: bool = True) -> LayerCache:
        g = self._group_of[cache_index]
        return LayerCache(
            pages=self._pages[cache_index],
            block_table=g.table_dev if g is not None else None,
            page_size=self.page_size,
            state=self._state[cache_index],
            writes=writes,
            window=g.window if g is not None else None,
        )

    def kv_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for pages in self._pages for t in pages.values())

    # ---- invariants (tests) -----------------------------------------------------
    def check_invariants(self) -> None:
        """No page lost, held twice or free while mapped."""
        rc = self._lib.fxh_check(self._h)
        if rc:
            raise CacheError(f"cache invariants broken: {_CHECKS.get(rc, rc)}")
