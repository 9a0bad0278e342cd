"""The cache manager: pages of keys and values with a block table per request,
and slots of fixed size for per-request state.

Counterpart in arhaamatiq/stride: KvCache (src/kv_cache.cpp:10-92), which has one
kind of page (64 tokens, all layers), a last-in-first-out free list, a slot id per
request and a host block table mirrored on the device. Here:

* Schedule entries of a model whose mixers ask for the same kind of cache
  (`CacheNeed`: heads, head size, window) form a *group*. A group has its own
  arena `[pages, layers of the group, 2, kv_heads, page_size, head_dim]`, its own
  free list and its own block table `[slots, pages per sequence]`; one page id
  covers all layers of its group.
* A request holds one *slot*: a row of every block table and one record of every
  state arena `[slots, ...]`, zeroed when the slot is taken.
* Pages come back when the request releases its slot, and, for a group with a
  window, as soon as every position of the page lies behind the window of all
  tokens still to come (`trim`).

Everything but the arenas is host data, so the bookkeeping runs without a GPU. The books
themselves (free lists, who holds which page, the block tables' content) are kept by the
native pool in `csrc/runtime.cpp`; this module owns the tensors, hands the pool the memory
of the block tables to write into, and turns its return codes into exceptions.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..kernels.build import library

NO_PAGE = -1
_I32P = ctypes.POINTER(ctypes.c_int32)


class CacheError(RuntimeError):
    pass


def _runtime():
    lib = library("runtime")
    if not getattr(lib, "_sb_typed", False):
        lib.sb_pool_create.restype = ctypes.c_void_p
        lib.sb_pool_create.argtypes = [ctypes.c_int, _I32P, ctypes.POINTER(_I32P), ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_int, _I32P, ctypes.POINTER(ctypes.c_uint8), ctypes.c_uint64]
        lib.sb_pool_destroy.argtypes = [ctypes.c_void_p]
        lib.sb_pool_destroy.restype = None
        for name, extra in (("acquire_slot", []), ("release_slot", [ctypes.c_int]), ("pages_needed", [ctypes.c_int, ctypes.c_int, _I32P]),
                            ("free_slots", [_I32P, ctypes.c_int]), ("free_list", [ctypes.c_int, _I32P, ctypes.c_int]),
                            ("ensure", [ctypes.c_int, ctypes.c_int]), ("trim", [ctypes.c_int, ctypes.c_int]),
                            ("take_dirty", [_I32P, ctypes.c_int]), ("held_count", [ctypes.c_int, ctypes.c_int]), ("check", [])):
            fn = getattr(lib, "sb_pool_" + name)
            fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_void_p, *extra]
        lib.sb_pool_free_pages.restype, lib.sb_pool_free_pages.argtypes = None, [ctypes.c_void_p, _I32P]
        lib._sb_typed = True
    return lib


class _Held:
    """`held[slot]` = {page index in the sequence: page id}, read from the block table."""

    def __init__(self, table: np.ndarray):
        self._table = table

    def __getitem__(self, slot: int) -> dict:
        row = self._table[slot]
        return {int(i): int(row[i]) for i in np.flatnonzero(row != NO_PAGE)}


@dataclass
class CacheGroup:
    kv_heads: int
    head_dim: int
    window: int
    dtype: torch.dtype
    page_size: int
    num_pages: int
    entries: list = field(default_factory=list)      # schedule entries served, in order
    arena: Optional[torch.Tensor] = None             # [pages, len(entries), 2, kv_heads, page_size, head_dim]
    table_host: Optional[np.ndarray] = None          # [slots, max_pages] int32, NO_PAGE where nothing is held
    table_pinned: Optional[torch.Tensor] = None      # the tensor behind table_host (pinned when the arena is on a GPU)
    table_device: Optional[torch.Tensor] = None
    manager: Optional["CacheManager"] = None
    index: int = 0

    @property
    def page_bytes(self) -> int:
        return len(self.entries) * 2 * self.kv_heads * self.page_size * self.head_dim * torch.finfo(self.dtype).bits // 8

    def layer_view(self, entry: int) -> torch.Tensor:
        """[pages, 2, kv_heads, page_size, head_dim] of one schedule entry."""
        return self.arena[:, self.entries.index(entry)]

    @property
    def held(self) -> _Held:
        """Per slot: {page index in the sequence: page id}."""
        return _Held(self.table_host)

    @property
    def free(self) -> list:
        """The free list, the next page to be handed out last."""
        buf = np.empty(self.num_pages, dtype=np.int32)
        n = self.manager._lib.sb_pool_free_list(self.manager._pool, self.index, buf.ctypes.data_as(_I32P), buf.size)
        return buf[:n].tolist()


@dataclass
class LayerCache:
    """What a mixer gets for one schedule entry."""
    pages: Optional[torch.Tensor] = None        # [pages, 2, kv_heads, page_size, head_dim]
    block_table: Optional[torch.Tensor] = None  # [slots, max_pages] int32 on the device
    page_size: int = 0
    state: Optional[torch.Tensor] = None        # [slots, *state_shape]
    writes: bool = True                         # False: the entry reads another entry's cache


class CacheManager:
    def __init__(self, needs: list, *, device, max_slots: int, max_context: int, page_size: int = 64,
                 num_pages: Optional[int] = None, cache_bytes: Optional[int] = None, shuffle_seed: int = 0):
        """`needs[i]` is the CacheNeed of schedule entry i, None, or ("shared", j) for an entry that
        reads entry j's cache. `num_pages` is the pool size in pages of every group; alternatively
        `cache_bytes` is divided among the groups in proportion to their bytes per page. A
        `shuffle_seed` other than 0 permutes the free lists, so that tests meet pages in every order."""
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        self.device = torch.device(device)
        self.max_slots = max_slots
        self.max_context = max_context
        self.page_size = page_size
        self.max_pages_per_seq = (max_context + page_size - 1) // page_size
        self.groups: list = []
        self.entry_group: dict = {}     # schedule entry -> (group index) for page needs
        self.entry_shared: dict = {}    # schedule entry -> entry whose cache it reads
        self.states: dict = {}          # schedule entry -> state arena
        # One slot and one page per group beyond those handed out: padding rows of a fixed-size batch
        # (a step recorded as a CUDA graph) write their key and value there.
        self.pad_slot = max_slots
        # Shared with the native pool, which writes them: tokens each slot's pages have been ensured for, and
        # whether the slot is held by a request.
        self.length = np.zeros(max_slots, dtype=np.int32)
        self.live = np.zeros(max_slots, dtype=np.uint8)

        for i, need in enumerate(needs):
            if need is None:
                continue
            if isinstance(need, tuple) and need[0] == "shared":
                self.entry_shared[i] = need[1]
                continue
            if need.kind == "state":
                self.states[i] = torch.zeros((max_slots + 1, *need.state_shape), dtype=need.state_dtype, device=self.device)
                continue
            if need.kind != "pages":
                raise CacheError(f"unknown cache need kind '{need.kind}'")
            dtype = need.dtype
            sig = (need.kv_heads, need.head_dim, need.window, dtype)
            for gi, g in enumerate(self.groups):
                if (g.kv_heads, g.head_dim, g.window, g.dtype) == sig:
                    g.entries.append(i)
                    self.entry_group[i] = gi
                    break
            else:
                self.groups.append(CacheGroup(need.kv_heads, need.head_dim, need.window, dtype, page_size, 0, [i],
                                              manager=self, index=len(self.groups)))
                self.entry_group[i] = len(self.groups) - 1
        for i, j in self.entry_shared.items():
            if j not in self.entry_group and j not in self.states:
                raise CacheError(f"schedule entry {i} reads the cache of entry {j}, which has none")

        if self.groups:
            if num_pages is None:
                if cache_bytes is None:
                    raise CacheError("give num_pages or cache_bytes")
                per_page_all = sum(g.page_bytes for g in self.groups)
                num_pages = int(cache_bytes // per_page_all)
            if num_pages <= 0:
                raise CacheError("the cache pool is smaller than one page")
        for g in self.groups:
            g.num_pages = num_pages
            g.arena = torch.zeros((num_pages + 1, len(g.entries), 2, g.kv_heads, page_size, g.head_dim), dtype=g.dtype, device=self.device)
            pin = self.device.type == "cuda"
            g.table_pinned = torch.full((max_slots + 1, self.max_pages_per_seq), NO_PAGE, dtype=torch.int32, pin_memory=pin)
            g.table_host = g.table_pinned.numpy()        # a view: the pool's edits go straight into the pinned copy
            g.table_host[self.pad_slot, 0] = num_pages
            g.table_device = g.table_pinned.to(self.device)

        self._lib = _runtime()
        n = len(self.groups)
        windows = (ctypes.c_int32 * max(n, 1))(*[g.window for g in self.groups])
        tables = (_I32P * max(n, 1))(*[g.table_host.ctypes.data_as(_I32P) for g in self.groups])
        self._pool = self._lib.sb_pool_create(n, windows, tables, page_size, num_pages or 0, max_slots, self.max_pages_per_seq,
                                              max_context, self.length.ctypes.data_as(_I32P),
                                              self.live.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8)), shuffle_seed)
        if not self._pool:
            raise CacheError(self._lib.sb_last_error().decode())
        self._counts = np.zeros(max(n, 1), dtype=np.int32)
        self._counts_p = self._counts.ctypes.data_as(_I32P)
        self._dirty = np.zeros((max(n, 1) * (max_slots + 1), 2), dtype=np.int32)

    def __del__(self):
        pool, self._pool = getattr(self, "_pool", None), None
        if pool:
            self._lib.sb_pool_destroy(pool)

    # ------------------------------------------------------------------ slots
    def acquire_slot(self) -> int:
        """A free slot id, its state records zeroed; -1 when every slot is taken."""
        slot = self._lib.sb_pool_acquire_slot(self._pool)
        if slot >= 0:
            for arena in self.states.values():
                arena[slot].zero_()
        return slot

    def release_slot(self, slot: int) -> None:
        """Give back the slot and every page it holds."""
        if self._lib.sb_pool_release_slot(self._pool, slot) < 0:
            raise CacheError(f"slot {slot} is released but not held")

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.max_slots and bool(self.live[slot])

    @property
    def live_slots(self) -> set:
        return {int(s) for s in np.flatnonzero(self.live)}

    @property
    def free_slots(self) -> list:
        buf = np.empty(self.max_slots, dtype=np.int32)
        return buf[:self._lib.sb_pool_free_slots(self._pool, buf.ctypes.data_as(_I32P), buf.size)].tolist()

    # ------------------------------------------------------------------ pages
    def pages_needed(self, slot: int, end: int) -> list:
        """Per group, how many new pages the slot needs to hold tokens up to position end-1."""
        if self._lib.sb_pool_pages_needed(self._pool, slot, end, self._counts_p) < 0:
            raise CacheError(f"slot {slot} is not held")
        return self._counts[:len(self.groups)].tolist()

    def free_pages(self) -> list:
        self._lib.sb_pool_free_pages(self._pool, self._counts_p)
        return self._counts[:len(self.groups)].tolist()

    def total_pages(self) -> list:
        return [g.num_pages for g in self.groups]

    def ensure(self, slot: int, end: int) -> bool:
        """Allocate pages so that the slot can hold tokens up to position end-1.
        Returns False, with nothing changed, if a group has too few free pages."""
        r = self._lib.sb_pool_ensure(self._pool, slot, end)
        if r == -1:
            raise CacheError(f"slot {slot} is not held")
        if r == -2:
            raise CacheError(f"sequence of {end} tokens exceeds the context capacity {self.max_context}")
        return r == 1

    def trim(self, slot: int, length: Optional[int] = None) -> int:
        """Give back the pages of windowed groups that no token of the slot at position `length` or later can
        see (`length` defaults to all tokens the slot has pages for). Call it once the steps that processed the
        tokens before `length` have finished on the GPU. Returns pages freed."""
        freed = self._lib.sb_pool_trim(self._pool, slot, -1 if length is None else length)
        if freed < 0:
            raise CacheError(f"slot {slot} is not held")
        return freed

    def sync(self) -> None:
        """Upload the block-table rows that changed since the last call."""
        n = self._lib.sb_pool_take_dirty(self._pool, self._dirty.ctypes.data_as(_I32P), len(self._dirty))
        if n < 0:
            raise CacheError("more block-table rows changed than there are")
        for gi, slot in self._dirty[:n].tolist():
            g = self.groups[gi]
            # From pinned memory and without waiting: a row that changes again before the copy runs only delivers
            # the later content early, which adds pages that no token of an earlier step looks at.
            g.table_device[slot].copy_(g.table_pinned[slot], non_blocking=True)

    # ------------------------------------------------------------------ views
    def layer_cache(self, entry: int) -> LayerCache:
        src = self.entry_shared.get(entry, entry)
        lc = LayerCache(writes=entry not in self.entry_shared)
        if src in self.entry_group:
            g = self.groups[self.entry_group[src]]
            lc.pages, lc.block_table, lc.page_size = g.layer_view(src), g.table_device, g.page_size
        if src in self.states:
            lc.state = self.states[src]
        return lc

    def check(self) -> None:
        """Invariants: every page is free or held by exactly one live slot, never both or twice."""
        if self._lib.sb_pool_check(self._pool) < 0:
            raise CacheError(self._lib.sb_last_error().decode())
