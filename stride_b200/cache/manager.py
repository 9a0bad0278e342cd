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

Everything but the arenas is host data, so the bookkeeping runs without a GPU.
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

NO_PAGE = -1


class CacheError(RuntimeError):
    pass


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
    free: list = field(default_factory=list)
    held: list = field(default_factory=list)         # per slot: {page index in the sequence: page id}

    @property
    def page_bytes(self) -> int:
        return len(self.entries) * 2 * self.kv_heads * self.page_size * self.head_dim * torch.finfo(self.dtype).bits // 8

    def layer_view(self, entry: int) -> torch.Tensor:
        """[pages, 2, kv_heads, page_size, head_dim] of one schedule entry."""
        return self.arena[:, self.entries.index(entry)]


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
        `cache_bytes` is divided among the groups in proportion to their bytes per page."""
        if page_size <= 0:
            raise CacheError("page_size must be positive")
        self.device = torch.device(device)
        self.max_slots = max_slots
        self.max_context = max_context
        self.page_size = page_size
        self.max_pages_per_seq = (max_context + page_size - 1) // page_size
        self._rng = random.Random(shuffle_seed) if shuffle_seed else None
        self.groups: list = []
        self.entry_group: dict = {}     # schedule entry -> (group index) for page needs
        self.entry_shared: dict = {}    # schedule entry -> entry whose cache it reads
        self.states: dict = {}          # schedule entry -> state arena
        self._dirty: set = set()        # (group, slot) rows to upload
        # One slot and one page per group beyond those handed out: padding rows of a fixed-size batch
        # (a step recorded as a CUDA graph) write their key and value there.
        self.pad_slot = max_slots
        self.free_slots = list(range(max_slots - 1, -1, -1))
        self.live_slots: set = set()
        self.length = [0] * max_slots   # tokens the slot's pages have been ensured for

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
                self.groups.append(CacheGroup(need.kv_heads, need.head_dim, need.window, dtype, page_size, 0, [i]))
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
            g.table_host = g.table_pinned.numpy()        # a view: host edits go straight into the pinned copy
            g.table_host[self.pad_slot, 0] = num_pages
            g.table_device = g.table_pinned.to(self.device)
            g.free = list(range(num_pages - 1, -1, -1))     # page 0 is handed out first
            if self._rng:
                self._rng.shuffle(g.free)
            g.held = [dict() for _ in range(max_slots)]

    # ------------------------------------------------------------------ slots
    def acquire_slot(self) -> int:
        """A free slot id, its state records zeroed; -1 when every slot is taken."""
        if not self.free_slots:
            return -1
        slot = self.free_slots.pop()
        self.live_slots.add(slot)
        self.length[slot] = 0
        for arena in self.states.values():
            arena[slot].zero_()
        return slot

    def release_slot(self, slot: int) -> None:
        """Give back the slot and every page it holds."""
        if slot not in self.live_slots:
            raise CacheError(f"slot {slot} is released but not held")
        for gi, g in enumerate(self.groups):
            if g.held[slot]:
                for index, page in g.held[slot].items():
                    g.free.append(page)
                    g.table_host[slot, index] = NO_PAGE
                g.held[slot].clear()
                self._dirty.add((gi, slot))
                if self._rng:
                    self._rng.shuffle(g.free)
        self.live_slots.discard(slot)
        self.length[slot] = 0
        self.free_slots.append(slot)

    # ------------------------------------------------------------------ pages
    def _wanted(self, g: CacheGroup, slot: int, start: int, end: int) -> list:
        """Page indices that tokens start..end-1 write or read and the slot does not hold."""
        if end <= start:
            return []
        # Pages before the one `start` falls in were allocated by earlier steps (and maybe trimmed since).
        held = g.held[slot]
        return [i for i in range(start // g.page_size, (end - 1) // g.page_size + 1) if i not in held]

    def pages_needed(self, slot: int, end: int) -> list:
        """Per group, how many new pages the slot needs to hold tokens up to position end-1."""
        return [len(self._wanted(g, slot, self.length[slot], end)) for g in self.groups]

    def free_pages(self) -> list:
        return [len(g.free) for g in self.groups]

    def total_pages(self) -> list:
        return [g.num_pages for g in self.groups]

    def ensure(self, slot: int, end: int) -> bool:
        """Allocate pages so that the slot can hold tokens up to position end-1.
        Returns False, with nothing changed, if a group has too few free pages."""
        if slot not in self.live_slots:
            raise CacheError(f"slot {slot} is not held")
        if end > self.max_context:
            raise CacheError(f"sequence of {end} tokens exceeds the context capacity {self.max_context}")
        wanted = [self._wanted(g, slot, self.length[slot], end) for g in self.groups]
        if any(len(w) > len(g.free) for w, g in zip(wanted, self.groups)):
            return False
        for gi, (w, g) in enumerate(zip(wanted, self.groups)):
            for index in w:
                page = g.free.pop()
                g.held[slot][index] = page
                g.table_host[slot, index] = page
            if w:
                self._dirty.add((gi, slot))
        self.length[slot] = max(self.length[slot], end)
        return True

    def trim(self, slot: int, length: Optional[int] = None) -> int:
        """Give back the pages of windowed groups that no token of the slot at position `length` or later can
        see (`length` defaults to all tokens the slot has pages for). Call it once the steps that processed the
        tokens before `length` have finished on the GPU. Returns pages freed."""
        freed = 0
        n = self.length[slot] if length is None else min(length, self.length[slot])
        for gi, g in enumerate(self.groups):
            if g.window <= 0:
                continue
            first_needed = n - g.window + 1      # the oldest key the next token (position n) reads
            for index in [i for i in g.held[slot] if (i + 1) * g.page_size <= first_needed]:
                g.free.append(g.held[slot].pop(index))
                g.table_host[slot, index] = NO_PAGE
                self._dirty.add((gi, slot))
                freed += 1
            if freed and self._rng:
                self._rng.shuffle(g.free)
        return freed

    def sync(self) -> None:
        """Upload the block-table rows that changed since the last call."""
        for gi, slot in sorted(self._dirty):
            g = self.groups[gi]
            # From pinned memory and without waiting: a row that changes again before the copy runs only delivers
            # the later content early, which adds pages that no token of an earlier step looks at.
            g.table_device[slot].copy_(g.table_pinned[slot], non_blocking=True)
        self._dirty.clear()

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
        for g in self.groups:
            seen = {}
            for p in g.free:
                if p in seen:
                    raise CacheError(f"page {p} is on the free list twice")
                seen[p] = "free"
            if g.table_host[self.pad_slot, 0] != g.num_pages:
                raise CacheError("the padding slot lost its page")
            for slot, held in enumerate(g.held):
                if held and slot not in self.live_slots:
                    raise CacheError(f"slot {slot} holds pages but is not live")
                for index, p in held.items():
                    if p in seen:
                        raise CacheError(f"page {p} is held by slot {slot} and is also {seen[p]}")
                    seen[p] = f"held by slot {slot}"
                    if g.table_host[slot, index] != p:
                        raise CacheError(f"block table of slot {slot} disagrees at index {index}")
            if len(seen) != g.num_pages:
                raise CacheError(f"{g.num_pages - len(seen)} pages are lost")
        if len(set(self.free_slots)) != len(self.free_slots) or set(self.free_slots) & self.live_slots:
            raise CacheError("slot bookkeeping is inconsistent")
        if len(self.free_slots) + len(self.live_slots) != self.max_slots:
            raise CacheError("a slot is lost")
