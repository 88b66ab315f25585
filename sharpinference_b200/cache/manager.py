"""The cache manager: paged keys and values with a block table per request, in groups of layers
with equal needs, and slots for per-request state of fixed size.

Reference precedent: ``PagedKvCache`` keeps 16-position pages and a block table, but one pool
per sequence, on the CPU, with nothing given back before the sequence ends
(src/SharpInference.Engine/PagedKvCache.cs:20-83, :103-158, :260-278); its GPU caches are
contiguous per sequence (src/SharpInference.Engine/CudaSequenceKvCache.cs:20-58); per-sequence
state of fixed size exists for another architecture (src/SharpInference.Engine/GdnStateCache.cs).

Here:

* Every schedule entry whose mixer declares a :class:`CacheSpec` writes into a *group*: the
  entries with equal specs.  A group owns one device tensor
  ``[entries, pages, 2 (K|V), kv_heads, page_size, head_dim]`` and one free list of page ids; a
  page id addresses the same page in every entry of the group, so a request has one block table
  per group (``table[logical_block] -> page id``, -1 where nothing is held).
* Pages are taken when a step is about to write positions (``reserve``: all or nothing for the
  whole step), and given back (a) when the request ends (``free_request``), (b) after a step, for
  groups whose mask forgets the past (chunk, window): every page that lies wholly below the
  lowest position a later query can see (``commit``).  A freed page is handed out again at once.
* Every live request holds one *state slot*: an index into per-entry tensors
  ``[slots, *StateSpec.shape]`` for mixers that keep state of fixed size.  The slot is assigned
  (and its state zeroed) at ``add_request`` and returned at ``free_request``, whether or not any
  mixer of the model has state.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..parts.base import CacheSpec, LayerSlot, StateSpec


class OutOfPages(RuntimeError):
    """A group has fewer free pages than a step needs.  Nothing was taken."""

    def __init__(self, group: int, needed: int, free: int):
        super().__init__(f"cache group {group}: {needed} page(s) needed, {free} free")
        self.group, self.needed, self.free = group, needed, free


class OutOfSlots(RuntimeError):
    """Every state slot is held by a live request."""


class CacheError(RuntimeError):
    """A misuse of the manager (unknown request, double free, ...)."""


class FreeList:
    """Ids ``0 .. n-1``; each is either free or held, never both, never twice."""

    def __init__(self, n: int):
        self.capacity = n
        self._free: List[int] = list(range(n - 1, -1, -1))   # pop() hands out low ids first
        self._held = bytearray(n)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.capacity - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError("free list is empty")
        i = self._free.pop()
        self._held[i] = 1
        return i

    def give_back(self, i: int) -> None:
        if not (0 <= i < self.capacity):
            raise CacheError(f"id {i} is outside [0, {self.capacity})")
        if not self._held[i]:
            raise CacheError(f"id {i} is given back twice (or was never taken)")
        self._held[i] = 0
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return bool(self._held[i])


@dataclass
class CacheGroup:
    index: int
    spec: CacheSpec
    entries: List[int]                  # schedule indices that WRITE into this group, in order
    pages: FreeList
    kv: Optional[torch.Tensor] = None   # [len(entries), num_pages, 2, kv_heads, page_size, head_dim]

    def lowest_needed(self, next_pos: int) -> int:
        """The lowest position that a query at ``next_pos`` or later can still read."""
        return self.spec.lowest_visible(next_pos)


@dataclass
class RequestCache:
    request_id: Hashable
    state_slot: int
    length: int = 0                                             # positions committed so far
    tables: Dict[int, List[int]] = field(default_factory=dict)  # group -> page per logical block (-1: none)
    reserved_until: int = 0                                     # positions covered by pages (>= length)
    version: int = 0                                            # changes with every change of the tables; never repeats
    released: Dict[int, int] = field(default_factory=dict)      # group -> blocks below this were given back


class CacheManager:
    def __init__(self, schedule: Sequence, blocks: Sequence, *, page_size: int, num_pages, max_requests: int,
                 dtype: torch.dtype, device="cuda:0", allocate: bool = True):
        """``schedule``/``blocks`` as in :class:`DecoderModel`.  ``num_pages`` is an int (every
        group gets that many) or a dict ``group index -> pages``.  ``allocate=False`` keeps the
        bookkeeping without device tensors (host-only tests)."""
        if page_size <= 0:
            raise ValueError(f"page_size must be positive, found {page_size}")
        if max_requests <= 0:
            raise ValueError(f"max_requests must be positive, found {max_requests}")
        self.page_size = page_size
        self.max_requests = max_requests
        self.dtype = dtype
        self.device = torch.device(device)
        self.groups: List[CacheGroup] = []
        self._entry_group: Dict[int, Tuple[int, int]] = {}      # schedule index -> (group, index within group)
        self._entry_state: Dict[int, torch.Tensor] = {}
        self._entry_state_spec: Dict[int, StateSpec] = {}
        self.requests: Dict[Hashable, RequestCache] = {}
        self.state_slots = FreeList(max_requests)
        self._schedule = list(schedule)
        self._no_pages: Dict[int, int] = {}

        by_spec: Dict[CacheSpec, CacheGroup] = {}
        for index, entry in enumerate(self._schedule):
            mixer = blocks[entry.layer].mixer
            spec = getattr(mixer, "cache_spec", None)
            if spec is not None and entry.cache_from is None:
                group = by_spec.get(spec)
                if group is None:
                    n = num_pages[len(self.groups)] if isinstance(num_pages, dict) else int(num_pages)
                    if n <= 0:
                        raise ValueError(f"cache group {len(self.groups)} needs at least one page, found {n}")
                    group = CacheGroup(len(self.groups), spec, [], FreeList(n))
                    by_spec[spec] = group
                    self.groups.append(group)
                self._entry_group[index] = (group.index, len(group.entries))
                group.entries.append(index)
            sspec = getattr(mixer, "state_spec", None)
            if sspec is not None:
                self._entry_state_spec[index] = sspec
        for index, entry in enumerate(self._schedule):
            if entry.cache_from is not None:
                self._entry_group[index] = self._entry_group[entry.cache_from]
        self._no_pages = dict.fromkeys((g.index for g in self.groups), 0)

        if allocate:
            for g in self.groups:
                s = g.spec
                g.kv = torch.zeros((len(g.entries), g.pages.capacity, 2, s.num_kv_heads, page_size, s.head_dim),
                                   dtype=dtype, device=self.device)
            for index, sspec in self._entry_state_spec.items():
                self._entry_state[index] = torch.zeros((max_requests, *sspec.shape), dtype=sspec.dtype,
                                                       device=self.device)

    # -- what the layers get -------------------------------------------------------------
    def layer_slots(self) -> List[LayerSlot]:
        slots = []
        for index, entry in enumerate(self._schedule):
            slot = LayerSlot(index=index, layer=entry.layer, page_size=self.page_size)
            if index in self._entry_group:
                gi, within = self._entry_group[index]
                slot.group = gi
                slot.kv = self.groups[gi].kv[within] if self.groups[gi].kv is not None else None
                slot.writes_cache = entry.cache_from is None
            slot.state = self._entry_state.get(index)
            slots.append(slot)
        return slots

    # -- requests ------------------------------------------------------------------------
    def add_request(self, request_id: Hashable) -> RequestCache:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already live")
        if self.state_slots.free_count == 0:
            raise OutOfSlots(f"all {self.max_requests} state slots are held")
        slot = self.state_slots.take()
        for state in self._entry_state.values():
            state[slot].zero_()
        rc = RequestCache(request_id, slot, tables={g.index: [] for g in self.groups}, version=self._next_version())
        self.requests[request_id] = rc
        return rc

    def _next_version(self) -> int:
        self._versions = getattr(self, "_versions", 0) + 1
        return self._versions

    def get(self, request_id: Hashable) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def free_request(self, request_id: Hashable) -> None:
        rc = self.requests.pop(request_id, None)
        if rc is None:
            raise CacheError(f"request {request_id!r} is not live (freed twice?)")
        for g in self.groups:
            for page in rc.tables[g.index]:
                if page >= 0:
                    g.pages.give_back(page)
        self.state_slots.give_back(rc.state_slot)

    # -- pages ---------------------------------------------------------------------------
    def pages_needed(self, request_id: Hashable, n_new: int) -> Dict[int, int]:
        """Pages each group must still take so that positions ``[length, length + n_new)`` can be written."""
        rc = self.get(request_id)
        end = rc.length + n_new
        if rc.length % self.page_size and (end - 1) // self.page_size == (rc.length - 1) // self.page_size:
            # everything falls into the block that holds the last committed position, which has its pages
            # (most decode steps: one shared answer, which callers only read)
            return self._no_pages
        need = {}
        blocks_end = (end + self.page_size - 1) // self.page_size
        for g in self.groups:
            table = rc.tables[g.index]
            first = rc.length // self.page_size
            have = sum(1 for b in range(first, min(len(table), blocks_end)) if table[b] >= 0)
            need[g.index] = max(0, blocks_end - first - have)
        return need

    def can_reserve(self, wants: Sequence[Tuple[Hashable, int]]) -> bool:
        total: Dict[int, int] = {g.index: 0 for g in self.groups}
        for request_id, n_new in wants:
            for gi, n in self.pages_needed(request_id, n_new).items():
                total[gi] += n
        return all(total[g.index] <= g.pages.free_count for g in self.groups)

    def reserve(self, wants: Sequence[Tuple[Hashable, int]]) -> None:
        """Take the pages for one step: each ``(request, n_new)`` will write positions
        ``[length, length + n_new)``.  All or nothing: on :class:`OutOfPages` nothing is held."""
        total: Dict[int, int] = {g.index: 0 for g in self.groups}
        for request_id, n_new in wants:
            if n_new <= 0:
                raise CacheError(f"request {request_id!r}: a step must bring at least one token")
            for gi, n in self.pages_needed(request_id, n_new).items():
                total[gi] += n
        for g in self.groups:
            if total[g.index] > g.pages.free_count:
                raise OutOfPages(g.index, total[g.index], g.pages.free_count)
        for request_id, n_new in wants:
            rc = self.get(request_id)
            end = rc.length + n_new
            if rc.length % self.page_size and (end - 1) // self.page_size == (rc.length - 1) // self.page_size:
                rc.reserved_until = max(rc.reserved_until, end)      # the pages are there already
                continue
            blocks_end = (end + self.page_size - 1) // self.page_size
            first = rc.length // self.page_size
            for g in self.groups:
                table = rc.tables[g.index]
                while len(table) < blocks_end:
                    table.append(-1)
                    rc.version = self._next_version()
                for b in range(first, blocks_end):
                    if table[b] < 0:
                        table[b] = g.pages.take()
                        rc.version = self._next_version()
            rc.reserved_until = max(rc.reserved_until, end)

    def commit(self, request_id: Hashable, n_new: int) -> None:
        """The step wrote ``n_new`` positions: advance the length and give back every page that no
        later query can see."""
        rc = self.get(request_id)
        if rc.length + n_new > rc.reserved_until:
            raise CacheError(f"request {request_id!r}: commit of {n_new} positions beyond what was reserved")
        rc.length += n_new
        for g in self.groups:
            if g.spec.kind == "full":
                continue
            lo = g.lowest_needed(rc.length)
            table = rc.tables[g.index]
            upto = min(lo // self.page_size, len(table))
            for b in range(rc.released.get(g.index, 0), upto):       # what lies below was given back before
                if table[b] >= 0:
                    g.pages.give_back(table[b])
                    table[b] = -1
                    rc.version = self._next_version()
            if upto > rc.released.get(g.index, 0):
                rc.released[g.index] = upto

    # -- accounting ----------------------------------------------------------------------
    def free_pages(self) -> Dict[int, int]:
        return {g.index: g.pages.free_count for g in self.groups}

    def held_pages(self, request_id: Hashable) -> Dict[int, int]:
        rc = self.get(request_id)
        return {g.index: sum(1 for p in rc.tables[g.index] if p >= 0) for g in self.groups}

    def max_blocks(self, request_ids: Sequence[Hashable]) -> int:
        return max((len(self.requests[r].tables[g.index]) for r in request_ids for g in self.groups), default=1) or 1

    def check_invariants(self) -> None:
        """No page lost, none held twice: every page of a group is either free or in exactly one table."""
        for g in self.groups:
            seen: Dict[int, Hashable] = {}
            for rid, rc in self.requests.items():
                for page in rc.tables[g.index]:
                    if page < 0:
                        continue
                    if page in seen:
                        raise CacheError(f"group {g.index}: page {page} is held by {seen[page]!r} and {rid!r}")
                    if not g.pages.is_held(page):
                        raise CacheError(f"group {g.index}: page {page} of {rid!r} is on the free list")
                    seen[page] = rid
            if len(seen) != g.pages.held_count:
                raise CacheError(f"group {g.index}: {g.pages.held_count} pages are marked held but "
                                 f"{len(seen)} are in block tables (a page was lost)")
        slots = [rc.state_slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or len(slots) != self.state_slots.held_count:
            raise CacheError("state slots: a slot is held twice or lost")
