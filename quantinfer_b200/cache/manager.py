"""The cache manager: pages of keys and values with a block table per request,
one pool per group of layers with the same need, and slots of fixed size.

The reference keeps a growable contiguous K and V vector per request and layer
(crates/quantinfer-runtime/src/cache.rs:8-22,94-127) and reserves the whole
capacity at admission (scheduler.rs:120-124). Here the memory is one pool per
group, cut into pages of `page_size` positions:

* a *group* is the set of cache entries whose mixers ask for the same thing
  (same kv heads, head size and window). One page id addresses the same page in
  every entry of the group, so one allocation serves all its layers; the
  group's pools are `[entries, num_pages, kv_heads, page_size, head_dim]`.
* a request has, per group, a *block table*: `table[b]` is the page that holds
  positions `b * page_size ... (b + 1) * page_size - 1`, or -1.
* groups with a window give pages back as soon as every position in them lies
  outside the window of all coming queries; all pages go back when the request
  closes, and a step that fails gives back what it took (`rollback`).
* a *slot* is a request's index into per-request arrays of fixed size: mixer
  state (`StateNeed` entries, `[num_slots, *shape]`, zeroed at `open`) and
  whatever the engine keeps per request (sampler state).
* state of fixed size is overwritten by a step, so a failed step cannot give it
  back the way it gives pages back: `prepare` copies the request's state rows
  aside (device to device, in stream order) and `rollback` copies them back.
  A model without such state pays nothing for this.

The bookkeeping is host-side and needs no device: `device=None` builds the
manager without pools, which is how the scheduler tests drive it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from ..errors import CacheError, OutOfPages
from .needs import PagedKVNeed, StateNeed


class PageAllocator:
    """Free pages of one pool, handed out last-freed-first."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError("a pool needs at least one page")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._held = [False] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free page left")
        p = self._free.pop()
        self._held[p] = True
        return p

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages or not self._held[page]:
            raise CacheError(f"page {page} is freed but not held")
        self._held[page] = False
        self._free.append(page)


@dataclass
class Group:
    need: PagedKVNeed
    entries: list            # cache entry indices, in pool order
    allocator: PageAllocator
    k: Optional[torch.Tensor] = None   # [entries, num_pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor] = None


@dataclass
class RequestCache:
    request_id: object
    slot: int
    length: int = 0                       # positions committed
    pending: int = 0                      # positions prepared but not committed
    tables: list = field(default_factory=list)   # per group: list of page ids or -1


@dataclass
class CacheView:
    """What a layer call sees of the cache: its entry's pages (or state) and
    which block table of the batch to use."""

    entry: int
    group: int = -1
    page_size: int = 0
    k_pages: Optional[torch.Tensor] = None
    v_pages: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None   # [num_slots, *shape] for StateNeed entries
    writes: bool = True


class CacheManager:
    def __init__(self, needs: list, page_size: int, num_pages: int, max_requests: int,
                 max_seq_len: int, dtype=torch.float32, device=None):
        """`needs[i]` is what cache entry i asks for (PagedKVNeed, StateNeed or None).
        `num_pages` is the size of every group's pool; `max_seq_len` bounds a block table."""
        if page_size <= 0 or max_requests <= 0 or max_seq_len <= 0:
            raise CacheError("page_size, max_requests and max_seq_len must be positive")
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_requests = max_requests
        self.max_seq_len = max_seq_len
        self.max_blocks = -(-max_seq_len // page_size)
        self.dtype = dtype
        self.device = torch.device(device) if device is not None else None
        self.needs = list(needs)
        self.groups: list[Group] = []
        self._entry_group: dict[int, tuple] = {}     # entry -> (group index, index in group)
        self.states: dict[int, torch.Tensor] = {}    # entry -> [num_slots, *shape]
        self._state_saved: dict[int, torch.Tensor] = {}   # the rows as they were before the step in flight
        by_need: dict[PagedKVNeed, int] = {}
        for entry, need in enumerate(self.needs):
            if isinstance(need, PagedKVNeed):
                if need not in by_need:
                    by_need[need] = len(self.groups)
                    self.groups.append(Group(need, [], PageAllocator(num_pages)))
                g = by_need[need]
                self._entry_group[entry] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(entry)
            elif isinstance(need, StateNeed):
                if self.device is not None:
                    self.states[entry] = torch.zeros((max_requests, *need.shape), dtype=need.dtype or dtype,
                                                     device=self.device)
                    self._state_saved[entry] = torch.zeros_like(self.states[entry])
            elif need is not None:
                raise CacheError(f"cache entry {entry} asks for {need!r}, which the manager does not know")
        if self.device is not None:
            for g in self.groups:
                shape = (len(g.entries), num_pages, g.need.num_kv_heads, page_size, g.need.head_dim)
                g.k = torch.zeros(shape, dtype=dtype, device=self.device)
                g.v = torch.zeros(shape, dtype=dtype, device=self.device)
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.requests: dict[object, RequestCache] = {}
        # block tables by slot, kept as arrays so that a batch's tables are one gather
        self.host_tables = [np.full((max_requests, self.max_blocks), -1, dtype=np.int32) for _ in self.groups]

    # ---- sizes ---------------------------------------------------------

    def pool_bytes(self) -> int:
        total = 0
        for g in self.groups:
            n = len(g.entries) * self.num_pages * g.need.num_kv_heads * self.page_size * g.need.head_dim
            total += 2 * n * torch.empty((), dtype=self.dtype).element_size()
        return total

    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].allocator.free_pages

    def min_free_pages(self) -> int:
        return min((g.allocator.free_pages for g in self.groups), default=self.num_pages)

    def pages_for(self, length: int) -> int:
        """Pages a request of `length` positions holds at most in any group."""
        return -(-length // self.page_size)

    def live_length(self, group: int, length: int) -> int:
        w = self.groups[group].need.window
        return length if w is None else min(length, w)

    # ---- requests -------------------------------------------------------

    def open(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already open")
        if not self._free_slots:
            raise CacheError(f"all {self.max_requests} request slots are in use")
        slot = self._free_slots.pop()
        rc = RequestCache(request_id, slot, tables=[[] for _ in self.groups])
        self.requests[request_id] = rc
        for st in self.states.values():
            st[slot].zero_()
        return rc

    def get(self, request_id) -> RequestCache:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not open") from None

    def prepare(self, request_id, n_new: int) -> None:
        """Makes sure positions length ... length + n_new - 1 have pages in every
        group. Takes nothing if any group runs out (raises OutOfPages)."""
        rc = self.get(request_id)
        if rc.pending:
            raise CacheError(f"request {request_id!r} has an uncommitted step")
        if n_new <= 0:
            raise CacheError("a step must add at least one position")
        end = rc.length + n_new
        if end > self.max_seq_len:
            raise CacheError(f"request {request_id!r} would reach {end} positions, the limit is {self.max_seq_len}")
        need_blocks = -(-end // self.page_size)
        taken = []
        try:
            for gi, g in enumerate(self.groups):
                table = rc.tables[gi]
                while len(table) < need_blocks:
                    page = g.allocator.alloc()
                    self.host_tables[gi][rc.slot, len(table)] = page
                    table.append(page)
                    taken.append((gi, page))
        except OutOfPages:
            for gi, page in reversed(taken):
                assert rc.tables[gi].pop() == page
                self.host_tables[gi][rc.slot, len(rc.tables[gi])] = -1
                self.groups[gi].allocator.free(page)
            raise OutOfPages(
                f"request {request_id!r} needs {need_blocks} pages per group for {end} positions; "
                f"a pool of {self.num_pages} pages has none left") from None
        for entry, st in self.states.items():
            self._state_saved[entry][rc.slot].copy_(st[rc.slot])
        rc.pending = n_new

    def commit(self, request_id) -> None:
        """The prepared positions are now written. Pages that a window has passed go back."""
        rc = self.get(request_id)
        rc.length += rc.pending
        rc.pending = 0
        for gi, g in enumerate(self.groups):
            w = g.need.window
            if w is None:
                continue
            # the next query sits at position >= rc.length and reads keys > position - w
            first_needed = max(0, rc.length - w + 1)
            table = rc.tables[gi]
            for b in range(min(first_needed // self.page_size, len(table))):
                if table[b] >= 0:
                    g.allocator.free(table[b])
                    table[b] = -1
                    self.host_tables[gi][rc.slot, b] = -1

    def rollback(self, request_id) -> None:
        """Undoes `prepare`: pages beyond the committed length go back, and state of fixed
        size is again what it was before the step."""
        rc = self.get(request_id)
        if rc.pending:
            for entry, st in self.states.items():
                st[rc.slot].copy_(self._state_saved[entry][rc.slot])
        keep = -(-rc.length // self.page_size)
        for gi, g in enumerate(self.groups):
            table = rc.tables[gi]
            while len(table) > keep:
                page = table.pop()
                self.host_tables[gi][rc.slot, len(table)] = -1
                if page >= 0:
                    g.allocator.free(page)
        rc.pending = 0

    def close(self, request_id) -> None:
        rc = self.get(request_id)
        for gi, g in enumerate(self.groups):
            for page in rc.tables[gi]:
                if page >= 0:
                    g.allocator.free(page)
            self.host_tables[gi][rc.slot, :] = -1
        del self.requests[request_id]
        self._free_slots.append(rc.slot)

    # ---- what kernels see -------------------------------------------------

    def table_row(self, request_id, group: int) -> list:
        return self.get(request_id).tables[group]

    def view(self, entry: int, writes: bool = True) -> CacheView:
        need = self.needs[entry]
        if isinstance(need, PagedKVNeed):
            g, idx = self._entry_group[entry]
            grp = self.groups[g]
            return CacheView(entry, g, self.page_size,
                             grp.k[idx] if grp.k is not None else None,
                             grp.v[idx] if grp.v is not None else None, None, writes)
        if isinstance(need, StateNeed):
            return CacheView(entry, state=self.states.get(entry), writes=writes)
        return CacheView(entry, writes=writes)

    # ---- self-check (tests) ---------------------------------------------

    def check_invariants(self) -> None:
        """No page lost, none held twice; every slot either free or owned."""
        for gi, g in enumerate(self.groups):
            held = []
            for rc in self.requests.values():
                held += [p for p in rc.tables[gi] if p >= 0]
            if len(held) != len(set(held)):
                raise CacheError(f"group {gi}: a page is held twice")
            free = g.allocator._free
            if len(free) != len(set(free)):
                raise CacheError(f"group {gi}: a page is on the free list twice")
            if set(held) & set(free):
                raise CacheError(f"group {gi}: a held page is also free")
            if len(held) + len(free) != g.allocator.num_pages:
                raise CacheError(f"group {gi}: {g.allocator.num_pages - len(held) - len(free)} pages are lost")
        for gi in range(len(self.groups)):
            mirror = np.full_like(self.host_tables[gi], -1)
            for rc in self.requests.values():
                mirror[rc.slot, :len(rc.tables[gi])] = rc.tables[gi]
            if not np.array_equal(mirror, self.host_tables[gi]):
                raise CacheError(f"group {gi}: the table arrays differ from the requests' tables")
        slots = [rc.slot for rc in self.requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots):
            raise CacheError("a slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise CacheError("a slot is lost")
