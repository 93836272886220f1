"""The cache manager: paged keys and values with a block table per request, and state slots.

Each entry of a model's run order tells the manager what it needs (:class:`CacheNeed`): pages holding
all keys, pages holding a window of them, a fixed-size state per request, or nothing.  Entries with the
same page geometry and the same policy form a *group*; a group has a pool of pages of its own, one page
id addresses the keys and values of all the group's entries (the reference's "one block, all layers"
layout, src/kv_cache.h:1-14), and every live request has one block table per group.  Pages go back to
the pool when a request is released and, in a window group, as soon as the window has passed them
(the reference keeps window layers in a second, ring-shaped cache: src/inference.cpp:1594-1609,
1650-1665).  Beside the pages there are ``max_requests`` state slots (the reference's per-sequence
``RecurrentState``, src/qwen_model.cpp:319-391, 620-634), zeroed when a request is admitted.

A page of a group is laid out ``[entry][K|V][kv_head][token in page][head_dim]``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from .pages import OutOfPages, OutOfSlots, PageAllocator, SlotAllocator


@dataclass(frozen=True)
class CacheNeed:
    """What one entry of the run order wants from the cache manager."""

    kind: str = "none"                    # "none" | "pages" | "state"
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None          # pages: None keeps all keys, W keeps the last W positions
    state_shape: Tuple[int, ...] = ()     # state: shape of one request's state
    state_dtype: str = "float32"

    @staticmethod
    def pages(kv_heads: int, head_dim: int, window: Optional[int] = None) -> "CacheNeed":
        if window is not None and window < 1:
            raise ValueError("a window must hold at least one position")
        return CacheNeed("pages", kv_heads, head_dim, window)

    @staticmethod
    def state(shape: Sequence[int], dtype: str = "float32") -> "CacheNeed":
        return CacheNeed("state", state_shape=tuple(shape), state_dtype=dtype)


@dataclass
class PageGroup:
    index: int
    kv_heads: int
    head_dim: int
    window: Optional[int]
    entries: List[int]                    # run-order entries whose keys and values live in this group
    allocator: PageAllocator
    pool: object = None                   # device tensor [pages, entries, 2, kv_heads, page_size, head_dim]

    def entry_slot(self, entry: int) -> int:
        return self.entries.index(entry)


@dataclass
class RequestCache:
    request_id: object
    length: int = 0                                          # tokens whose keys are in the cache
    tables: List[List[int]] = field(default_factory=list)    # per group: page of each logical block, -1 once freed
    first_live: List[int] = field(default_factory=list)      # per group: first logical block still held
    slot: int = -1


class CacheManager:
    def __init__(self, needs: Sequence[CacheNeed], page_size: int, num_pages, max_requests: int):
        """``needs[i]`` is the need of run-order entry i (an entry that borrows another entry's cache has
        kind "none").  ``num_pages`` is one number for every group or a list with one number per group, in
        the order in which groups first appear."""
        if page_size < 1:
            raise ValueError("page_size must be >= 1")
        self.page_size = page_size
        self.max_requests = max_requests
        self.needs = list(needs)
        self.groups: List[PageGroup] = []
        self.entry_group: Dict[int, int] = {}
        keys: Dict[Tuple, int] = {}
        for i, need in enumerate(self.needs):
            if need.kind != "pages":
                continue
            key = (need.kv_heads, need.head_dim, need.window)
            if key not in keys:
                keys[key] = len(self.groups)
                self.groups.append(PageGroup(len(self.groups), need.kv_heads, need.head_dim, need.window, [], None))
            g = self.groups[keys[key]]
            g.entries.append(i)
            self.entry_group[i] = g.index
        counts = list(num_pages) if isinstance(num_pages, (list, tuple)) else [num_pages] * len(self.groups)
        if len(counts) != len(self.groups):
            raise ValueError(f"{len(counts)} page counts for {len(self.groups)} groups")
        for g, n in zip(self.groups, counts):
            g.allocator = PageAllocator(n)
        self.state_entries = [i for i, need in enumerate(self.needs) if need.kind == "state"]
        self.slots = SlotAllocator(max_requests)
        self.state: Dict[int, object] = {}        # entry -> device tensor [max_requests, *state_shape]
        self.requests: Dict[object, RequestCache] = {}
        self.device = None
        self.poison = False

    # ---- device memory ---------------------------------------------------------------------------
    def materialize(self, device, dtype, poison: bool = False) -> None:
        """Allocate the pools and the state on ``device``.  ``poison`` fills pages with NaN at the start
        and whenever they are freed, so that a kernel that reads a position it must not see shows."""
        import torch
        self.device, self.poison = device, poison
        for g in self.groups:
            shape = (g.allocator.num_pages, len(g.entries), 2, g.kv_heads, self.page_size, g.head_dim)
            g.pool = (torch.full(shape, float("nan"), dtype=dtype, device=device) if poison
                      else torch.zeros(shape, dtype=dtype, device=device))
        for e in self.state_entries:
            need = self.needs[e]
            self.state[e] = torch.zeros((self.max_requests,) + need.state_shape,
                                        dtype=getattr(torch, need.state_dtype), device=device)

    def pool_bytes(self) -> int:
        return sum(g.pool.numel() * g.pool.element_size() for g in self.groups if g.pool is not None)

    # ---- requests --------------------------------------------------------------------------------
    def add_request(self, request_id) -> RequestCache:
        if request_id in self.requests:
            raise ValueError(f"request {request_id!r} is already live")
        slot = self.slots.alloc()                      # raises OutOfSlots
        rc = RequestCache(request_id, 0, [[] for _ in self.groups], [0] * len(self.groups), slot)
        self.requests[request_id] = rc
        for t in self.state.values():
            t[slot].zero_()
        return rc

    def has_request(self, request_id) -> bool:
        return request_id in self.requests

    def length(self, request_id) -> int:
        return self.requests[request_id].length

    def _first_needed_block(self, g: PageGroup, start: int) -> int:
        """First logical block that a query at position ``start`` (or later) can still see."""
        if g.window is None:
            return 0
        return max(0, start - g.window + 1) // self.page_size

    def pages_needed(self, request_id, n_new: int) -> List[int]:
        """Pages that :meth:`reserve` would take from each group for ``n_new`` more tokens."""
        rc = self.requests[request_id]
        blocks = -(-(rc.length + n_new) // self.page_size)
        return [max(0, blocks - len(rc.tables[g.index])) for g in self.groups]

    def pages_for_new_request(self, n_tokens: int) -> List[int]:
        blocks = -(-n_tokens // self.page_size)
        return [blocks for _ in self.groups]

    def free_pages(self) -> List[int]:
        return [g.allocator.num_free for g in self.groups]

    def can_reserve(self, request_id, n_new: int) -> bool:
        return all(n <= g.allocator.num_free for n, g in zip(self.pages_needed(request_id, n_new), self.groups))

    def reserve(self, request_id, n_new: int) -> None:
        """Give the request pages for positions ``[length, length + n_new)`` in every group, or raise
        :class:`OutOfPages` and take nothing."""
        rc = self.requests[request_id]
        need = self.pages_needed(request_id, n_new)
        for n, g in zip(need, self.groups):
            if n > g.allocator.num_free:
                raise OutOfPages(f"request {request_id!r}: group {g.index} needs {n} pages for {n_new} more tokens, "
                                 f"{g.allocator.num_free} of {g.allocator.num_pages} free")
        for n, g in zip(need, self.groups):
            rc.tables[g.index].extend(g.allocator.alloc(n))

    def unreserve(self, request_id) -> None:
        """Give back the pages reserved beyond the request's length (a step that did not run)."""
        rc = self.requests[request_id]
        blocks = -(-rc.length // self.page_size)
        for g in self.groups:
            table = rc.tables[g.index]
            self._free(g, [p for p in table[blocks:] if p >= 0])
            del table[blocks:]

    def advance(self, request_id, n_new: int) -> None:
        """The request's ``n_new`` tokens are in the cache now.  Window groups give back the pages that no
        later position can see."""
        rc = self.requests[request_id]
        rc.length += n_new
        if rc.length > len(rc.tables[0]) * self.page_size if self.groups else False:
            raise RuntimeError(f"request {request_id!r} advanced past its reserved pages")
        for g in self.groups:
            if g.window is None:
                continue
            keep_from = self._first_needed_block(g, rc.length)
            table = rc.tables[g.index]
            passed = [table[b] for b in range(rc.first_live[g.index], min(keep_from, len(table)))]
            if passed:
                self._free(g, passed)
                for b in range(rc.first_live[g.index], min(keep_from, len(table))):
                    table[b] = -1
            rc.first_live[g.index] = max(rc.first_live[g.index], min(keep_from, len(table)))

    def truncate(self, request_id, length: int) -> None:
        """Forget everything from position ``length`` on (pages wholly past it are given back).  Only a
        request without window groups or state can go back."""
        rc = self.requests[request_id]
        if length > rc.length:
            raise ValueError("truncate cannot lengthen a request")
        if any(g.window is not None for g in self.groups) or self.state_entries:
            if length != rc.length:
                raise ValueError("a request with windowed pages or state cannot be rewound")
        blocks = -(-length // self.page_size)
        for g in self.groups:
            table = rc.tables[g.index]
            self._free(g, table[blocks:])
            del table[blocks:]
        rc.length = length

    def release(self, request_id) -> None:
        rc = self.requests.pop(request_id)
        for g in self.groups:
            self._free(g, [p for p in rc.tables[g.index] if p >= 0])
        self.slots.free(rc.slot)

    def _free(self, g: PageGroup, pages: List[int]) -> None:
        released = g.allocator.free(pages)
        if self.poison and g.pool is not None and released:
            import torch
            g.pool[torch.tensor(released, device=g.pool.device)] = float("nan")

    # ---- what a step needs -----------------------------------------------------------------------
    def block_table(self, request_id, group: int) -> List[int]:
        return self.requests[request_id].tables[group]

    def slot_of(self, request_id) -> int:
        return self.requests[request_id].slot

    def token_slots(self, request_id, group: int, start: int, n: int) -> List[int]:
        """Physical token slots (page * page_size + offset) of positions ``[start, start + n)``."""
        table = self.requests[request_id].tables[group]
        ps = self.page_size
        if n >= 64:
            # a long portion: page by page instead of token by token
            out = []
            p = start
            while p < start + n:
                page = table[p // ps]
                if page < 0:
                    raise RuntimeError(f"request {request_id!r}: position {p} lies in a page that was given back")
                stop = min(start + n, (p // ps + 1) * ps)
                out.extend(range(page * ps + p % ps, page * ps + p % ps + (stop - p)))
                p = stop
            return out
        out = []
        for p in range(start, start + n):
            page = table[p // ps]
            if page < 0:
                raise RuntimeError(f"request {request_id!r}: position {p} lies in a page that was given back")
            out.append(page * ps + p % ps)
        return out

    def check(self) -> None:
        """Raise AssertionError unless no page is lost, held twice or free while held."""
        for g in self.groups:
            g.allocator.check()
            held: Dict[int, int] = {}
            for rc in self.requests.values():
                for p in rc.tables[g.index]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            for p in range(g.allocator.num_pages):
                assert g.allocator.refcount(p) == held.get(p, 0), \
                    f"group {g.index} page {p}: refcount {g.allocator.refcount(p)}, held by {held.get(p, 0)} tables"
        self.slots.check()
        slots = [rc.slot for rc in self.requests.values()]
        assert len(slots) == len(set(slots)), "two requests share a state slot"
        assert self.slots.num_free == self.max_requests - len(slots), "a state slot is lost"
