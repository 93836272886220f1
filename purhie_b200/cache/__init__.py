"""The cache manager's bookkeeping as Python sees it (``cache/cache.cpp``): pages with a free list and reference
counts, groups of run-order entries with pools of their own, a block table per request and group, state slots.
These classes drive the host library's own objects through its test entry points; no device is involved.
Request ids may be any hashable value.
"""
from __future__ import annotations

import json
from ctypes import c_char_p, c_int, c_longlong, c_void_p
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

from .. import native
from ..native import CheckError, OutOfPages, OutOfSlots

_DECLARED = False


def _lib():
    global _DECLARED
    L = native.lib()
    if not _DECLARED:
        P = c_void_p
        for name, res, args in [
            ("qe_pages_create", P, [c_int]), ("qe_pages_free_handle", None, [P]), ("qe_pages_alloc", c_char_p, [P, c_int]),
            ("qe_pages_release", c_char_p, [P, c_char_p]), ("qe_pages_share", c_int, [P, c_int]),
            ("qe_pages_num_free", c_int, [P]), ("qe_pages_check", c_int, [P]),
            ("qe_slots_create", P, [c_int]), ("qe_slots_free_handle", None, [P]), ("qe_slots_alloc", c_int, [P]),
            ("qe_slots_release", c_int, [P, c_int]), ("qe_slots_check", c_int, [P]),
            ("qe_cache_create", P, [c_char_p, c_int, c_char_p, c_int]), ("qe_cache_free_handle", None, [P]),
            ("qe_cache_add_request", c_int, [P, c_longlong]), ("qe_cache_release", c_int, [P, c_longlong]),
            ("qe_cache_reserve", c_int, [P, c_longlong, c_int]), ("qe_cache_unreserve", c_int, [P, c_longlong]),
            ("qe_cache_advance", c_int, [P, c_longlong, c_int]), ("qe_cache_truncate", c_int, [P, c_longlong, c_int]),
            ("qe_cache_length", c_int, [P, c_longlong]), ("qe_cache_can_reserve", c_int, [P, c_longlong, c_int]),
            ("qe_cache_check", c_int, [P]), ("qe_cache_info", c_char_p, [P]),
            ("qe_cache_pages_needed", c_char_p, [P, c_longlong, c_int]),
            ("qe_cache_token_slots", c_char_p, [P, c_longlong, c_int, c_int, c_int]),
        ]:
            native.declare(name, res, args)
        _DECLARED = True
    return L


@dataclass(frozen=True)
class CacheNeed:
    """What one entry of the run order wants from the cache manager."""

    kind: str = "none"                    # "none" | "pages" | "state"
    kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None          # pages: None keeps all keys, W keeps the last W positions
    state_shape: Tuple[int, ...] = ()
    value_dim: int = 0                    # pages: width of a value row where it differs from a key row's (0: head_dim)

    @staticmethod
    def pages(kv_heads: int, head_dim: int, window: Optional[int] = None, value_dim: int = 0) -> "CacheNeed":
        if window is not None and window < 1:
            raise ValueError("a window must hold at least one position")
        return CacheNeed("pages", kv_heads, head_dim, window, value_dim=0 if value_dim == head_dim else value_dim)

    @staticmethod
    def state(shape: Sequence[int]) -> "CacheNeed":
        return CacheNeed("state", state_shape=tuple(shape))

    def to_json(self) -> dict:
        if self.kind == "pages":
            return {"kind": "pages", "kv_heads": self.kv_heads, "head_dim": self.head_dim, "window": self.window or 0,
                    "value_dim": self.value_dim}
        if self.kind == "state":
            return {"kind": "state", "shape": list(self.state_shape)}
        return {"kind": "none"}


class PageAllocator:
    def __init__(self, num_pages: int):
        self._h = _lib().qe_pages_create(num_pages)
        if not self._h:
            raise native.last_error()
        self.num_pages = num_pages

    def __del__(self):
        try:
            _lib().qe_pages_free_handle(self._h)
        except Exception:
            pass

    @property
    def num_free(self) -> int:
        return _lib().qe_pages_num_free(self._h)

    def alloc(self, n: int) -> List[int]:
        return native.answer(_lib().qe_pages_alloc(self._h, n))

    def free(self, pages) -> List[int]:
        """Drop one reference of each page; returns the pages that became free."""
        return native.answer(_lib().qe_pages_release(self._h, json.dumps(list(pages)).encode()))

    def share(self, page: int) -> None:
        native.check(_lib().qe_pages_share(self._h, page))

    def check(self) -> None:
        native.check(_lib().qe_pages_check(self._h))


class SlotAllocator:
    def __init__(self, num_slots: int):
        self._h = _lib().qe_slots_create(num_slots)

    def __del__(self):
        try:
            _lib().qe_slots_free_handle(self._h)
        except Exception:
            pass

    def alloc(self) -> int:
        return native.check(_lib().qe_slots_alloc(self._h))

    def free(self, slot: int) -> None:
        native.check(_lib().qe_slots_release(self._h, slot))

    def check(self) -> None:
        native.check(_lib().qe_slots_check(self._h))


class CacheManager:
    def __init__(self, needs: Sequence[CacheNeed], page_size: int, num_pages, max_requests: int):
        """``needs[i]`` is the need of run-order entry i.  ``num_pages``: one number for every group, or one per group
        in the order in which groups first appear."""
        self._h = _lib().qe_cache_create(json.dumps([n.to_json() for n in needs]).encode(), page_size,
                                         json.dumps(num_pages).encode(), max_requests)
        if not self._h:
            raise native.last_error()
        self.page_size, self.max_requests = page_size, max_requests
        self._ids: Dict[object, int] = {}
        self._next = 1

    def __del__(self):
        try:
            _lib().qe_cache_free_handle(self._h)
        except Exception:
            pass

    def _id(self, rid) -> int:
        return self._ids[rid]

    def info(self) -> dict:
        return native.answer(_lib().qe_cache_info(self._h))

    # ---- requests
    def add_request(self, rid) -> None:
        if rid in self._ids:
            raise ValueError(f"request {rid!r} is already live")
        native.check(_lib().qe_cache_add_request(self._h, self._next))
        self._ids[rid] = self._next
        self._next += 1

    def has_request(self, rid) -> bool:
        return rid in self._ids

    def release(self, rid) -> None:
        native.check(_lib().qe_cache_release(self._h, self._ids.pop(rid)))

    def length(self, rid) -> int:
        return native.check(_lib().qe_cache_length(self._h, self._id(rid)))

    def reserve(self, rid, n: int) -> None:
        native.check(_lib().qe_cache_reserve(self._h, self._id(rid), n))

    def unreserve(self, rid) -> None:
        native.check(_lib().qe_cache_unreserve(self._h, self._id(rid)))

    def advance(self, rid, n: int) -> None:
        native.check(_lib().qe_cache_advance(self._h, self._id(rid), n))

    def truncate(self, rid, length: int) -> None:
        native.check(_lib().qe_cache_truncate(self._h, self._id(rid), length))

    def can_reserve(self, rid, n: int) -> bool:
        return bool(native.check(_lib().qe_cache_can_reserve(self._h, self._id(rid), n)))

    def pages_needed(self, rid, n: int) -> List[int]:
        return native.answer(_lib().qe_cache_pages_needed(self._h, self._id(rid), n))

    # ---- what a step needs
    def block_table(self, rid, group: int) -> List[int]:
        return self.info()["requests"][str(self._id(rid))]["tables"][group]

    def slot_of(self, rid) -> int:
        return self.info()["requests"][str(self._id(rid))]["slot"]

    def token_slots(self, rid, group: int, start: int, n: int) -> List[int]:
        return native.answer(_lib().qe_cache_token_slots(self._h, self._id(rid), group, start, n))

    # ---- accounting
    def free_pages(self) -> List[int]:
        return self.info()["free_pages"]

    def total_pages(self) -> List[int]:
        return self.info()["total_pages"]

    @property
    def groups(self) -> List[dict]:
        return self.info()["groups"]

    @property
    def state_entries(self) -> List[int]:
        return self.info()["state_entries"]

    @property
    def entry_group(self) -> Dict[int, int]:
        return {int(k): v for k, v in self.info()["entry_group"].items()}

    @property
    def free_slots(self) -> int:
        return self.info()["free_slots"]

    def check(self) -> None:
        """Raise :class:`CheckError` unless no page is lost, held twice or free while held."""
        native.check(_lib().qe_cache_check(self._h))


__all__ = ["CacheManager", "CacheNeed", "PageAllocator", "SlotAllocator", "OutOfPages", "OutOfSlots", "CheckError"]
