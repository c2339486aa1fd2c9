"""The cache manager: page and slot bookkeeping (native, host side) together
with the device tensors that the page and slot numbers index.

Layers whose mixers need the same thing (kv heads, head size, window) form a
group with its own page pool, page size and block tables.  A layer that reads
another layer's cache owns nothing.  Every request also gets a state slot; a
mixer with state of fixed size finds its tensor [slots, ...] there.  Hunyuan
Dense has one group (all layers, every earlier position) and no state.
"""
from __future__ import annotations

from ctypes import c_int, c_int64, c_void_p
from dataclasses import dataclass
from typing import Sequence

import numpy as np

from ..csrc import build


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    pass


@dataclass(frozen=True)
class GroupSpec:
    num_pages: int
    page_size: int
    window: int = 0


_lib = None


def _host():
    global _lib
    if _lib is None:
        lib = build.load_host()
        I, L, P = c_int, c_int64, c_void_p
        sig = {
            "crane_cache_create": ([I, P, P, P, I], P),
            "crane_cache_destroy": ([P], None),
            "crane_cache_admit": ([P, L], I),
            "crane_cache_extend": ([P, L, I], I),
            "crane_cache_pages_needed": ([P, L, I, I], I),
            "crane_cache_release": ([P, L], I),
            "crane_cache_length": ([P, L], I),
            "crane_cache_slot": ([P, L], I),
            "crane_cache_block_table": ([P, L, I, P, I], I),
            "crane_cache_fill_step": ([P, I, P, P, P, I, I, I, I, I, P, P], I),
            "crane_cache_free_pages": ([P, I], I),
            "crane_cache_total_pages": ([P, I], I),
            "crane_cache_free_slots": ([P], I),
            "crane_cache_live": ([P], I),
            "crane_cache_pages_reused": ([P], L),
            "crane_cache_check": ([P], I),
        }
        for name, (args, res) in sig.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, res
        _lib = lib
    return _lib


class PageTable:
    """Bookkeeping only: which request holds which pages and which slot."""

    def __init__(self, groups: Sequence[GroupSpec], max_requests: int):
        self.groups = list(groups)
        self.max_requests = int(max_requests)
        n = len(self.groups)
        arr = lambda vals: (c_int * n)(*vals)
        self._lib = _host()
        self._h = self._lib.crane_cache_create(
            n, arr([g.num_pages for g in groups]), arr([g.page_size for g in groups]),
            arr([g.window for g in groups]), self.max_requests)
        if not self._h:
            raise CacheError(f"invalid cache geometry: {groups}, max_requests={max_requests}")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.crane_cache_destroy(h)

    @property
    def handle(self):
        return self._h

    def admit(self, rid: int) -> int:
        s = self._lib.crane_cache_admit(self._h, rid)
        if s == -2:
            raise CacheError(f"request {rid} is already live")
        if s < 0:
            raise CacheError(f"no free state slot for request {rid} "
                             f"({self.max_requests} requests are live)")
        return s

    def extend(self, rid: int, n_new: int) -> None:
        r = self._lib.crane_cache_extend(self._h, rid, n_new)
        if r == -1:
            raise OutOfPages(f"request {rid}: not enough free pages for {n_new} more tokens "
                             f"(free per group: {[self.free_pages(g) for g in range(len(self.groups))]})")
        if r != 0:
            raise CacheError(f"request {rid} is not live")

    def try_extend(self, rid: int, n_new: int) -> bool:
        return self._lib.crane_cache_extend(self._h, rid, n_new) == 0

    def pages_needed(self, rid: int, n_new: int, group: int) -> int:
        return self._lib.crane_cache_pages_needed(self._h, rid, n_new, group)

    def release(self, rid: int) -> None:
        if self._lib.crane_cache_release(self._h, rid) != 0:
            raise CacheError(f"request {rid} is not live (released twice?)")

    def is_live(self, rid: int) -> bool:
        return self._lib.crane_cache_length(self._h, rid) >= 0

    def length(self, rid: int) -> int:
        n = self._lib.crane_cache_length(self._h, rid)
        if n < 0:
            raise CacheError(f"request {rid} is not live")
        return n

    def slot(self, rid: int) -> int:
        s = self._lib.crane_cache_slot(self._h, rid)
        if s < 0:
            raise CacheError(f"request {rid} is not live")
        return s

    def block_table_into(self, rid: int, group: int, out: np.ndarray) -> int:
        """Fills the int32 row ``out`` (contiguous); returns the blocks in use."""
        n = self._lib.crane_cache_block_table(self._h, rid, group, out.ctypes.data, out.shape[0])
        if n < 0:
            raise CacheError(f"request {rid} is not live")
        return n

    def block_table(self, rid: int, group: int, capacity: int) -> np.ndarray:
        out = np.empty(capacity, dtype=np.int32)
        self.block_table_into(rid, group, out)
        return out

    def fill_step(self, ids: np.ndarray, counts: np.ndarray, meta: np.ndarray, off_positions: int,
                  off_tok_entry: int, off_cu_q: int, off_kv_len: int, off_slots: int,
                  off_tables: np.ndarray, max_blocks: np.ndarray) -> int:
        """One native call that writes positions, entry of each token, cu_q,
        kv_len, slots and every group's block-table rows of a step into the
        int32 block ``meta``.  Returns the number of tokens."""
        n = self._lib.crane_cache_fill_step(
            self._h, len(ids), ids.ctypes.data, counts.ctypes.data, meta.ctypes.data, off_positions,
            off_tok_entry, off_cu_q, off_kv_len, off_slots, off_tables.ctypes.data,
            max_blocks.ctypes.data)
        if n < 0:
            raise CacheError("a request of the step is not live")
        return n

    def free_pages(self, group: int = 0) -> int:
        return self._lib.crane_cache_free_pages(self._h, group)

    def total_pages(self, group: int = 0) -> int:
        return self._lib.crane_cache_total_pages(self._h, group)

    def free_slots(self) -> int:
        return self._lib.crane_cache_free_slots(self._h)

    def live(self) -> int:
        return self._lib.crane_cache_live(self._h)

    def pages_reused(self) -> int:
        return int(self._lib.crane_cache_pages_reused(self._h))

    def check(self) -> None:
        """Raises unless every page and slot is free or held exactly once."""
        code = self._lib.crane_cache_check(self._h)
        if code:
            what = {1: "a slot is free twice", 2: "a slot is held twice", 3: "a slot is lost",
                    4: "a page is free twice", 5: "a page is held twice", 6: "a page is lost"}
            raise CacheError("cache bookkeeping is inconsistent: " + what.get(code, str(code)))
