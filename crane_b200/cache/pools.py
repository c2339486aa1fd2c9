"""Device side of the cache: per layer the K and V page pools, or the state
tensor, laid out for the page and slot numbers of ``PageTable``.

The K pool of a layer is [pages, kv_heads, page_size, head_dim], its V pool
[pages, kv_heads, page_size, v_head_dim] (as wide as the keys unless the mixer
says otherwise): the ``page_size x width`` slab of one (page, head) is
contiguous.  Pages are
never cleared: what a request may read is decided by its length, not by the
pages' content.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..parts.base import CacheNeed, LayerCache
from .manager import GroupSpec, PageTable


def group_layers(needs: List[CacheNeed]) -> Tuple[List[Tuple[int, int, int, int]], List[int]]:
    """Group keys (kv_heads, head_dim, window, value width) in order of first use,
    and for every layer the index of its group (-1: the layer holds no pages)."""
    keys: List[Tuple[int, int, int, int]] = []
    of_layer: List[int] = []
    for need in needs:
        if need.kind != "kv":
            of_layer.append(-1)
            continue
        key = (need.kv_heads, need.head_dim, need.window, need.value_dim)
        if key not in keys:
            keys.append(key)
        of_layer.append(keys.index(key))
    return keys, of_layer


def bytes_per_page(needs: List[CacheNeed], page_size: int, elem_size: int) -> List[int]:
    """Per group, the bytes one page number costs across the group's layers."""
    keys, of_layer = group_layers(needs)
    out = [0] * len(keys)
    for need, g in zip(needs, of_layer):
        if g >= 0:
            out[g] += need.kv_heads * page_size * (need.head_dim + need.value_dim) * elem_size
    return out


class CachePools:
    def __init__(self, needs: List[CacheNeed], pages_per_group: List[int], page_size: int,
                 max_requests: int, dtype: torch.dtype, device):
        self.needs = needs
        keys, self.group_of_layer = group_layers(needs)
        if len(pages_per_group) != len(keys):
            raise ValueError("one page count per layer group is needed")
        self.groups = [GroupSpec(pages_per_group[g], page_size, keys[g][2]) for g in range(len(keys))]
        self.table = PageTable(self.groups, max_requests) if keys else PageTable(
            [GroupSpec(0, page_size, 0)], max_requests)
        self.page_size = page_size
        self.layers: List[LayerCache] = []
        for need, g in zip(needs, self.group_of_layer):
            if need.kind == "kv":
                k_shape = (pages_per_group[g], need.kv_heads, page_size, need.head_dim)
                v_shape = (pages_per_group[g], need.kv_heads, page_size, need.value_dim)
                # zeros, not uninitialised memory: rows that a tile loads but masks must be finite
                self.layers.append(LayerCache(need, g, torch.zeros(k_shape, dtype=dtype, device=device),
                                              torch.zeros(v_shape, dtype=dtype, device=device), page_size))
            elif need.kind == "state":
                st = torch.zeros((max_requests, *need.state_shape), dtype=need.state_dtype,
                                 device=device)
                self.layers.append(LayerCache(need, -1, state=st))
            else:
                self.layers.append(LayerCache(need))

    def nbytes(self) -> int:
        n = 0
        for lc in self.layers:
            for t in (lc.k, lc.v, lc.state):
                if t is not None:
                    n += t.numel() * t.element_size()
        return n
