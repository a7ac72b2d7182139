"""Paged key/value storage.

Layers whose mixers ask for the same kind of storage (same number of key/value heads, head
size and window) form a *group* with a page pool, block tables and tensors of its own:

    storage[layer_in_group][0=keys | 1=values][page][kv_head][token_in_page][head_dim]

A page holds ``PAGE`` consecutive tokens of one sequence, for every layer of the group at
once, so a sequence's block table (its list of pages) is shared by the group's layers.  One
(page, head) is a contiguous ``PAGE x head_dim`` tile, the unit the attention kernels load.

A group with a window gives a page back to its pool as soon as every token of the page lies
before the window of the sequence's next token (``trim``): a long sequence then holds about
``window / PAGE + 2`` pages of that group, while a group without a window holds them all.
The block-table entry of a page that was given back is never read again (the kernels start at
the window's first key), so it is left as it is.

The reference keeps one dense array per layer of ``(n_kv_heads, max_seq, head_dim)`` for a
single sequence (src/cache.rs:10-29); paging replaces ``max_seq`` by the pages a sequence
actually holds, so many sequences of unequal length share the memory.
"""
from __future__ import annotations

import heapq
from dataclasses import dataclass

import numpy as np
import torch

from ..parts.base import KVRequest
from .slots import CacheError

PAGE = 64  # tokens per page


def pages_for(n_tokens: int) -> int:
    return (n_tokens + PAGE - 1) // PAGE


@dataclass
class LayerKV:
    """One layer's view of its group: what the kernels need."""
    k: torch.Tensor            # [n_pages, n_kv_heads, PAGE, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor  # int32 [n_slots, max_pages]
    page: int
    n_kv_heads: int
    head_dim: int
    window: int = 0


class PagePool:
    """Free pages are handed out lowest number first (a heap): the pages a prompt takes in one
    go are then neighbours in memory, also after many batches have come and gone."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._free = list(range(self.n_pages))      # a heap: sorted lists are heaps
        self._held: set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise CacheError(f"cache is full: {n} pages wanted, {len(self._free)} free "
                             f"of {self.n_pages}")
        out = [heapq.heappop(self._free) for _ in range(n)]
        self._held.update(out)
        return out

    def release(self, pages: list[int]) -> None:
        for p in pages:
            if p not in self._held:
                raise CacheError(f"page {p} is not held (released twice)")
            self._held.remove(p)
            heapq.heappush(self._free, p)


class CacheGroup:
    def __init__(self, request: KVRequest, layers: list[int], n_pages: int, n_slots: int,
                 max_seq_len: int, dtype: torch.dtype, device):
        self.request = request
        self.layers = list(layers)
        self.pool = PagePool(n_pages)
        self.max_pages = max(1, pages_for(max_seq_len))
        self.storage = torch.zeros(
            (len(self.layers), 2, n_pages, request.n_kv_heads, PAGE, request.head_dim),
            dtype=dtype, device=device)
        self.block_table = torch.zeros((n_slots, self.max_pages), dtype=torch.int32, device=device)
        self._table_host = np.zeros((n_slots, self.max_pages), dtype=np.int32)
        self._pages: dict[int, list[int]] = {}   # slot -> page of every page index (-1: given back)
        self._dirty: set[int] = set()

    def bytes(self) -> int:
        return self.storage.numel() * self.storage.element_size()

    def pages_needed(self, slot: int, n_tokens: int) -> int:
        return max(0, pages_for(n_tokens) - len(self._pages.get(slot, ())))

    def ensure(self, slot: int, n_tokens: int) -> None:
        need = self.pages_needed(slot, n_tokens)
        if need == 0:
            return
        have = self._pages.setdefault(slot, [])
        if len(have) + need > self.max_pages:
            raise CacheError(f"slot {slot}: {n_tokens} tokens exceed the longest sequence")
        new = self.pool.alloc(need)
        self._table_host[slot, len(have):len(have) + need] = new
        have.extend(new)
        self._dirty.add(slot)

    def trim(self, slot: int, length: int) -> int:
        """Give back the pages that lie wholly before the window of the token at position
        ``length`` (the next one the sequence writes); returns how many.  That token reads the
        keys at ``length - window + 1 .. length``."""
        w = self.request.window
        pages = self._pages.get(slot)
        if w <= 0 or not pages:
            return 0
        first_needed = max(0, length - w + 1) // PAGE
        gone = [p for p in pages[:first_needed] if p >= 0]
        if gone:
            self.pool.release(gone)
            pages[:first_needed] = [-1] * first_needed
        return len(gone)

    def release(self, slot: int) -> None:
        pages = self._pages.pop(slot, None)
        if pages:
            self.pool.release([p for p in pages if p >= 0])

    def pages_of(self, slot: int) -> list[int]:
        """The pages the slot holds now, in order of page index (pages given back left out)."""
        return [p for p in self._pages.get(slot, ()) if p >= 0]

    def flush(self) -> None:
        """Bring the device block table up to date (one copy per changed row span)."""
        if not self._dirty:
            return
        lo, hi = min(self._dirty), max(self._dirty) + 1
        src = torch.from_numpy(self._table_host[lo:hi])
        self.block_table[lo:hi].copy_(src, non_blocking=False)
        self._dirty.clear()

    def layer_view(self, layer: int) -> LayerKV:
        i = self.layers.index(layer)
        r = self.request
        return LayerKV(self.storage[i, 0], self.storage[i, 1], self.block_table, PAGE,
                       r.n_kv_heads, r.head_dim, r.window)
