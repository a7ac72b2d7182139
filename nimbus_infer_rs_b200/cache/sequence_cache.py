"""Everything a live sequence holds between steps: a slot, its length, its pages in every
cache group, and its rows of fixed-size state.

Write protocol (src/cache.rs:35-57, src/engine.rs:273-274,288-289): a step writes keys and
values at positions ``len .. len+T`` of each of its sequences; the length is advanced by the
engine when the step has been launched.
"""
from __future__ import annotations

import torch

from ..parts.base import KVRequest, StateRequest
from .paged import PAGE, CacheGroup, pages_for
from .slots import CacheError, SlotAllocator


class SequenceCache:
    def __init__(self, kv_requests: dict[int, KVRequest], state_requests: dict[int, StateRequest],
                 *, cache_tokens: int, max_seq_len: int, dtype: torch.dtype, device,
                 n_slots: int | None = None):
        """``kv_requests`` / ``state_requests``: per schedule entry (a layer that runs twice
        has two), for entries that keep storage of their own.  ``cache_tokens``: the most tokens live sequences hold at any time, each
        sequence counted in whole pages of 64."""
        if cache_tokens <= 0:
            raise ValueError("cache_tokens must be positive")
        self.max_seq_len = int(max_seq_len)
        self.n_pages = pages_for(cache_tokens)
        self.cache_tokens = self.n_pages * PAGE
        self.n_slots = int(n_slots) if n_slots else max(1, min(self.n_pages, 4096))
        self.slots = SlotAllocator(self.n_slots)
        self.dtype = dtype
        self.device = device
        self.lens = [0] * self.n_slots

        by_request: dict[KVRequest, list[int]] = {}
        for layer, req in sorted(kv_requests.items()):
            by_request.setdefault(req, []).append(layer)
        self.groups = [CacheGroup(req, layers, self.n_pages, self.n_slots, self.max_seq_len,
                                  dtype, device) for req, layers in by_request.items()]
        self._group_of = {l: g for g in self.groups for l in g.layers}

        self.state: dict[int, torch.Tensor] = {
            layer: torch.zeros((self.n_slots, req.n_elements), dtype=torch.float32, device=device)
            for layer, req in sorted(state_requests.items()) if req.n_elements > 0}

    # ---------------------------------------------------------------- views for mixers
    def layer_kv(self, layer: int):
        g = self._group_of.get(layer)
        return None if g is None else g.layer_view(layer)

    def layer_state(self, layer: int):
        return self.state.get(layer)

    # ---------------------------------------------------------------- slots
    def alloc_slot(self) -> int:
        s = self.slots.alloc()
        self.lens[s] = 0
        for t in self.state.values():
            t[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.slots.free(slot)
        for g in self.groups:
            g.release(slot)
        self.lens[slot] = 0

    # ---------------------------------------------------------------- growth
    def reserve(self, growth: list[tuple[int, int]]) -> None:
        """Make room for ``n_new`` more tokens in each ``(slot, n_new)``; all or nothing."""
        seen = set()
        for slot, n_new in growth:
            self.slots.check_held(slot)
            if slot in seen:
                raise CacheError(f"slot {slot} appears twice in one step")
            seen.add(slot)
            if n_new < 0 or self.lens[slot] + n_new > self.max_seq_len:
                raise CacheError(
                    f"slot {slot}: length {self.lens[slot]} + {n_new} exceeds the longest "
                    f"sequence of the model ({self.max_seq_len})")
        for g in self.groups:
            need = sum(g.pages_needed(s, self.lens[s] + n) for s, n in growth)
            if need > g.pool.n_free:
                raise CacheError(
                    f"cache is full: this step needs {need} more pages of {PAGE} tokens, "
                    f"{g.pool.n_free} of {g.pool.n_pages} are free")
        for g in self.groups:
            for s, n in growth:
                g.ensure(s, self.lens[s] + n)
            g.flush()

    def advance(self, slot: int, n: int) -> None:
        """The step that wrote ``n`` more tokens of ``slot`` has been launched.  Groups with a
        window give back the pages no later token reads; work launched later on the same
        stream may write them again, which is after every read of this step."""
        self.lens[slot] += n
        for g in self.groups:
            g.trim(slot, self.lens[slot])

    # ---------------------------------------------------------------- accounting
    def tokens_held(self) -> int:
        return sum(pages_for(self.lens[s]) * PAGE for s in self.slots.held)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + sum(
            t.numel() * 4 for t in self.state.values())
