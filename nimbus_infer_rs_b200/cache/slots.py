"""Hand-out of sequence slots.  A slot is a small integer that names one live sequence in
every per-sequence table (lengths, block tables, state rows).  Freed slots are handed out
again, most recently freed first, and nothing is cleared but the state rows."""
from __future__ import annotations


class CacheError(RuntimeError):
    """A request the cache cannot honour (no slot, no page, bad slot, over length).  Raised on
    the host before anything is launched."""


class SlotAllocator:
    def __init__(self, n_slots: int):
        if n_slots <= 0:
            raise ValueError("n_slots must be positive")
        self.n_slots = int(n_slots)
        self._free = list(range(self.n_slots - 1, -1, -1))  # pop() gives the lowest first
        self._held: set[int] = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> frozenset[int]:
        return frozenset(self._held)

    def alloc(self) -> int:
        if not self._free:
            raise CacheError(f"no free sequence slot (all {self.n_slots} are held)")
        s = self._free.pop()
        self._held.add(s)
        return s

    def free(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"slot {slot} is not held (freed twice or never handed out)")
        self._held.remove(slot)
        self._free.append(slot)

    def check_held(self, slot: int) -> None:
        if slot not in self._held:
            raise CacheError(f"slot {slot} is not held")
