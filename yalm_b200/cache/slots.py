"""Slot bookkeeping of the cache, on the host: which slot belongs to which
live sequence.  A slot is acquired when a sequence starts, released when its
batch ends, and handed out again; no slot is ever lost, held twice or freed
twice (each misuse raises).
"""
from __future__ import annotations

from typing import List


class SlotError(RuntimeError):
    pass


class SlotAllocator:
    def __init__(self, n_slots: int, what: str = "slot"):
        """``what`` names the thing in messages: the same bookkeeping hands out the
        cache's pages."""
        self.what = what
        if n_slots <= 0:
            raise SlotError(f"a cache needs at least one {what}, got {n_slots}")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))   # pop() gives the lowest
        self._held = [False] * n_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held(self) -> List[int]:
        return [s for s in range(self.n_slots) if self._held[s]]

    def acquire(self, n: int = 1) -> List[int]:
        if n > len(self._free):
            raise SlotError(f"{n} {self.what}s wanted but only {len(self._free)} of {self.n_slots} are free")
        out = []
        for _ in range(n):
            s = self._free.pop()
            assert not self._held[s]
            self._held[s] = True
            out.append(s)
        return out

    def release(self, slots) -> None:
        slots = list(slots)
        for s in slots:
            if not 0 <= s < self.n_slots:
                raise SlotError(f"{self.what} {s} does not exist (0..{self.n_slots - 1})")
            if not self._held[s]:
                raise SlotError(f"{self.what} {s} is released but not held")
        if len(set(slots)) != len(slots):
            raise SlotError(f"a {self.what} is released twice in one call: {slots}")
        for s in slots:
            self._held[s] = False
            self._free.append(s)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Invariant: every slot is either free or held, exactly once."""
        free = sorted(self._free)
        held = self.held
        if sorted(free + held) != list(range(self.n_slots)) or len(set(free)) != len(free):
            raise SlotError(f"{self.what} table corrupt: free={free} held={held}")
