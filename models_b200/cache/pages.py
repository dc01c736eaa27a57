"""Free lists with ownership checks: pages of a cache group, and slots of the batch.

The counterpart in integrallis/models is one KvCache object per session, grown lazily and reset when
the session closes (backend-java/.../cache/KvCache.java:284-322,
backend-java/.../PureJavaBackend.java:536-544).  Here storage is allocated once and handed out in
fixed units, so giving a unit back and handing it out again costs nothing and moves no memory.
"""

from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """No free page (or slot) is left for what a step needs."""


class FreeList:
    """Hands out the integers [first, first + count) and takes them back.  An id is never held
    twice, never lost, and cannot be given back twice."""

    def __init__(self, count: int, first: int = 0, what: str = "unit"):
        if count < 0:
            raise ValueError(f"{what} count must be >= 0, got {count}")
        self.what = what
        self.first = first
        self.count = count
        # lowest id on top, so a fresh pool hands out ascending ids and a released id is reused first
        self._free: List[int] = list(range(first + count - 1, first - 1, -1))
        self._held = set()

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return len(self._held)

    def take(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} left (all {self.count} are held)")
        unit = self._free.pop()
        self._held.add(unit)
        return unit

    def give_back(self, unit: int) -> None:
        if unit not in self._held:
            raise ValueError(f"{self.what} {unit} is not held (given back twice, or never taken)")
        self._held.remove(unit)
        self._free.append(unit)

    def is_held(self, unit: int) -> bool:
        return unit in self._held

    def check(self) -> None:
        """Every id is either free or held, exactly once."""
        free = list(self._free)
        if len(set(free)) != len(free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        if set(free) & self._held:
            raise AssertionError(f"a {self.what} is both free and held")
        if len(free) + len(self._held) != self.count:
            raise AssertionError(f"{self.count - len(free) - len(self._held)} {self.what}s are lost")
