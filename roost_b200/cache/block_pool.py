"""A pool of page ids with reference counts.

Ids run 0 .. capacity-1. Free ids sit on a LIFO stack that hands out 0 first, so a page that has just been
given back is the next one taken: reuse is certain and the order of ids is a function of the call sequence.
Allocation is all-or-none; a release of a free page raises and changes nothing. The design follows the
reference's pool (src/Starlings.Roost.Engine/Blocks/BlockPool.cs:65-173, invariants :312-349); forks and
copy-on-write are not built, but the count per page is kept so that sharing can be added.
"""
from __future__ import annotations

NULL_PAGE = -1


class PoolError(RuntimeError):
    pass


class BlockPool:
    def __init__(self, capacity: int, name: str = "pool"):
        if capacity < 0:
            raise ValueError(f"{name}: capacity {capacity} is negative")
        self.name = name
        self.capacity = capacity
        self._refs = [0] * capacity
        self._free = list(range(capacity - 1, -1, -1))  # pop() gives 0 first

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.capacity - len(self._free)

    def try_allocate(self, n: int) -> list[int] | None:
        """n pages, or None (and nothing taken) when fewer are free."""
        if n < 0:
            raise ValueError(f"{self.name}: cannot allocate {n} pages")
        if n > len(self._free):
            return None
        out = []
        for _ in range(n):
            p = self._free.pop()
            self._refs[p] = 1
            out.append(p)
        return out

    def release(self, page: int) -> None:
        if not 0 <= page < self.capacity:
            raise PoolError(f"{self.name}: page {page} is outside 0..{self.capacity - 1}")
        if self._refs[page] <= 0:
            raise PoolError(f"{self.name}: page {page} is already free (double release)")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refs(self, page: int) -> int:
        return self._refs[page]

    def check_invariants(self) -> None:
        """Every id is either free (count 0, once on the stack) or held (count > 0, not on the stack)."""
        seen = set()
        for p in self._free:
            if not 0 <= p < self.capacity:
                raise PoolError(f"{self.name}: free stack holds id {p}")
            if p in seen:
                raise PoolError(f"{self.name}: page {p} is on the free stack twice")
            seen.add(p)
            if self._refs[p] != 0:
                raise PoolError(f"{self.name}: page {p} is free but has count {self._refs[p]}")
        for p in range(self.capacity):
            if p not in seen and self._refs[p] <= 0:
                raise PoolError(f"{self.name}: page {p} is neither free nor held (lost)")
