"""Host-side bookkeeping of the cache: a pool of fixed-size pages and a table of slots.

Both are plain free lists with the invariants checked on every call: a page or slot is never
handed out twice, never freed twice, and never lost (`check` recounts them).
"""
from __future__ import annotations


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    pass


class FreeList:
    """Ids 0..n-1, each either free or held."""

    def __init__(self, n: int, what: str):
        if n <= 0:
            raise CacheError(f"a pool of {n} {what}s")
        self.n, self.what = int(n), what
        self._free = list(range(self.n - 1, -1, -1))     # pop() hands out the lowest id first
        self._held = [False] * self.n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def take(self, count: int = 1) -> list[int]:
        if count < 0:
            raise CacheError(f"asked for {count} {self.what}s")
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            self._held[i] = True
        return out

    def give_back(self, ids) -> None:
        ids = list(ids)
        for i in ids:
            if not 0 <= i < self.n:
                raise CacheError(f"{self.what} {i} is not of this pool (0..{self.n - 1})")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} freed twice (or never handed out)")
            self._held[i] = False
        # released ids are reused first, lowest id on top
        self._free.extend(sorted(ids, reverse=True))

    def is_held(self, i: int) -> bool:
        return self._held[i]

    def check(self) -> None:
        """Recounts: every id is exactly once either free or held."""
        seen = [0] * self.n
        for i in self._free:
            seen[i] += 1
        for i in range(self.n):
            if seen[i] + (1 if self._held[i] else 0) != 1:
                state = "both free and held" if seen[i] and self._held[i] else \
                    ("lost" if not seen[i] else "in the free list twice")
                raise CacheError(f"{self.what} {i} is {state}")
