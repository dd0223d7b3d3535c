"""Host-side bookkeeping of the cache: which slots and pages are free. Pure Python, no device memory, so the
accounting (nothing lost, nothing held twice, nothing freed twice) is testable anywhere."""
from __future__ import annotations


class CacheError(RuntimeError):
    """A request the cache cannot serve: out of slots or pages, a slot used after release, a double release."""


class FreeList:
    """`count` numbered items; `take` hands out free ones (the most recently returned first), `give` returns them."""

    def __init__(self, count: int, what: str) -> None:
        self.count = int(count)
        self.what = what
        self._free = list(range(self.count - 1, -1, -1))  # pop() yields the lowest number
        self._held = [False] * self.count

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.count - len(self._free)

    def take(self, n: int = 1) -> list[int]:
        if n > len(self._free):
            raise CacheError(f"out of {self.what}s: {n} wanted, {len(self._free)} of {self.count} free")
        out = [self._free.pop() for _ in range(n)]
        for item in out:
            self._held[item] = True
        return out

    def give(self, items) -> None:
        items = list(items)
        for item in items:
            if not 0 <= item < self.count:
                raise CacheError(f"{self.what} {item} does not exist")
            if not self._held[item]:
                raise CacheError(f"{self.what} {item} is released twice (or was never taken)")
            self._held[item] = False
        self._free.extend(items)  # last given back, first taken again

    def is_held(self, item: int) -> bool:
        return 0 <= item < self.count and self._held[item]

    def check(self) -> None:
        """Every item is either free or held, exactly once."""
        assert len(set(self._free)) == len(self._free), f"a {self.what} is on the free list twice"
        for item in range(self.count):
            assert self._held[item] != (item in self._free), f"{self.what} {item} is lost or both free and held"
