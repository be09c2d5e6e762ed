"""Host-side allocators of the cache: sequence slots and pages.

Both hand out small integers from a free list, refuse to hand out more than
they have, and refuse to take back what is not out: a slot or a page is never
lost, held twice or freed twice."""
from typing import Iterable, List


class CacheFull(RuntimeError):
    """The cache has no free slot or page left for the request."""


class FreeList:
    def __init__(self, count: int, what: str):
        self.count, self.what = count, what
        self._free = list(range(count - 1, -1, -1))     # pop() hands out 0 first
        self._out = set()

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def in_use(self):
        return frozenset(self._out)

    def alloc(self, n: int = 1) -> List[int]:
        if n < 0:
            raise ValueError(f"cannot allocate {n} {self.what}s")
        if n > len(self._free):
            raise CacheFull(f"{n} {self.what}(s) wanted, {len(self._free)} of {self.count} free")
        got = [self._free.pop() for _ in range(n)]
        self._out.update(got)
        return got

    def free(self, items: Iterable[int]) -> None:
        items = list(items)
        seen = set()
        for i in items:
            if i not in self._out or i in seen:
                raise ValueError(f"{self.what} {i} is not in use (freed twice, or never allocated)")
            seen.add(i)
        for i in items:
            self._out.discard(i)
            self._free.append(i)
