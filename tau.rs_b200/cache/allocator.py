"""Host bookkeeping of numbered things that are handed out and given back.

Used for cache pages and for sequence slots.  Every misuse is an error rather than a
silent repair: taking more than there is, giving back something that is not out, or
giving it back twice.  `check()` verifies that nothing is lost or held twice.
"""
from __future__ import annotations

from typing import Iterable, List


class CacheFull(RuntimeError):
    """The cache cannot hold what the step asks for."""


class FreeList:
    def __init__(self, count: int, what: str = "item"):
        self.count = count
        self.what = what
        # Lowest numbers go out first, and a number that comes back goes out again
        # next, so reuse happens early and tests meet it.
        self._free: List[int] = list(range(count - 1, -1, -1))
        self._out = [False] * count

    @property
    def available(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.count - len(self._free)

    def take(self, wanted: int = 1) -> List[int]:
        if wanted > len(self._free):
            raise CacheFull(f"{wanted} {self.what}(s) wanted, {len(self._free)} of {self.count} free")
        taken = [self._free.pop() for _ in range(wanted)]
        for index in taken:
            self._out[index] = True
        return taken

    def give_back(self, indices: Iterable[int]) -> None:
        indices = list(indices)
        for index in indices:
            if not 0 <= index < self.count:
                raise ValueError(f"{self.what} {index} does not exist")
            if not self._out[index]:
                raise ValueError(f"{self.what} {index} is given back but is not in use")
            self._out[index] = False
        self._free.extend(reversed(indices))

    def is_out(self, index: int) -> bool:
        return 0 <= index < self.count and self._out[index]

    def check(self) -> None:
        if len(set(self._free)) != len(self._free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        if any(self._out[index] for index in self._free):
            raise AssertionError(f"a {self.what} is both free and in use")
        if len(self._free) + sum(self._out) != self.count:
            raise AssertionError(f"a {self.what} is lost")
