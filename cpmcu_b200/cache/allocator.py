"""Host-side bookkeeping of what the cache hands out: sequence slots and pages.

Nothing here touches a device.  A handle that is given back twice, or that was
never handed out, is an error, so a leak or a double free shows at once.
"""
from __future__ import annotations

from typing import List


class CacheFull(RuntimeError):
    """The cache has no free slot or not enough free pages for the request."""


class HandleError(RuntimeError):
    """A slot or page was freed twice, or was never handed out."""


class FreeList:
    """Integers 0..n-1; lowest free number first, so runs are reproducible."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free: List[int] = list(range(self.n - 1, -1, -1))   # pop() gives the lowest
        self._held = [False] * self.n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def take(self, count: int = 1) -> List[int]:
        if count > len(self._free):
            raise CacheFull(f"{count} {self.what}(s) wanted, {len(self._free)} of {self.n} free")
        out = [self._free.pop() for _ in range(count)]
        for i in out:
            self._held[i] = True
        return out

    def give_back(self, handles) -> None:
        for i in handles:
            if not (0 <= i < self.n) or not self._held[i]:
                raise HandleError(f"{self.what} {i} is not held (freed twice, or never handed out)")
        for i in handles:
            self._held[i] = False
        self._free.extend(handles)
        self._free.sort(reverse=True)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]
