"""Free lists with checks: nothing is lost, held twice or freed twice."""
from __future__ import annotations


class CacheFull(RuntimeError):
    """No room left: pages, slots or positions (the reference raises
    RuntimeError("context window full"), alpacca/model.py:441-442)."""


class IdPool:
    """Hands out the ids 0..n-1.  The lowest free id comes first, so that a
    freed id is used again at once (which is what the tests of reuse rely on)."""

    def __init__(self, n: int, what: str = "id"):
        self.n, self.what = int(n), what
        self._free = list(range(self.n - 1, -1, -1))   # stack; pop() gives the lowest after a sort
        self._held = bytearray(self.n)
        self._unsorted = False

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are in use)")
        if self._unsorted:
            self._free.sort(reverse=True)
            self._unsorted = False
        i = self._free.pop()
        assert not self._held[i], f"{self.what} {i} was on the free list while held"
        self._held[i] = 1
        return i

    def alloc_many(self, k: int) -> list[int]:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.alloc() for _ in range(k)]

    def free(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise ValueError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise ValueError(f"{self.what} {i} is freed twice (or was never given out)")
        self._held[i] = 0
        if self._free and self._free[-1] < i:
            self._unsorted = True
        self._free.append(i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and bool(self._held[i])

    def check(self) -> None:
        """Raises if the books do not balance."""
        free = set(self._free)
        assert len(free) == len(self._free), f"a {self.what} is on the free list twice"
        for i in range(self.n):
            assert bool(self._held[i]) != (i in free), f"{self.what} {i} is both held and free, or neither"
