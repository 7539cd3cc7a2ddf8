"""Bookkeeping of cache pages and state slots (host only, no tensors).

``IdPool`` hands out integer ids (pages of one group, or state slots) and takes
them back.  It refuses to free an id that is not held, so a page can neither be
lost, held twice nor freed twice without an exception.  Freed ids are reused
last-in-first-out: a page that was just given back is the next to be handed out,
which makes reuse happen early and reproducibly.
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """A group has fewer free pages than an append needs."""


class IdPool:
    def __init__(self, count: int, what: str = "page"):
        if count < 0:
            raise ValueError(f"{what} count must be >= 0, got {count}")
        self.count = count
        self.what = what
        self._free = list(range(count - 1, -1, -1))     # pop() hands out 0 first
        self._held: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return len(self._held)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages(f"no free {self.what} (all {self.count} are held)")
        i = self._free.pop()
        self._held.add(i)
        return i

    def give_back(self, i: int) -> None:
        if i not in self._held:
            raise RuntimeError(f"{self.what} {i} is given back but is not held")
        self._held.remove(i)
        self._free.append(i)

    def check(self) -> None:
        """Every id is either free or held, exactly once."""
        if len(set(self._free)) != len(self._free):
            raise AssertionError(f"a {self.what} is on the free list twice")
        if set(self._free) & self._held:
            raise AssertionError(f"a {self.what} is both free and held")
        if len(self._free) + len(self._held) != self.count:
            raise AssertionError(f"a {self.what} was lost")
