"""Host-side bookkeeping of the cache: which sequence slots and which pages are free.

Both allocators refuse what would corrupt the cache: handing out what is held, freeing what is not
held (twice, or never acquired), or an id out of range.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """No free slot, or not enough free pages."""


class ContextLengthExceeded(CacheError):
    """A sequence would grow beyond what one sequence may hold.  Mirrors the reference's
    GenerationError::MaxSequenceLengthExceeded { actual, max }
    (crates/burn-lm-llama/src/generation/generate.rs:21-23)."""

    def __init__(self, actual: int, maximum: int):
        super().__init__(f"sequence of {actual} tokens exceeds the maximum of {maximum}")
        self.actual, self.maximum = actual, maximum


class IdAllocator:
    """Ids 0..n-1, handed out lowest first so that a freed id is used again soon."""

    def __init__(self, n: int, what: str):
        self.n, self.what = n, what
        self._free = list(range(n - 1, -1, -1))   # pop() gives the lowest
        self._held = [False] * n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def all_held(self, ids) -> bool:
        """Whether every id of a (non-empty) list is held."""
        return min(ids) >= 0 and max(ids) < self.n and all(map(self._held.__getitem__, ids))

    def acquire(self) -> int:
        if not self._free:
            raise CacheFull(f"no free {self.what} (all {self.n} are held)")
        i = self._free.pop()
        if self._held[i]:
            raise CacheError(f"{self.what} {i} was on the free list while held")
        self._held[i] = True
        return i

    def acquire_many(self, k: int) -> list:
        if k > len(self._free):
            raise CacheFull(f"{k} {self.what}s wanted, {len(self._free)} of {self.n} free")
        return [self.acquire() for _ in range(k)]

    def release(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} is out of range 0..{self.n - 1}")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is released but not held")
        self._held[i] = False
        self._free.append(i)
        # keep "lowest first": the list is sorted descending except for the new tail
        if len(self._free) > 1 and self._free[-2] < i:
            self._free.sort(reverse=True)
