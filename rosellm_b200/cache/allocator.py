"""Page and slot allocators: plain host bookkeeping, no tensors.

The reference's ``GlobalKVBlockManager`` hands out block ids from a LIFO free
list and then a bump counter, and raises ``RuntimeError("no more KV blocks
available")`` from inside a step when both are empty
(rosellm/roseinfer/engine.py:4410-4417).  Here allocation is all-or-nothing
and reports failure to the caller, which decides what to do (the scheduler
stops admitting or preempts).  Freed ids go on a stack, so the page freed last
is the page handed out next: a test with few pages re-uses them at once.
"""
from __future__ import annotations


class DoubleFree(RuntimeError):
    pass


class IdAllocator:
    """Hands out ids ``0..capacity-1``; every id is either free or held, never both."""

    def __init__(self, capacity: int, what: str = "id") -> None:
        if capacity <= 0:
            raise ValueError(f"{what} capacity must be positive")
        self.capacity = int(capacity)
        self.what = what
        self._free = list(range(self.capacity - 1, -1, -1))  # pop() gives 0 first
        self._held = [False] * self.capacity

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.capacity - len(self._free)

    def is_held(self, i: int) -> bool:
        return self._held[i]

    def alloc(self, n: int = 1) -> list[int] | None:
        """``n`` ids, or ``None`` (and nothing taken) when fewer are free."""
        if n < 0:
            raise ValueError("n must be non-negative")
        if n > len(self._free):
            return None
        if n == 0:
            return []
        out = self._free[-n:]
        del self._free[-n:]
        out.reverse()  # the order pop() would have given
        held = self._held
        for i in out:
            held[i] = True
        return out

    def free(self, ids) -> None:
        for i in ids:
            if not 0 <= i < self.capacity:
                raise ValueError(f"{self.what} {i} out of range 0..{self.capacity - 1}")
            if not self._held[i]:
                raise DoubleFree(f"{self.what} {i} freed while not held")
            self._held[i] = False
            self._free.append(i)

    def check(self) -> None:
        """Raise if the free list and the held flags disagree."""
        if len(set(self._free)) != len(self._free):
            raise AssertionError(f"{self.what}: an id is twice on the free list")
        for i in self._free:
            if self._held[i]:
                raise AssertionError(f"{self.what} {i} is both free and held")
        if sum(self._held) + len(self._free) != self.capacity:
            raise AssertionError(f"{self.what}: an id is lost")
