"""Fixed-size unit allocators: cache pages and per-request state slots.

Tensor-free, like the reference's ``BlockAllocator`` (edgerag/cache/allocator.py:76-196): a LIFO
free stack (a unit that was just freed is the next one handed out, which makes stale-page faults
show early), all-or-nothing allocation, and errors that separate an expected condition (the pool
is exhausted) from bugs (freeing a unit twice, or one that was never handed out).  Sharing of
units between requests is not built, so a unit is either free or held by exactly one owner.
"""

from __future__ import annotations

from dataclasses import dataclass


class AllocatorError(RuntimeError):
    """Misuse of an allocator: always a bug of the caller."""


class OutOfPagesError(AllocatorError):
    """Not enough free units.  An expected condition: the caller waits, preempts or rejects."""


class DoubleFreeError(AllocatorError):
    """A unit was freed that is not held."""


@dataclass
class AllocatorStats:
    allocations: int = 0
    frees: int = 0
    failed_allocations: int = 0
    peak_used: int = 0

    def to_dict(self) -> dict[str, int]:
        return dict(self.__dict__)


class UnitAllocator:
    """Hands out integer ids ``0 .. capacity-1``; used for pages (per cache group) and state slots."""

    def __init__(self, capacity: int, what: str = "page") -> None:
        if capacity <= 0:
            raise ValueError(f"{what} capacity must be positive, got {capacity}")
        self.capacity = capacity
        self.what = what
        # Unit 0 is on top of the stack, so a fresh pool hands out 0, 1, 2, ...
        self._free: list[int] = list(range(capacity - 1, -1, -1))
        self._held = bytearray(capacity)
        self.stats = AllocatorStats()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.capacity - len(self._free)

    def is_held(self, unit: int) -> bool:
        self._validate(unit)
        return bool(self._held[unit])

    def allocate(self, n: int = 1) -> list[int]:
        """``n`` units, or ``OutOfPagesError`` with the pool untouched."""
        if n < 0:
            raise ValueError(f"cannot allocate {n} {self.what}s")
        if n > len(self._free):
            self.stats.failed_allocations += 1
            raise OutOfPagesError(f"need {n} {self.what}s, {len(self._free)} of {self.capacity} free")
        units = [self._free.pop() for _ in range(n)]
        for u in units:
            self._held[u] = 1
        self.stats.allocations += n
        self.stats.peak_used = max(self.stats.peak_used, self.num_used)
        return units

    def free(self, units: list[int]) -> None:
        """Give units back.  Checks all of them before changing anything."""
        seen = set()
        for u in units:
            self._validate(u)
            if not self._held[u] or u in seen:
                raise DoubleFreeError(f"{self.what} {u} is not held (double free)")
            seen.add(u)
        for u in units:
            self._held[u] = 0
            self._free.append(u)
        self.stats.frees += len(units)

    def _validate(self, unit: int) -> None:
        if not 0 <= unit < self.capacity:
            raise AllocatorError(f"{self.what} id {unit} is outside [0, {self.capacity})")

    def check_invariants(self) -> None:
        """Every unit is either on the free stack exactly once or marked held; never both."""
        if len(set(self._free)) != len(self._free):
            raise AllocatorError(f"a {self.what} is on the free stack twice")
        for u in self._free:
            if self._held[u]:
                raise AllocatorError(f"{self.what} {u} is free and held")
        if sum(self._held) + len(self._free) != self.capacity:
            raise AllocatorError(f"{self.what}s lost: {sum(self._held)} held + {len(self._free)} free != {self.capacity}")

    def to_dict(self) -> dict[str, object]:
        return {"capacity": self.capacity, "free": self.num_free, "used": self.num_used, **self.stats.to_dict()}
