"""A pool of numbered units (slots, pages) that are held by one owner at a time.

The bookkeeping is on the host and is exact: a unit is either free or held; taking from an empty
pool and giving back a unit that is not held are errors, never silent.
"""
from __future__ import annotations


class PoolError(RuntimeError):
    pass


class Pool:
    def __init__(self, size: int, what: str = "unit"):
        if size < 0:
            raise ValueError(f"pool of {size} {what}s")
        self.size, self.what = int(size), what
        # last given back is first taken again, so that reuse happens soon and shows faults soon
        self._free = list(range(self.size - 1, -1, -1))
        self._held = [False] * self.size

    @property
    def free(self) -> int:
        return len(self._free)

    @property
    def held(self) -> int:
        return self.size - len(self._free)

    def is_held(self, unit: int) -> bool:
        return 0 <= unit < self.size and self._held[unit]

    def take(self) -> int:
        if not self._free:
            raise PoolError(f"no free {self.what} (all {self.size} are held)")
        unit = self._free.pop()
        self._held[unit] = True
        return unit

    def give_back(self, unit: int) -> None:
        if not 0 <= unit < self.size:
            raise PoolError(f"{self.what} {unit} does not exist (there are {self.size})")
        if not self._held[unit]:
            raise PoolError(f"{self.what} {unit} is given back but is not held")
        self._held[unit] = False
        self._free.append(unit)

    def check(self) -> None:
        """Every unit is free or held, none both, none twice."""
        if len(set(self._free)) != len(self._free):
            raise PoolError(f"a {self.what} is on the free list twice")
        for u in self._free:
            if self._held[u]:
                raise PoolError(f"{self.what} {u} is both free and held")
        if sum(self._held) + len(self._free) != self.size:
            raise PoolError(f"{self.what}s lost: {sum(self._held)} held + {len(self._free)} free != {self.size}")
