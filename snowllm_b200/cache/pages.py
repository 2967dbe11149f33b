"""Page and slot pools: free lists with ownership checks
(the role of BlockAllocator and StateSlots, snowllm/engine/block_manager.py:107-177).

A page is held by whoever took it until it is released; releasing a page that is free, or one
this pool never gave out, is a bug in the caller and raises.  Pages come back in LIFO order, so
a page that was just given back is the next one handed out: reuse shows up at once in tests."""
from __future__ import annotations

from ..errors import CapacityError


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must not be negative")
        self.total = num_pages
        self._free = list(range(num_pages - 1, -1, -1))     # pop() gives page 0 first
        self._refs = [0] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> list[int] | None:
        """n pages, or None (and nothing taken) when fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._refs[p] = 1
        return pages

    def retain(self, pages) -> None:
        for p in pages:
            if self._refs[p] <= 0:
                raise CapacityError(f"page {p} is free and cannot be shared")
            self._refs[p] += 1

    def release(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.total:
                raise CapacityError(f"page {p} does not belong to this pool")
            if self._refs[p] <= 0:
                raise CapacityError(f"page {p} is freed twice")
            self._refs[p] -= 1
            if self._refs[p] == 0:
                self._free.append(p)

    def held(self) -> int:
        return self.total - len(self._free)


class StateSlots:
    """Slots for per-request state of fixed size; one extra slot (index ``count``) is never
    handed out and serves padding rows."""

    def __init__(self, count: int):
        self.count = count
        self._free = list(range(count - 1, -1, -1))
        self._taken = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def dummy(self) -> int:
        return self.count

    def alloc(self) -> int | None:
        if not self._free:
            return None
        s = self._free.pop()
        self._taken[s] = True
        return s

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.count or not self._taken[slot]:
            raise CapacityError(f"slot {slot} is freed twice or was never taken")
        self._taken[slot] = False
        self._free.append(slot)
