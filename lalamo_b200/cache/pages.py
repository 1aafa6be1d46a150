"""Host-side allocators: a pool of cache pages and a pool of state slots.

Both hand out small integers from a LIFO free list (a page or slot given back is the next one
handed out, so reuse happens early and shows faults early) and keep an ownership record that
makes the invariants checkable: nothing is lost, held twice or freed twice.
"""

from __future__ import annotations

__all__ = ["OutOfPages", "OutOfSlots", "PagePool", "SlotPool"]


class OutOfPages(RuntimeError):
    """The pool cannot supply the pages asked for.  Nothing was allocated."""

    def __init__(self, wanted: int, free: int, group: str = "") -> None:
        super().__init__(f"cache pool{' ' + group if group else ''}: {wanted} pages wanted, {free} free")
        self.wanted = wanted
        self.free = free


class OutOfSlots(RuntimeError):
    pass


class _IdPool:
    def __init__(self, count: int, what: str) -> None:
        if count < 0:
            raise ValueError(f"a pool cannot hold {count} {what}s")
        self._what = what
        self.count = count
        self._free = list(range(count - 1, -1, -1))  # pop() hands out 0 first
        self._held = [False] * count

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.count - len(self._free)

    def _take(self) -> int:
        index = self._free.pop()
        self._held[index] = True
        return index

    def _give_back(self, index: int) -> None:
        if not 0 <= index < self.count:
            raise ValueError(f"{self._what} {index} is outside the pool of {self.count}")
        if not self._held[index]:
            raise ValueError(f"{self._what} {index} is freed twice")
        self._held[index] = False
        self._free.append(index)

    def is_held(self, index: int) -> bool:
        return self._held[index]

    def check(self) -> None:
        """Raises if the free list and the ownership record disagree."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError(f"a {self._what} is on the free list twice")
        for index in range(self.count):
            if self._held[index] == (index in free):
                raise AssertionError(f"{self._what} {index} is {'held and free' if index in free else 'lost'}")


class PagePool(_IdPool):
    def __init__(self, num_pages: int, name: str = "") -> None:
        super().__init__(num_pages, "page")
        self.name = name

    def allocate(self, count: int) -> list[int]:
        """``count`` pages, or :class:`OutOfPages` with nothing taken."""
        if count > len(self._free):
            raise OutOfPages(count, len(self._free), self.name)
        return [self._take() for _ in range(count)]

    def release(self, pages: list[int]) -> None:
        for page in pages:
            self._give_back(page)


class SlotPool(_IdPool):
    def __init__(self, num_slots: int) -> None:
        super().__init__(num_slots, "slot")

    def allocate(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.count} state slots are in use")
        return self._take()

    def release(self, slot: int) -> None:
        self._give_back(slot)
