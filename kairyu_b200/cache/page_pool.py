"""Bookkeeping of which physical pages are free (kairyu/engine/core/pages.py:12-47).

Pages are handed out last-freed-first.  Page ids below ``reserved`` are never
handed out: page 0 is where padding rows of a replayed graph point.
"""

from __future__ import annotations

from typing import Iterable


class OutOfPages(MemoryError):
    pass


class PagePool:
    def __init__(self, num_pages: int, *, reserved: int = 0) -> None:
        if num_pages < 1 or reserved < 0 or reserved >= num_pages:
            raise ValueError(f"need num_pages >= 1 and 0 <= reserved < num_pages, got {num_pages}, {reserved}")
        self.num_pages = num_pages
        self.reserved = reserved
        self._free: list[int] = list(range(num_pages - 1, reserved - 1, -1))
        self._held: set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return len(self._held)

    @property
    def capacity(self) -> int:
        return self.num_pages - self.reserved

    def allocate(self, count: int) -> list[int]:
        if count < 0:
            raise ValueError(f"cannot allocate {count} pages")
        if count > len(self._free):
            raise OutOfPages(
                f"requested {count} pages but only {len(self._free)} of {self.capacity} are free"
            )
        pages = [self._free.pop() for _ in range(count)]
        self._held.update(pages)
        return pages

    def free(self, pages: Iterable[int]) -> None:
        page_list = list(pages)
        if len(set(page_list)) != len(page_list):
            raise ValueError(f"duplicate page ids in one free call: {page_list}")
        not_held = [page for page in page_list if page not in self._held]
        if not_held:
            raise ValueError(f"pages {not_held} are not held (freed twice, or never allocated)")
        for page in page_list:
            self._held.discard(page)
            self._free.append(page)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        if free & self._held:
            raise AssertionError(f"pages both free and held: {sorted(free & self._held)}")
        expected = set(range(self.reserved, self.num_pages))
        if free | self._held != expected:
            raise AssertionError(f"pages lost: {sorted(expected - free - self._held)}")
