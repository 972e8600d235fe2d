"""Host-side ownership of one pool of fixed-size cache pages. No tensors, no GPU.

Behaviour follows the reference's ``PagePool`` (damendaemon/pages.py:8-56): capacity =
tokens // page_size, lowest page ids first, freed pages reused last-in first-out, a
change that does not fit raises ``PageCapacityError`` before anything is mutated.
Added here: a request's page list may have holes (pages behind a window that were
given back), and promises, counts of pages a request may still claim, so that an
admitted request can never run dry in the middle of decoding.
"""
from __future__ import annotations


class PageCapacityError(Exception):
    """The pool cannot give the pages asked for right now; nothing was changed."""


class PagePool:
    def __init__(self, n_pages: int, page_size: int):
        if type(n_pages) is not int or type(page_size) is not int or n_pages <= 0 or page_size <= 0:
            raise ValueError("a page pool needs a positive page count and page size")
        self.n_pages, self.page_size = n_pages, page_size
        self._free = list(reversed(range(n_pages)))
        self._owner = [None] * n_pages            # owner key of each page, None when free
        self._promised = {}                       # owner -> pages promised in total
        self._held = {}                           # owner -> pages held now
        self.high_water_pages = 0

    # ---- accounting ----
    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def used_pages(self) -> int:
        return self.n_pages - len(self._free)

    @property
    def unpromised_pages(self) -> int:
        """Free pages that no admitted request has a claim on."""
        owed = sum(max(0, self._promised.get(o, 0) - self._held.get(o, 0)) for o in self._promised)
        return len(self._free) - owed

    def held(self, owner) -> int:
        return self._held.get(owner, 0)

    def pages_for(self, tokens: int) -> int:
        return (tokens + self.page_size - 1) // self.page_size

    # ---- promises ----
    def promise(self, owner, n_pages: int):
        """Set aside n_pages (in total, held ones included) for owner, or raise."""
        current = max(self._promised.get(owner, 0), self._held.get(owner, 0))
        extra = max(0, n_pages - current)
        if extra > self.unpromised_pages:
            raise PageCapacityError(f"{extra} more pages promised, {self.unpromised_pages} without a claim")
        self._promised[owner] = max(n_pages, self._promised.get(owner, 0))

    def can_take(self, owner, n_pages: int) -> bool:
        within = max(0, self._promised.get(owner, 0) - self._held.get(owner, 0))
        beyond = max(0, n_pages - within)
        return beyond <= self.unpromised_pages and n_pages <= len(self._free)

    # ---- pages ----
    def take(self, owner, n_pages: int) -> list:
        if n_pages < 0:
            raise ValueError("negative page count")
        if not self.can_take(owner, n_pages):
            raise PageCapacityError(f"{n_pages} pages asked for, {len(self._free)} free, "
                                    f"{self.unpromised_pages} without a claim")
        pages = [self._free.pop() for _ in range(n_pages)]
        for p in pages:
            self._owner[p] = owner
        self._held[owner] = self._held.get(owner, 0) + n_pages
        self.high_water_pages = max(self.high_water_pages, self.used_pages)
        return pages

    def give_back(self, owner, pages):
        pages = list(pages)
        for p in pages:
            if not 0 <= p < self.n_pages or self._owner[p] != owner:
                raise ValueError(f"page {p} is not held by {owner!r}")
        if len(set(pages)) != len(pages):
            raise ValueError("a page is given back twice")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)
        self._held[owner] = self._held.get(owner, 0) - len(pages)

    def forget(self, owner):
        """Drop owner's promise; it must hold no pages any more."""
        if self._held.get(owner, 0):
            raise ValueError(f"{owner!r} still holds pages")
        self._promised.pop(owner, None)
        self._held.pop(owner, None)

    def check(self):
        """Invariant: every page is either free once or held by one owner."""
        assert len(set(self._free)) == len(self._free), "a page is free twice"
        for p in self._free:
            assert self._owner[p] is None, f"free page {p} has an owner"
        held = {}
        for p, o in enumerate(self._owner):
            if o is not None:
                held[o] = held.get(o, 0) + 1
        assert len(self._free) + sum(held.values()) == self.n_pages, "a page was lost"
        for o, n in self._held.items():
            assert held.get(o, 0) == n, f"held count of {o!r} is off"
