"""Block allocator of one page pool.

The reference tracks a ``free`` set, an owner and a generation per device slot and refuses
stale handles (mini_hisparse/allocator.py:16-66); whole lifetimes are reserved at admission so
that a running request never runs out (mini_hisparse/engine.py:53-55, 91-95;
mini_hisparse/storage.py:177-212).  This allocator keeps those guarantees for a pool whose
pages are valid in every layer of a group: a LIFO free list (a page just given back is the
next one handed out, so reuse is exercised early), an owner per page, all-or-nothing
allocation, and page credits that admission reserves.
"""
from __future__ import annotations


class CapacityError(RuntimeError):
    """Not enough pages, credits or slots; nothing was changed."""


class PageAllocator:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("num_pages must be positive")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))  # pop() hands out page 0 first
        self._owner: list[object | None] = [None] * num_pages
        self.generation = [0] * num_pages
        self._reserved: dict[object, int] = {}    # owner -> credits reserved
        self._held: dict[object, int] = {}        # owner -> pages held now
        self.peak_in_use = 0
        self.allocations = 0
        self.reuses = 0

    # ---- credits ------------------------------------------------------------------
    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def in_use(self) -> int:
        return self.num_pages - len(self._free)

    def _promised(self) -> int:
        """Pages that reservations may still claim beyond what their owners already hold."""
        return sum(max(0, r - self._held.get(o, 0)) for o, r in self._reserved.items())

    def available_credits(self) -> int:
        return len(self._free) - self._promised()

    def reserve(self, owner, pages: int) -> None:
        if owner in self._reserved:
            raise ValueError(f"{owner!r} already holds a reservation")
        if pages > self.available_credits():
            raise CapacityError(
                f"cannot reserve {pages} pages for {owner!r}: {self.available_credits()} of "
                f"{self.num_pages} are unpromised"
            )
        self._reserved[owner] = pages

    # ---- pages ----------------------------------------------------------------------
    def alloc(self, owner, n: int) -> list[int]:
        """n pages for owner, or CapacityError with nothing changed."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        held = self._held.get(owner, 0)
        reserved = self._reserved.get(owner)
        if reserved is not None and held + n <= reserved:
            pass  # inside its reservation: the credits were set aside at admission
        else:
            inside = max(0, (reserved or 0) - held)
            if n - inside > self.available_credits():
                raise CapacityError(
                    f"{owner!r} needs {n} more pages; {self.available_credits()} of "
                    f"{self.num_pages} are free and unpromised"
                )
        if n > len(self._free):
            raise CapacityError(f"{owner!r} needs {n} pages; {len(self._free)} are free")
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            assert self._owner[p] is None, f"page {p} handed out twice"
            self._owner[p] = owner
            if self.generation[p]:
                self.reuses += 1
            self.generation[p] += 1
        self._held[owner] = held + n
        self.allocations += n
        self.peak_in_use = max(self.peak_in_use, self.in_use)
        return pages

    def free(self, owner, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is outside the pool")
            if self._owner[p] is None:
                raise ValueError(f"page {p} freed twice")
            if self._owner[p] != owner:
                raise ValueError(f"page {p} belongs to {self._owner[p]!r}, not to {owner!r}")
        if len(set(pages)) != len(pages):
            raise ValueError("a page is named twice in one free")
        for p in pages:
            self._owner[p] = None
            self._free.append(p)
        if pages:
            self._held[owner] -= len(pages)

    def release_owner(self, owner) -> None:
        """Drop the owner's reservation; it must hold no pages any more."""
        if self._held.get(owner, 0):
            raise ValueError(f"{owner!r} still holds {self._held[owner]} pages")
        self._held.pop(owner, None)
        self._reserved.pop(owner, None)

    def owner_of(self, page: int):
        return self._owner[page]

    def held(self, owner) -> int:
        return self._held.get(owner, 0)

    # ---- checks ------------------------------------------------------------------------
    def assert_invariants(self) -> None:
        free = set(self._free)
        assert len(free) == len(self._free), "a page is twice in the free list"
        owned = {p for p, o in enumerate(self._owner) if o is not None}
        assert not (free & owned), f"pages both free and owned: {sorted(free & owned)}"
        assert free | owned == set(range(self.num_pages)), "a page is lost"
        counts: dict[object, int] = {}
        for o in self._owner:
            if o is not None:
                counts[o] = counts.get(o, 0) + 1
        for o, n in self._held.items():
            assert counts.get(o, 0) == n, f"{o!r}: holds {counts.get(o, 0)} pages, book says {n}"
        assert self._promised() <= len(self._free), "more pages promised than free"
