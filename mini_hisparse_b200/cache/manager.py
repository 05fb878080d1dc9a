"""The cache manager: page pools with a block table per request, and fixed-size state slots.

Cache entries (one per owning entry of the model's run order) are sorted into groups by what
they need.  Entries that need per-position memory in pages and whose needs compare equal form a
*page group*: one pool ``[entries, pages, *need.page_shape(page_size)]`` (for keys and values:
``[2, kv_heads, page_size, head_dim]``), one allocator, one block table per request, so a page
id is valid in every layer of the group.  Entries that
need a fixed-size state form a *state group*: a tensor ``[entries, slots, *shape]`` indexed by
the request's slot.  The reference has one homogeneous pool per (layer, page)
(mini_hisparse/allocator.py:18-22) and keeps per-request bookkeeping in
mini_hisparse/storage.py:177-212; its invariant checker (storage.py:415-441) is the model for
:meth:`assert_invariants`.

Pages are given back when a request closes and, in a windowed group, as soon as every key of a
page lies behind the window of all tokens still to come.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.spec import CacheNeed, PagedNeed, StateNeed
from .allocator import CapacityError, PageAllocator

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class CacheConfig:
    """Sizes of the cache that are not the model's: the reference's CacheConfig
    (mini_hisparse/config.py:12-30) without its host pool and index budget."""

    num_pages: int
    page_size: int = 16
    max_requests: int = 8
    max_pages_per_request: int | None = None
    dtype: torch.dtype = torch.bfloat16
    device: str = "cuda:0"
    allocate_storage: bool = True
    # Debugging aid: a page that is given back is overwritten with POISON in every layer, so that
    # a kernel that reads a stale page (through an old block-table entry, or beyond its keys)
    # produces numbers far outside anything a model computes instead of plausible ones.  The
    # value is finite on purpose: kernels load whole pages and multiply masked positions by
    # zero, which a NaN would survive.
    debug_poison: bool = False

    def __post_init__(self):
        for name in ("num_pages", "page_size", "max_requests"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be positive")
        if self.dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("KV dtype must be float32 or bfloat16")


POISON = 1.0e30


@dataclass
class _RequestPages:
    pages: list[int] = field(default_factory=list)   # logical page index -> page id or -1
    first_live: int = 0                               # logical pages below this were given back


class PageGroup:
    def __init__(self, gid: int, need: PagedNeed, entries: list[int], cfg: CacheConfig):
        self.gid, self.need, self.entries, self.cfg = gid, need, entries, cfg
        self.allocator = PageAllocator(cfg.num_pages)
        # the table is indexed by logical page: a full group never needs more entries than the
        # pool has pages; a windowed group gives pages back and can run far past the pool's size
        self.width = cfg.max_pages_per_request or cfg.num_pages
        if need.window is None:
            self.width = min(self.width, cfg.num_pages)
        self.tables: dict[int, _RequestPages] = {}       # slot -> pages
        # the block tables as one array [slot, logical page], -1 where no page is held; kept in
        # step with ``tables`` so that a step copies rows instead of walking Python lists
        self.table_np = np.full((cfg.max_requests, self.width), -1, np.int32)
        self.page_shape = tuple(int(n) for n in need.page_shape(cfg.page_size))
        shape = (len(entries), cfg.num_pages, *self.page_shape)
        self.storage = (
            torch.zeros(shape, dtype=cfg.dtype, device=cfg.device) if cfg.allocate_storage else None
        )
        self.poisoned = 0

    def give_back(self, owner, pages: list[int]) -> None:
        """Free pages; with debug_poison their old content is destroyed first (stream order makes
        that safe: kernels launched earlier have read them, later ones see the poison)."""
        if pages and self.cfg.debug_poison and self.storage is not None:
            index = torch.as_tensor(pages, dtype=torch.long, device=self.storage.device)
            self.storage.index_fill_(1, index, POISON)
            self.poisoned += len(pages)
        self.allocator.free(owner, pages)

    @property
    def window(self):
        return self.need.window

    def page_bytes(self) -> int:
        """Bytes of one page id: one page in every entry of the group."""
        n = 1
        for extent in self.page_shape:
            n *= extent
        return len(self.entries) * n * self.cfg.dtype.itemsize

    def pages_for(self, total_tokens: int, max_step_tokens: int | None = None) -> int:
        """Pages a request of total_tokens can hold at once."""
        P = self.cfg.page_size
        full = -(-total_tokens // P)
        if self.window is None:
            return full
        step = max_step_tokens or total_tokens
        return min(full, -(-(self.window + step) // P) + 2)


class StateGroup:
    def __init__(self, gid: int, need: StateNeed, entries: list[int], cfg: CacheConfig):
        self.gid, self.need, self.entries = gid, need, entries
        dtype = _TORCH_DTYPES[need.dtype]
        shape = (len(entries), cfg.max_requests, *need.shape)
        self.storage = torch.zeros(shape, dtype=dtype, device=cfg.device) if cfg.allocate_storage else None

    def zero_slot(self, slot: int):
        if self.storage is not None:
            self.storage[:, slot].zero_()


@dataclass
class _Request:
    slot: int
    length: int = 0
    reserved_tokens: int | None = None


class CacheManager:
    def __init__(self, needs: list[CacheNeed | None], cfg: CacheConfig):
        """``needs[i]`` is what cache entry i asks for (None: nothing)."""
        self.cfg = cfg
        self.page_groups: list[PageGroup] = []
        self.state_groups: list[StateGroup] = []
        self.entry_group: list[tuple[str, int, int] | None] = [None] * len(needs)
        by_need: dict[CacheNeed, list[int]] = {}
        for i, need in enumerate(needs):
            if need is not None:
                by_need.setdefault(need, []).append(i)
        for need, entries in by_need.items():
            if isinstance(need, PagedNeed):
                g = PageGroup(len(self.page_groups), need, entries, cfg)
                self.page_groups.append(g)
                for j, e in enumerate(entries):
                    self.entry_group[e] = ("pages", g.gid, j)
            elif isinstance(need, StateNeed):
                g = StateGroup(len(self.state_groups), need, entries, cfg)
                self.state_groups.append(g)
                for j, e in enumerate(entries):
                    self.entry_group[e] = ("state", g.gid, j)
            else:
                raise TypeError(f"unknown cache need {need!r}")
        self.requests: dict[object, _Request] = {}
        self._free_slots = list(range(cfg.max_requests - 1, -1, -1))
        self.stats = {"opened": 0, "closed": 0, "window_pages_freed": 0}

    # ---- requests -------------------------------------------------------------------------
    def can_ever_fit(self, total_tokens: int, max_step_tokens: int | None = None) -> bool:
        return all(
            g.pages_for(total_tokens, max_step_tokens) <= g.cfg.num_pages
            and -(-total_tokens // g.cfg.page_size) <= g.width
            for g in self.page_groups
        )

    def open(self, request, reserve_tokens: int | None = None, max_step_tokens: int | None = None) -> int:
        """Take a state slot (zeroed) and, if ``reserve_tokens`` is given, page credits for that many
        tokens in every page group.  Raises CapacityError with nothing changed."""
        if request in self.requests:
            raise ValueError(f"request {request!r} is already open")
        if not self._free_slots:
            raise CapacityError(f"all {self.cfg.max_requests} request slots are taken")
        if reserve_tokens is not None:
            wants = [g.pages_for(reserve_tokens, max_step_tokens) for g in self.page_groups]
            for g, n in zip(self.page_groups, wants):
                if n > g.width:
                    raise CapacityError(
                        f"request {request!r} needs {n} pages, more than a block table holds ({g.width})"
                    )
                if n > g.allocator.available_credits():
                    raise CapacityError(
                        f"request {request!r} needs {n} pages; {g.allocator.available_credits()} of "
                        f"{g.cfg.num_pages} are unpromised"
                    )
            for g, n in zip(self.page_groups, wants):
                g.allocator.reserve(request, n)
        slot = self._free_slots.pop()
        self.requests[request] = _Request(slot, 0, reserve_tokens)
        for g in self.page_groups:
            g.tables[slot] = _RequestPages()
        for g in self.state_groups:
            g.zero_slot(slot)
        self.stats["opened"] += 1
        return slot

    def length(self, request) -> int:
        return self.requests[request].length

    def slot(self, request) -> int:
        return self.requests[request].slot

    def ensure(self, request, new_length: int) -> None:
        """Make every position below new_length have a page in every group (all or nothing)."""
        req = self.requests[request]
        if req.reserved_tokens is not None and new_length > req.reserved_tokens:
            raise CapacityError(
                f"request {request!r} grows to {new_length} tokens but reserved {req.reserved_tokens}"
            )
        P = self.cfg.page_size
        need_pages = -(-new_length // P)
        plans = []
        for g in self.page_groups:
            rp = g.tables[req.slot]
            extra = need_pages - len(rp.pages)
            if need_pages > g.width:
                raise CapacityError(
                    f"request {request!r} needs {need_pages} pages, more than a block table holds ({g.width})"
                )
            plans.append((g, rp, max(0, extra)))
        got = []
        try:
            for g, rp, extra in plans:
                got.append((g, rp, g.allocator.alloc(request, extra)))
        except CapacityError:
            for g, rp, pages in got:
                g.allocator.free(request, pages)
            raise
        for g, rp, pages in got:
            if pages:
                g.table_np[req.slot, len(rp.pages): len(rp.pages) + len(pages)] = pages
            rp.pages.extend(pages)

    def has_pages(self, request, new_length: int) -> bool:
        """True if every position below new_length already has a page in every group."""
        req = self.requests[request]
        need_pages = -(-new_length // self.cfg.page_size)
        return all(len(g.tables[req.slot].pages) >= need_pages for g in self.page_groups)

    def advance(self, request, count: int) -> None:
        """The request's first ``length + count`` positions are now cached; windows move on."""
        req = self.requests[request]
        req.length += count
        P = self.cfg.page_size
        for g in self.page_groups:
            if g.window is None:
                continue
            # the next token (position req.length) sees keys > req.length - window
            first_needed = max(0, req.length - g.window + 1)
            rp = g.tables[req.slot]
            dead = min(first_needed // P, len(rp.pages))
            if dead > rp.first_live:
                pages = [p for p in rp.pages[rp.first_live:dead] if p >= 0]
                g.give_back(request, pages)
                for i in range(rp.first_live, dead):
                    rp.pages[i] = -1
                g.table_np[req.slot, rp.first_live:dead] = -1
                self.stats["window_pages_freed"] += len(pages)
                rp.first_live = dead

    def close(self, request) -> None:
        """Give back everything the request holds: pages, credits, block-table row, state slot."""
        req = self.requests.pop(request)
        for g in self.page_groups:
            rp = g.tables.pop(req.slot)
            g.table_np[req.slot, : len(rp.pages)] = -1
            g.give_back(request, [p for p in rp.pages if p >= 0])
            g.allocator.release_owner(request)
        self._free_slots.append(req.slot)
        self.stats["closed"] += 1

    # ---- views for the step function ----------------------------------------------------------
    def table_rows(self, gid: int, slots, width: int | None = None) -> np.ndarray:
        """Block-table rows [len(slots), width] int32 of the given slots, -1 where no page is held."""
        g = self.page_groups[gid]
        return g.table_np[np.asarray(slots, np.intp), : (width or g.width)]

    def entry_storage(self, entry: int):
        kind, gid, j = self.entry_group[entry]
        g = self.page_groups[gid] if kind == "pages" else self.state_groups[gid]
        return kind, g, (g.storage[j] if g.storage is not None else None)

    # ---- checks and numbers ----------------------------------------------------------------------
    def assert_invariants(self) -> None:
        live_slots = [r.slot for r in self.requests.values()]
        assert len(set(live_slots)) == len(live_slots), "two requests share a slot"
        assert not (set(live_slots) & set(self._free_slots)), "a live slot is in the free list"
        assert len(set(self._free_slots)) == len(self._free_slots), "a slot is twice in the free list"
        assert len(live_slots) + len(self._free_slots) == self.cfg.max_requests, "a slot is lost"
        for g in self.page_groups:
            g.allocator.assert_invariants()
            seen: dict[int, object] = {}
            for name, r in self.requests.items():
                rp = g.tables[r.slot]
                for p in rp.pages:
                    if p < 0:
                        continue
                    assert p not in seen, f"page {p} is in the tables of {seen[p]!r} and {name!r}"
                    seen[p] = name
                    assert g.allocator.owner_of(p) == name, f"page {p}: table and allocator disagree"
                assert all(p < 0 for p in rp.pages[: rp.first_live]), "a passed page is still mapped"
                row = g.table_np[r.slot]
                assert row[: len(rp.pages)].tolist() == rp.pages and (row[len(rp.pages):] == -1).all(), \
                    "the table array and the page lists differ"
                assert len(rp.pages) >= -(-r.length // self.cfg.page_size), "a cached position has no page"
            assert len(seen) == g.allocator.in_use, "the allocator holds pages that no table names"
            assert set(g.tables) == set(live_slots), "tables and live slots differ"

    def snapshot(self) -> dict:
        return {
            "requests_live": len(self.requests),
            "slots_free": len(self._free_slots),
            "page_groups": [
                {
                    "entries": len(g.entries),
                    "window": g.window,
                    "pages_total": g.cfg.num_pages,
                    "pages_free": g.allocator.free_pages,
                    "pages_peak": g.allocator.peak_in_use,
                    "pages_reused": g.allocator.reuses,
                    "pages_poisoned": g.poisoned,
                    "credits_available": g.allocator.available_credits(),
                    "page_bytes": g.page_bytes(),
                }
                for g in self.page_groups
            ],
            "state_groups": [
                {"entries": len(g.entries), "shape": list(g.need.shape), "dtype": g.need.dtype}
                for g in self.state_groups
            ],
            **self.stats,
        }
