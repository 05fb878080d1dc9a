"""The cache manager without a GPU: no page lost, held twice or freed twice, under random orders
of requests; windows give pages back; state slots; failures change nothing."""
import random

import pytest
import torch

from mini_hisparse_b200.cache import CacheConfig, CacheManager, CapacityError, PageAllocator
from mini_hisparse_b200.parts.spec import PagedKVNeed, StateNeed


def manager(num_pages=12, page_size=4, max_requests=4, needs=None, width=None):
    needs = needs or [PagedKVNeed(kv_heads=2, head_dim=16)] * 3
    cfg = CacheConfig(num_pages=num_pages, page_size=page_size, max_requests=max_requests,
                      max_pages_per_request=width, dtype=torch.float32, device="cpu",
                      allocate_storage=False)
    return CacheManager(needs, cfg)


def test_allocator_all_or_nothing_and_double_free():
    a = PageAllocator(4)
    got = a.alloc("x", 3)
    assert sorted(got) == [0, 1, 2] and a.free_pages == 1
    with pytest.raises(CapacityError):
        a.alloc("y", 2)
    assert a.free_pages == 1 and a.held("y") == 0       # nothing changed
    a.free("x", got[:1])
    with pytest.raises(ValueError, match="twice"):
        a.free("x", got[:1])
    with pytest.raises(ValueError, match="belongs"):
        a.free("y", got[1:2])
    again = a.alloc("y", 1)
    assert again == got[:1] and a.reuses == 1           # the page just freed is used again at once
    a.assert_invariants()


def test_reservations_hold_pages_for_their_owner():
    a = PageAllocator(10)
    a.reserve("x", 6)
    assert a.available_credits() == 4
    with pytest.raises(CapacityError):
        a.reserve("y", 5)
    a.reserve("y", 4)
    with pytest.raises(CapacityError):
        a.alloc("z", 1)                                  # every free page is promised
    a.alloc("x", 6)
    a.alloc("y", 4)
    with pytest.raises(CapacityError):
        a.alloc("x", 1)                                  # beyond its reservation, nothing free
    a.assert_invariants()


def test_groups_by_need_and_state_slots():
    full = PagedKVNeed(kv_heads=2, head_dim=16)
    win = PagedKVNeed(kv_heads=2, head_dim=16, window=8)
    state = StateNeed(shape=(5,), dtype="float32")
    m = manager(needs=[full, win, full, state, None, win])
    assert len(m.page_groups) == 2 and len(m.state_groups) == 1
    assert m.entry_group[0][:2] == m.entry_group[2][:2] and m.entry_group[0][2] != m.entry_group[2][2]
    assert m.entry_group[1][1] == m.entry_group[5][1] != m.entry_group[0][1]
    assert m.entry_group[3][0] == "state" and m.entry_group[4] is None


def test_window_pages_come_back_and_are_used_again():
    win = PagedKVNeed(kv_heads=1, head_dim=16, window=8)
    m = manager(num_pages=5, page_size=4, needs=[win], width=16)
    m.open("a")
    held = []
    for step in range(40):                    # 40 tokens through a pool of 5 pages (20 tokens)
        n = m.length("a")
        m.ensure("a", n + 1)
        m.advance("a", 1)
        m.assert_invariants()
        held.append(m.page_groups[0].allocator.in_use)
    assert max(held) <= 4 and m.stats["window_pages_freed"] >= 6
    assert m.page_groups[0].allocator.reuses > 0
    row = m.table_rows(0, [m.slot("a")], 10)[0]
    assert (row[: (40 - 8 + 1) // 4] == -1).all() and (row[8:10] >= 0).all()
    m.close("a")
    assert m.page_groups[0].allocator.free_pages == 5


def test_open_failure_changes_nothing():
    m = manager(num_pages=6, page_size=4, max_requests=2)
    m.open("a", reserve_tokens=16)
    with pytest.raises(CapacityError):
        m.open("b", reserve_tokens=12)          # 3 pages wanted, 2 unpromised
    assert "b" not in m.requests and len(m._free_slots) == 1
    m.open("b", reserve_tokens=8)
    with pytest.raises(CapacityError, match="slots"):
        m.open("c")
    m.ensure("a", 16)
    with pytest.raises(CapacityError, match="reserved"):
        m.ensure("a", 17)
    m.assert_invariants()


def test_ensure_is_all_or_nothing_across_groups():
    full = PagedKVNeed(kv_heads=2, head_dim=16)
    other = PagedKVNeed(kv_heads=1, head_dim=32)
    m = manager(num_pages=4, page_size=4, needs=[full, other])
    m.open("a")
    m.open("b")
    m.ensure("a", 12)
    m.page_groups[1].allocator.alloc("b", 1)       # the second group has no page left for "b"...
    m.page_groups[1].tables[m.slot("b")].pages.append(3)
    before = [g.allocator.free_pages for g in m.page_groups]
    with pytest.raises(CapacityError):
        m.ensure("b", 8)                            # ...group 0 could serve it, group 1 cannot
    assert [g.allocator.free_pages for g in m.page_groups] == before


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    full = PagedKVNeed(kv_heads=2, head_dim=16)
    win = PagedKVNeed(kv_heads=2, head_dim=16, window=6)
    m = manager(num_pages=10, page_size=4, max_requests=3, needs=[full, win, full, StateNeed((3,))], width=64)
    live, names = {}, iter(range(10_000))
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 3:
            name = f"r{next(names)}"
            try:
                m.open(name, reserve_tokens=rng.choice([None, 8, 20]))
                live[name] = 0
            except CapacityError:
                pass
        elif op < 0.85 and live:
            name = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 9])
            try:
                m.ensure(name, live[name] + n)
                m.advance(name, n)
                live[name] += n
            except CapacityError:
                pass
        elif live:
            name = rng.choice(list(live))
            m.close(name)
            del live[name]
        m.assert_invariants()
        for name, n in live.items():
            assert m.length(name) == n
            row = m.table_rows(0, [m.slot(name)], 10)[0]
            assert (row[: -(-n // 4)] >= 0).all()     # the full group maps every cached position
    for name in list(live):
        m.close(name)
    m.assert_invariants()
    assert all(g.allocator.free_pages == 10 for g in m.page_groups)
    assert m.page_groups[0].allocator.reuses > 0
