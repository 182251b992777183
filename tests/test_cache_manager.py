"""The page pool and the cache manager: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; state slots."""

import random

import pytest

from kairyu_b200.cache import CacheLayout, CacheManager, OutOfPages, PagePool
from kairyu_b200.parts.base import PagedKVSpec, StateSpec


def test_page_pool_basics():
    pool = PagePool(6, reserved=1)
    assert pool.capacity == 5 and pool.num_free == 5
    pages = pool.allocate(3)
    assert len(set(pages)) == 3 and 0 not in pages
    with pytest.raises(OutOfPages):
        pool.allocate(3)
    pool.free(pages[:2])
    with pytest.raises(ValueError, match="not held"):
        pool.free(pages[:1])  # freed twice
    with pytest.raises(ValueError, match="duplicate"):
        pool.free([pages[2], pages[2]])
    with pytest.raises(ValueError, match="not held"):
        pool.free([0])  # the reserved page is never held
    # last freed, first handed out again
    assert pool.allocate(1)[0] == pages[1]
    pool.check()
    with pytest.raises(ValueError):
        PagePool(1, reserved=1)


def layout(window=None, state=False):
    full = (PagedKVSpec(2, 16),)
    slots = {0: full, 1: full}
    if window is not None:
        slots[2] = (PagedKVSpec(2, 16, window=window),)
        slots[3] = (PagedKVSpec(2, 16, window=window),)
    if state:
        slots[4] = (StateSpec((3, 5)),)
    return CacheLayout.from_slot_specs(slots)


def test_layout_groups_slots_by_their_needs():
    plan = layout(window=20, state=True)
    assert [g.slots for g in plan.groups] == [(0, 1), (2, 3)]
    assert plan.groups[0].spec.window is None and plan.groups[1].spec.window == 20
    assert plan.group_of_slot == {0: 0, 1: 0, 2: 1, 3: 1}
    assert [(b.slot, b.spec.shape) for b in plan.states] == [(4, (3, 5))]


def test_grow_advance_release():
    cache = CacheManager(layout(), num_pages=9, page_size=4, max_requests=3)
    cache.admit("a")
    assert cache.ensure_capacity("a", 10)
    assert len(cache.block_table("a", 0)) == 3 and cache.free_pages() == 5
    assert cache.ensure_capacity("a", 10)  # idempotent
    assert cache.free_pages() == 5
    cache.advance("a", 10)
    assert cache.ensure_capacity("a", 13) and cache.free_pages() == 4
    cache.admit("b")
    assert not cache.ensure_capacity("b", 17)  # 5 pages wanted, 4 free: nothing changes
    assert cache.block_table("b", 0) == [] and cache.free_pages() == 4
    cache.check()
    cache.release("a")
    assert cache.ensure_capacity("b", 17)
    cache.check()
    with pytest.raises(ValueError):
        cache.admit("b")
    with pytest.raises(ValueError):
        cache.advance("b", -1)
    cache.release("b")
    assert cache.free_pages() == 8 and cache.live_requests == 0


def test_request_slots_run_out_and_come_back():
    cache = CacheManager(layout(state=True), num_pages=9, page_size=4, max_requests=2)
    a = cache.admit("a").state_slot
    b = cache.admit("b").state_slot
    assert {a, b} == {0, 1}
    assert sorted(cache.take_fresh_state_slots()) == [0, 1] and cache.take_fresh_state_slots() == []
    with pytest.raises(OutOfPages):
        cache.admit("c")
    cache.release("a")
    assert cache.admit("c").state_slot == a
    assert cache.take_fresh_state_slots() == [a]  # a slot that changes hands is zeroed again
    cache.check()


def test_window_group_gives_pages_back_as_it_moves():
    cache = CacheManager(layout(window=10), num_pages=40, page_size=4, max_requests=2)
    cache.admit("a")
    position = 0
    held_window = []
    for chunk in (7, 9, 1, 1, 30, 2, 1, 1, 1, 25):
        assert cache.ensure_capacity("a", position + chunk, query_start=position)
        full, window = cache.block_table("a", 0), cache.block_table("a", 1)
        # every key a query of this chunk can see has a page
        for query in range(position, position + chunk):
            for key in range(max(0, query - 10 + 1), query + 1):
                assert window[key // 4] >= 0
                assert full[key // 4] >= 0
        position += chunk
        cache.advance("a", position)
        held_window.append(sum(1 for page in window if page >= 0))
        cache.check()
    # the full group holds everything, the window group only what later queries can read
    assert sum(1 for page in cache.block_table("a", 0) if page >= 0) == -(-position // 4)
    assert held_window[-1] <= 10 // 4 + 2
    assert cache.free_pages(1) > cache.free_pages(0)
    cache.release("a")
    assert cache.free_pages(0) == cache.free_pages(1) == 39


def test_can_hold():
    cache = CacheManager(layout(window=8), num_pages=5, page_size=4, max_requests=2)
    assert cache.can_hold(16)
    assert not cache.can_hold(17)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = random.Random(seed)
    cache = CacheManager(layout(window=rng.choice([None, 6, 21]), state=True), num_pages=30, page_size=rng.choice([1, 4, 16]), max_requests=5)
    live: dict[str, int] = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            name = f"r{counter}"
            counter += 1
            cache.admit(name)
            live[name] = 0
        elif action < 0.8 and live:
            name = rng.choice(sorted(live))
            grow = rng.choice([1, 1, 1, 2, 5, 17])
            if cache.ensure_capacity(name, live[name] + grow, query_start=live[name]):
                live[name] += grow
                cache.advance(name, live[name])
        elif live:
            name = rng.choice(sorted(live))
            cache.release(name)
            del live[name]
        cache.check()
        cache.take_fresh_state_slots()
    for name in list(live):
        cache.release(name)
    cache.check()
    assert all(pool.num_held == 0 for pool in cache.pools)


def test_values_may_be_narrower_than_keys_and_get_pages_of_their_own_shape():
    """A mixer describes what it keeps: keys of one width, values of another.  Slots whose needs
    are equal share a group (one geometry, one block table); the storage gives K and V their own shapes."""
    import torch

    from kairyu_b200.cache import CacheStorage

    narrow = PagedKVSpec(2, 24, None, v_head_dim=8)
    layout = CacheLayout.from_slot_specs({0: (PagedKVSpec(2, 16),), 1: (narrow,), 2: (narrow,)})
    assert [group.slots for group in layout.groups] == [(0,), (1, 2)]
    storage = CacheStorage(layout, num_pages=5, page_size=4, max_requests=2, dtype=torch.float32, device="cpu")
    assert tuple(storage.k[1].shape) == (2, 5, 4, 2, 24) and tuple(storage.v[1].shape) == (2, 5, 4, 2, 8)
    view = storage.view(2, writes=True)
    assert tuple(view.k.shape) == (5, 4, 2, 24) and tuple(view.v.shape) == (5, 4, 2, 8) and view.group == 1
    assert CacheStorage.bytes_per_page(layout, 4, 4) == 4 * 2 * 4 * (2 * 16 + 2 * (24 + 8))
