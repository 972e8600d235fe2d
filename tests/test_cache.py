"""The page pool and the cache manager on the host: no page lost, held twice or freed twice,
under random orders of requests; mirrors the reference's tests/test_pages.py:6-50."""
import random

import pytest

from damendaemon_b200.cache import CacheManager, PageCapacityError, PagedKeyValues, PagePool, RequestState


def test_pool_lowest_first_and_last_freed_first_reused():
    pool = PagePool(6, 16)
    a = pool.take("a", 2)
    b = pool.take("b", 2)
    assert a == [0, 1] and b == [2, 3]
    pool.give_back("a", a)
    assert pool.take("c", 3) == [1, 0, 4]       # the freed ones first, last freed first
    pool.check()


def test_pool_refusals_change_nothing():
    pool = PagePool(4, 8)
    held = pool.take("a", 3)
    with pytest.raises(PageCapacityError):
        pool.take("b", 2)
    assert pool.free_pages == 1 and pool.held("b") == 0
    with pytest.raises(ValueError):
        pool.give_back("b", held[:1])           # not the owner
    with pytest.raises(ValueError):
        pool.give_back("a", [held[0], held[0]])  # twice in one call
    pool.give_back("a", held[:1])
    with pytest.raises(ValueError):
        pool.give_back("a", held[:1])           # freed twice
    with pytest.raises(ValueError):
        pool.give_back("a", [99])
    pool.check()
    for bad in ((0, 16), (4, 0), (4.0, 16)):
        with pytest.raises(ValueError):
            PagePool(*bad)


def test_promises_keep_room_for_admitted_requests():
    pool = PagePool(10, 16)
    pool.promise("a", 6)
    assert pool.unpromised_pages == 4
    with pytest.raises(PageCapacityError):
        pool.promise("b", 5)
    pool.promise("b", 4)
    assert pool.take("a", 6) and pool.take("b", 4)
    with pytest.raises(PageCapacityError):
        pool.take("a", 1)
    pool.give_back("a", [0])                    # a window passed page 0: a may take one again
    assert pool.unpromised_pages == 0 and pool.can_take("a", 1) and not pool.can_take("c", 1)


def manager(window=None, kv_tokens=256, page=16, requests=4, context=128):
    needs = [[PagedKeyValues(2, 16, None)], [PagedKeyValues(2, 16, None)]]
    if window:
        needs.append([PagedKeyValues(2, 16, window), RequestState((3, 5))])
    return CacheManager(needs, kv_tokens, page, requests, context)


def test_groups_by_need_and_block_tables():
    m = manager(window=24)
    assert [g.layers for g in m.groups] == [[0, 1], [2]]
    assert m.state_needs[2].shape == (3, 5)
    m.admit("a")
    m.extend([("a", 40)])
    assert m.groups[0].tables["a"] == [0, 1, 2] and m.groups[1].tables["a"] == [0, 1, 2]
    m.advance("a", 40)
    # window 24 at length 40: keys before 17 are gone, so block 0 (keys 0..15) went back
    assert m.groups[0].tables["a"] == [0, 1, 2] and m.groups[1].tables["a"] == [-1, 1, 2]
    assert m.groups[1].table_array[m.slot_of["a"]].tolist()[:4] == [-1, 1, 2, -1]
    m.extend([("a", 50)])
    assert m.groups[1].tables["a"] == [-1, 1, 2, 0]      # the page that was given back is used again
    m.check()
    m.release("a")
    m.release("a")                                         # a second release is harmless
    assert m.used_tokens == 0 and (m.groups[1].table_array == -1).all()
    m.check()


def test_bytes_needed_counts_every_group_and_the_state_rows():
    m = manager(window=24)        # 256 tokens: two layers of all keys, one windowed layer, 2 heads x 16, state 3 x 5 per request
    assert m.bytes_needed(2) == 3 * 256 * 2 * 2 * 16 * 2 + 4 * 15 * 4
    assert manager().bytes_needed(4) == 2 * 256 * 2 * 2 * 16 * 4


def test_extend_is_all_or_nothing():
    m = manager(kv_tokens=64)
    m.admit("a"), m.admit("b")
    m.extend([("a", 30)])
    with pytest.raises(PageCapacityError):
        m.extend([("a", 33), ("b", 32)])
    assert m.groups[0].tables["a"] == [0, 1] and m.groups[0].tables["b"] == []
    m.advance("a", 30)
    for bad in ([("zz", 1)], [("a", 31), ("a", 32)], [("a", 129)], [("b", 16), ("a", 3)]):
        with pytest.raises((ValueError, PageCapacityError)):
            m.extend(bad)
    m.check()
    with pytest.raises(ValueError):
        m.admit("a")
    m.admit("c"), m.admit("d")
    with pytest.raises(PageCapacityError):
        m.admit("e")


def test_reserve_never_fits_versus_wait():
    m = manager(kv_tokens=64, context=128)
    m.admit("a")
    with pytest.raises(ValueError, match="pool has"):
        m.reserve("a", 100, 16)
    m.reserve("a", 48, 16)
    m.admit("b")
    with pytest.raises(PageCapacityError):
        m.reserve("b", 32, 16)
    m.reserve("b", 16, 16)
    m.extend([("a", 48), ("b", 16)])
    m.check()


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 24])
def test_random_orders(seed, window):
    rng = random.Random(seed)
    m = manager(window=window, kv_tokens=160, requests=5, context=128)
    live, names = {}, iter(range(10 ** 6))
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 5:
            r = next(names)
            m.admit(r)
            live[r] = 0
        elif action < 0.75 and live:
            k = rng.randint(1, len(live))
            chosen = rng.sample(sorted(live), k)
            growth = [(r, min(128, live[r] + rng.choice((1, 1, 2, 7, 16, 33)))) for r in chosen]
            before = {g.name: {r: list(t) for r, t in g.tables.items()} for g in m.groups}
            try:
                m.extend(growth)
            except PageCapacityError:
                assert before == {g.name: {r: list(t) for r, t in g.tables.items()} for g in m.groups}
            else:
                for r, n in growth:
                    m.advance(r, n)
                    live[r] = n
        elif live:
            r = rng.choice(sorted(live))
            m.release(r)
            del live[r]
        m.check()
        for g in m.groups:
            for r, n in live.items():
                table = g.tables[r]
                first = g.first_needed_block(n)
                assert all(p >= 0 for p in table[first:g.pool.pages_for(n)]), "a needed page is missing"
                row = g.table_array[m.slot_of[r]]
                assert row[:len(table)].tolist() == table and (row[len(table):] == -1).all()
    for r in list(live):
        m.release(r)
    m.check()
    assert m.used_tokens == 0


def test_a_paged_need_of_a_mixers_own():
    """A need the manager has never heard of (one plane of compressed rows instead of keys and values): a frozen
    dataclass that says what a page looks like. It gets a group, an arena and block tables of its own, beside the
    keys and values of other layers, with no change to the manager."""
    import torch
    from dataclasses import dataclass
    from typing import Optional
    from damendaemon_b200.cache import PagedNeed

    @dataclass(frozen=True)
    class LatentRows(PagedNeed):
        width: int
        window: Optional[int] = None

        def page_shape(self, page_size):
            return (page_size, self.width)

        @property
        def label(self):
            return f"latent{self.width}"

    m = CacheManager([[PagedKeyValues(2, 16)], [LatentRows(24)], [LatentRows(24)], [LatentRows(24, window=20)]], 128, 8, 3, 64)
    assert [g.name for g in m.groups] == ["kv2x16.all", "latent24.all", "latent24.w20"]
    assert [g.layers for g in m.groups] == [[0], [1, 2], [3]]
    assert m.bytes_needed(2) == 16 * (1 * 2 * 2 * 8 * 16 + 2 * 8 * 24 + 1 * 8 * 24) * 2
    assert m.bytes_per_token(2) == (2 * 2 * 16 + 2 * 24 + 24) * 2
    m.allocate("cpu", torch.float32)
    assert m.groups[1].arena.shape == (2, 16, 8, 24) and m.layer_view(2).pages.shape == (16, 8, 24)
    assert m.layer_view(0).kv.shape == (16, 2, 2, 8, 16)
    m.admit("a")
    m.extend([("a", 30)])
    m.advance("a", 30)
    assert m.groups[1].tables["a"] == [0, 1, 2, 3] and m.groups[2].tables["a"] == [-1, 1, 2, 3]
    m.release("a")
    m.check()
    assert m.used_tokens == 0
    with pytest.raises(TypeError):
        CacheManager([[object()]], 128, 8, 3, 64)
