"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; windows give pages back; state slots are reused and zeroed."""
import random

import pytest
import torch

from tinyinfer_b200.cache import CacheManager, IdPool, OutOfPages, RELEASED
from tinyinfer_b200.parts import FixedStateSpec, PagedKVSpec

FULL = PagedKVSpec(2, 16, None)
WIN = PagedKVSpec(2, 16, 24)


def test_id_pool_refuses_double_free_and_exhaustion():
    p = IdPool(3)
    a, b, c = p.take(), p.take(), p.take()
    assert {a, b, c} == {0, 1, 2} and p.num_free == 0
    with pytest.raises(OutOfPages):
        p.take()
    p.give_back(b)
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back(b)
    assert p.take() == b                        # the page just given back is reused first
    p.check()


def test_groups_follow_the_mixers_needs():
    m = CacheManager([FULL, WIN, FULL, WIN, None, FixedStateSpec((4,))], page_size=16,
                     num_pages=10, max_requests=4)
    assert len(m.groups) == 2
    assert m.groups[0].cache_slots == [0, 2] and m.groups[1].cache_slots == [1, 3]
    assert m.group_of_slot(4) is None and m.group_of_slot(3) == 1


def test_append_is_all_or_nothing():
    m = CacheManager([FULL, WIN], page_size=16, num_pages=4, max_requests=4)
    m.reserve_step([("a", 40)])                 # 3 pages in each group
    assert m.free_pages() == [1, 1]
    with pytest.raises(OutOfPages):
        m.reserve_step([("a", 9), ("b", 17)])   # a needs 1, b needs 2: nothing may change
    assert m.free_pages() == [1, 1] and m.length("a") == 40 and not m.has_request("b")
    m.check()
    with pytest.raises(ValueError, match="twice"):
        m.reserve_step([("a", 1), ("a", 1)])
    with pytest.raises(ValueError, match="allows"):
        m.reserve_step([("a", 1)], max_position=40)


def test_window_gives_pages_back_behind_it():
    m = CacheManager([FULL, WIN], page_size=16, num_pages=64, max_requests=2)
    m.reserve_step([("a", 100)])
    assert m.release_passed("a") == 4           # next token 100 reads keys >= 77: blocks 0..3 go
    assert m.block_table(1, "a")[:5] == [RELEASED] * 4 + [m.block_table(1, "a")[4]]
    assert RELEASED not in m.block_table(0, "a")
    assert m.free_pages() == [64 - 7, 64 - 3]
    for _ in range(60):
        m.reserve_step([("a", 1)])
        m.release_passed("a")
        m.check()
    assert m.free_pages()[1] >= 64 - 3          # the window never holds more than 3 pages
    m.free_request("a")
    assert m.free_pages() == [64, 64]
    m.check()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = CacheManager([FULL, WIN, FULL], page_size=16, num_pages=40, max_requests=5)
    live = {}
    for step in range(400):
        action = rng.random()
        if action < 0.15 and live:
            r = rng.choice(list(live))
            m.free_request(r)
            del live[r]
        else:
            items = []
            for r in rng.sample(list(live), k=min(len(live), rng.randint(0, 3))):
                items.append((r, rng.choice([1, 1, 1, 2, 7, 30])))
            if rng.random() < 0.3 and len(live) + 1 <= 5:
                items.append((f"r{step}", rng.randint(1, 90)))
            if not items:
                continue
            before = (m.free_pages(), {r: m.length(r) for r in live})
            try:
                starts = m.reserve_step(items)
            except OutOfPages:
                assert (m.free_pages(), {r: m.length(r) for r in live}) == before
                if live:                                  # make room as a scheduler would
                    r = rng.choice(list(live))
                    m.free_request(r)
                    del live[r]
                continue
            for (r, n), s in zip(items, starts):
                assert s == live.get(r, 0)
                live[r] = s + n
                m.release_passed(r)
        m.check()
        for g in m.groups:                                # every readable position has a page
            for r, length in live.items():
                table = g.tables[r]
                assert len(table) == -(-length // 16)
                first = g.first_needed_block(length)
                assert all(p != RELEASED for p in table[first:])
    for r in list(live):
        m.free_request(r)
    m.check()
    assert m.free_pages() == [40, 40] and m.state_slots.num_free == 5


def test_state_slots_are_zeroed_on_reuse():
    m = CacheManager([FixedStateSpec((3,)), FULL], page_size=16, num_pages=4, max_requests=2,
                     kv_dtype=torch.float32, device="cpu")
    m.add_request("a")
    view = m.view(0, True, [], torch.tensor([m.state_slot("a")]))
    view.state[m.state_slot("a")] = 7.0
    slot = m.state_slot("a")
    m.free_request("a")
    m.add_request("b")
    assert m.state_slot("b") == slot and not view.state[slot].any()
    m.add_request("c")
    with pytest.raises(OutOfPages, match="state slot"):
        m.add_request("d")
    with pytest.raises(KeyError):
        m.free_request("zzz")
    m.check()
    # paged views carry the group's table and this layer's pages (one more page than the pool)
    pv = m.view(1, False, ["table"], None)
    assert pv.pages.shape == (5, 2, 2, 16, 16) and pv.block_table == "table" and not pv.writes
