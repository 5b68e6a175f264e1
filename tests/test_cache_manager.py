"""The cache manager on the host: no page is lost, held twice or freed twice, under random
orders of requests; windows give pages back; reserving is all or nothing; state slots."""
import random

import pytest
import torch

from wllm_b200.cache import CacheGroupSpec, CacheManager, OutOfPages, PagePool, StateSpec


def manager(pages=8, page_size=4, window=None, max_requests=4, states=(), device=None, groups=None):
    groups = groups or [CacheGroupSpec("all", 2, 1, 8, window)]
    return CacheManager(groups, page_size, pages, max_requests, states, torch.float32, device)


def test_pool_is_a_stack_and_guards_double_free():
    p = PagePool(3)
    a, b = p.take(), p.take()
    assert (a, b) == (0, 1)
    p.give(a)
    assert p.take() == a            # the page given back last is taken first
    p.give(b)
    with pytest.raises(RuntimeError, match="freed twice"):
        p.give(b)
    p.take(), p.take()
    with pytest.raises(OutOfPages):
        p.take()


def test_pages_grow_at_page_edges_and_come_back_on_close():
    m = manager()
    r = m.open("a")
    m.reserve([(r, 4)]); m.commit(r, 4)
    assert len(r.tables[0]) == 1
    m.reserve([(r, 1)]); m.commit(r, 1)
    assert len(r.tables[0]) == 2 and m.free_pages() == [6]
    assert m.token_slots(r, 0, 3, 2) == [r.tables[0][0] * 4 + 3, r.tables[0][1] * 4]
    m.close(r)
    assert m.free_pages() == [8]
    with pytest.raises(RuntimeError, match="closed twice"):
        m.close(r)
    m.check()


def test_reserve_is_all_or_nothing():
    m = manager(pages=4)
    a, b = m.open("a"), m.open("b")
    m.reserve([(a, 8)]); m.commit(a, 8)          # 2 pages
    before = ([list(t) for t in a.tables], [list(t) for t in b.tables], m.free_pages())
    with pytest.raises(OutOfPages) as e:
        m.reserve([(a, 4), (b, 8)])              # needs 1 + 2 > 2 free
    assert e.value.needed == 3 and e.value.free == 2
    assert ([list(t) for t in a.tables], [list(t) for t in b.tables], m.free_pages()) == before
    assert a.reserved == 0 and b.reserved == 0
    m.reserve([(a, 4), (b, 4)])
    m.check()


def test_cancelled_reservation_returns_surplus_pages():
    m = manager()
    r = m.open("a")
    m.reserve([(r, 3)]); m.commit(r, 3)
    m.reserve([(r, 9)])
    assert m.free_pages() == [5]
    m.cancel_reservation(r)
    assert m.free_pages() == [7] and r.reserved == 0 and r.num_tokens == 3
    m.check()


def test_window_group_gives_back_pages_it_has_passed():
    m = manager(pages=6, page_size=4, window=6)
    r = m.open("a")
    for _ in range(30):
        m.reserve([(r, 1)]); m.commit(r, 1)
        m.check()
        first_needed = r.num_tokens - 6 + 1           # oldest key the next token reads
        for i, page in enumerate(r.tables[0]):
            assert (page == -1) == ((i + 1) * 4 <= first_needed)
    held = sum(p >= 0 for p in r.tables[0])
    assert held <= 3 and m.free_pages() == [6 - held] and m.groups[0].pool.takes > 6
    m.close(r)
    assert m.free_pages() == [6]


def test_groups_have_pools_and_tables_of_their_own():
    groups = [CacheGroupSpec("all", 2, 1, 8, None), CacheGroupSpec("win", 1, 2, 16, 4)]
    m = manager(pages=5, page_size=4, groups=groups)
    r = m.open("a")
    m.reserve([(r, 12)]); m.commit(r, 12)
    assert [p >= 0 for p in r.tables[0]] == [True] * 3 and [p >= 0 for p in r.tables[1]] == [False, False, True]
    assert m.free_pages() == [2, 4]
    with pytest.raises(OutOfPages) as e:
        m.reserve([(r, 12)])
    assert e.value.group == "all"


def test_state_slots_are_zeroed_and_reused():
    m = manager(max_requests=2, states=[StateSpec("s", (3,), torch.float32)], device="cpu")
    a = m.open("a")
    m.slots.tensors["s"][a.slot] += 5
    b = m.open("b")
    with pytest.raises(OutOfPages, match="request slots"):
        m.open("c")
    m.close(a)
    c = m.open("c")
    assert c.slot == a.slot and float(m.slots.tensors["s"][c.slot].abs().sum()) == 0.0
    with pytest.raises(KeyError):
        m.open("b")
    m.close(b); m.close(c)
    assert m.slots.num_free == 2


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("window", [None, 10])
def test_random_orders_lose_nothing(seed, window):
    rng = random.Random(seed)
    m = manager(pages=12, page_size=4, window=window, max_requests=5)
    live, n_open = {}, 0
    for _ in range(400):
        act = rng.random()
        if act < 0.25 and len(live) < 5:
            live[n_open] = m.open(n_open)
            n_open += 1
        elif act < 0.85 and live:
            picks = rng.sample(sorted(live), k=rng.randint(1, len(live)))
            wants = [(live[i], rng.randint(1, 9)) for i in picks]
            free_before = m.free_pages()
            try:
                m.reserve(wants)
            except OutOfPages:
                assert m.free_pages() == free_before
                if rng.random() < 0.5:                       # as the scheduler does: drop the youngest
                    m.close(live.pop(max(live)))
                continue
            for rc, n in wants:
                if rng.random() < 0.1:
                    m.cancel_reservation(rc)
                else:
                    m.commit(rc, n)
        elif live:
            m.close(live.pop(rng.choice(sorted(live))))
        m.check()
    for rc in live.values():
        m.close(rc)
    m.check()
    assert m.free_pages() == [12] and m.slots.num_free == 5
