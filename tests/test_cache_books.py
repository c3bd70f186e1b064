"""The cache manager's books: pages, block tables, windows, slots (no GPU)."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from cajeta_llm_b200.cache.manager import CacheManager
from cajeta_llm_b200.cache.pages import CacheBooks, CacheError, GroupSpec, PageAllocator
from cajeta_llm_b200.parts.base import KvNeed, StateNeed


def test_allocator_refuses_double_free_and_exhaustion():
    a = PageAllocator(3)
    p = a.take(2)
    assert a.take(2) is None and a.free_count == 1          # all or nothing
    a.give_back(p)
    with pytest.raises(CacheError, match="freed twice"):
        a.give_back([p[0]])
    a.check()


def books(pages=8, window=0, page_tokens=4, max_seqs=3, ctx=64):
    groups = [GroupSpec(2, 16, 0)] + ([GroupSpec(2, 16, window)] if window else [])
    return CacheBooks(groups, [pages] * len(groups), page_tokens, max_seqs, ctx)


def test_page_drawn_only_at_a_boundary_and_released_pages_are_reused():
    b = books()
    s = b.admit()
    assert b.pages_needed(s, 4) == [1] and b.reserve(s, 4)
    b.commit(s, 4)
    assert b.pages_needed(s, 1) == [1]                       # position 4 opens page 1
    assert b.reserve(s, 1)
    b.commit(s, 1)
    assert b.pages_needed(s, 3) == [0]                       # positions 5..7 stay in page 1
    held = b.groups[0].held_pages(s)
    b.release(s)
    assert b.free_pages() == [8]
    s2 = b.admit()
    assert b.length[s2] == 0                                 # a recycled slot starts at position 0
    b.reserve(s2, 8)
    assert set(b.groups[0].held_pages(s2)) & set(held)      # the freed pages are used again
    b.check()


def test_reserve_is_all_or_nothing_across_groups():
    b = CacheBooks([GroupSpec(2, 16, 0), GroupSpec(1, 8, 0)], [4, 2], 4, 2, 64)
    s = b.admit()
    assert not b.reserve(s, 12)                              # group 1 has only 2 pages
    assert b.free_pages() == [4, 2] and b.groups[0].held_pages(s) == []
    assert b.reserve(s, 8)
    b.check()


def test_window_pages_are_given_back_once_the_window_has_passed_them():
    b = books(pages=8, window=6, page_tokens=4)
    s = b.admit()
    assert b.reserve(s, 9)
    b.commit(s, 9)          # next token 9 reads keys [4, 9]: page 0 (positions 0..3) is dead in the window group
    assert len(b.groups[0].held_pages(s)) == 3 and len(b.groups[1].held_pages(s)) == 2
    assert b.groups[1].table[s, 0] == -1 and b.groups[1].table[s, 1] >= 0
    for _ in range(20):
        assert b.reserve(s, 1)
        b.commit(s, 1)
        L = int(b.length[s])
        live_from = (L + 1 - 6) // 4
        assert int(b.groups[1].first_live[s]) == live_from
        assert len(b.groups[1].held_pages(s)) <= 3          # ceil((w - 1) / P) + 1 pages at most
        b.check()
    b.release(s)
    assert b.free_pages() == [8, 8]


def test_limits_and_misuse():
    b = books(ctx=8)
    s = b.admit()
    with pytest.raises(CacheError, match="limit"):
        b.reserve(s, 9)
    with pytest.raises(CacheError, match="without reserved pages"):
        b.commit(s, 5)
    with pytest.raises(CacheError, match="holds no request"):
        b.reserve(2, 1)
    b.release(s)
    with pytest.raises(CacheError, match="holds no request"):
        b.release(s)
    assert [b.admit() is not None for _ in range(4)] == [True, True, True, False]


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2 ** 31), st.sampled_from([0, 5, 9]), st.sampled_from([2, 4, 16]))
def test_random_orders_lose_no_page(seed, window, page_tokens):
    rng = random.Random(seed)
    b = books(pages=12, window=window, page_tokens=page_tokens, max_seqs=4, ctx=40)
    live = {}
    for _ in range(120):
        op = rng.random()
        if op < 0.25 and b.free_slots:
            s = b.admit()
            live[s] = 0
        elif op < 0.85 and live:
            s = rng.choice(list(live))
            n = rng.randint(1, 9)
            if live[s] + n > 40:
                continue
            need = b.pages_needed(s, n)
            free = b.free_pages()
            ok = b.reserve(s, n)
            assert ok == all(x <= f for x, f in zip(need, free))
            if ok:
                b.commit(s, n)
                live[s] += n
                assert int(b.length[s]) == live[s]
            else:
                assert b.free_pages() == free
        elif live:
            s = rng.choice(list(live))
            b.release(s)
            del live[s]
        b.check()
        for g in b.groups:
            assert g.allocator.free_count + sum(len(g.held_pages(s)) for s in live) == g.allocator.num_pages
    for s in list(live):
        b.release(s)
    assert all(f == 12 for f in b.free_pages())


@settings(max_examples=40, deadline=None)
@given(st.integers(0, 2 ** 31), st.sampled_from([0, 6]), st.sampled_from([2, 4]))
def test_one_token_each_equals_one_by_one(seed, window, page_tokens):
    """The decode step's batch calls leave the books exactly as the one-by-one calls do,
    and refuse (changing nothing) exactly when the pages for all of them are not there."""
    rng = random.Random(seed)
    a = books(pages=9, window=window, page_tokens=page_tokens, max_seqs=4, ctx=30)
    b = books(pages=9, window=window, page_tokens=page_tokens, max_seqs=4, ctx=30)
    live = []
    for _ in range(80):
        op = rng.random()
        if op < 0.2 and a.free_slots:
            s = a.admit()
            assert b.admit() == s
            n = rng.randint(0, 5)
            if n and a.reserve(s, n):
                a.commit(s, n)
                assert b.reserve(s, n)
                b.commit(s, n)
            live.append(s)
        elif op < 0.9 and live:
            slots = rng.sample(live, rng.randint(1, len(live)))
            if any(int(a.length[s]) + 1 > 30 for s in slots):
                continue
            needs = [a.pages_needed(s, 1) for s in slots]
            fits = a.fits(needs)
            before = (a.free_pages(), [g.table.copy() for g in a.groups])
            got = a.reserve_one_each(slots)
            assert (got is not None) == fits
            if got is None:
                assert a.free_pages() == before[0] and all((g.table == t).all() for g, t in zip(a.groups, before[1]))
                continue
            assert [int(x) for x in got] == [int(b.length[s]) for s in slots]
            a.commit_one_each(slots)
            for s in slots:
                assert b.reserve(s, 1)
                b.commit(s, 1)
        elif live:
            s = live.pop(rng.randrange(len(live)))
            a.release(s)
            b.release(s)
        a.check()
        assert (a.length == b.length).all() and a.free_pages() == b.free_pages()
        for ga, gb in zip(a.groups, b.groups):
            assert (ga.first_live == gb.first_live).all() and (ga.next_page == gb.next_page).all()
            # which page ids are drawn depends on the order of takes and returns; how many each holds does not
            assert [len(ga.held_pages(s)) for s in live] == [len(gb.held_pages(s)) for s in live]
    with pytest.raises(CacheError):
        a.reserve_one_each([3] if 3 not in live else [7])


def test_manager_groups_layers_by_their_needs():
    full, win = KvNeed(2, 16, 0), KvNeed(2, 16, 8)
    m = CacheManager([full, win, full, win, None], [None, None, None, None, StateNeed((3,))], [None, None, None, 1, None],
                     page_tokens=4, max_seqs=2, max_tokens_per_seq=32, num_pages=6, cache_dtype=None, device=None)
    assert m.num_groups == 2
    assert m.entry_group == [0, 1, 0, 1, None]
    assert m.entry_plane == [0, 0, 1, 0, None]               # entry 3 reads entry 1's plane
    with pytest.raises(CacheError, match="caches nothing"):
        CacheManager([None, full], [None, None], [None, 0], 4, 2, 32, 6, None, None)
    with pytest.raises(CacheError, match="window"):
        CacheManager([win, full], [None, None], [None, 0], 4, 2, 32, 6, None, None)


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2 ** 31), st.sampled_from([0, 5, 9]), st.sampled_from([2, 4, 16]))
def test_native_books_agree_with_the_plain_books_call_for_call(seed, window, page_tokens):
    """The engine's books (native code) and the plain Python books, driven by the same random
    order of admissions, reservations (one request, a whole step, one token each), commits and
    releases: the same answers, page ids, tables, lengths and free counts after every call."""
    import numpy as np
    import plain_books as PB
    rng = random.Random(seed)
    specs = [(2, 16, 0)] + ([(2, 16, window)] if window else [])
    a = CacheBooks([GroupSpec(*s) for s in specs], [11] * len(specs), page_tokens, 4, 48)
    b = PB.CacheBooks([PB.GroupSpec(*s) for s in specs], [11] * len(specs), page_tokens, 4, 48)
    live = []
    for _ in range(150):
        op = rng.random()
        if op < 0.2:
            s = a.admit()
            assert s == b.admit()
            if s is not None:
                live.append(s)
        elif op < 0.5 and live:
            s, n = rng.choice(live), rng.randint(1, 11)
            if int(b.length[s]) + n > 48:
                with pytest.raises(CacheError, match="limit"):
                    a.reserve(s, n)
                continue
            assert a.pages_needed(s, n) == b.pages_needed(s, n)
            ok = a.reserve(s, n)
            assert ok == b.reserve(s, n)
            if ok:
                a.commit(s, n)
                b.commit(s, n)
        elif op < 0.7 and live:
            # a whole step: all of its requests or none
            slots = rng.sample(live, rng.randint(1, len(live)))
            ns = [rng.randint(1, 9) for _ in slots]
            if any(int(b.length[s]) + n > 48 for s, n in zip(slots, ns)):
                continue
            needs = [b.pages_needed(s, n) for s, n in zip(slots, ns)]
            short = a.reserve_step(slots, ns)
            assert (short is None) == b.fits(needs)
            if short is None:
                for s, n in zip(slots, ns):
                    assert b.reserve(s, n)
                for s, n in zip(slots, ns):
                    a.commit(s, n)
                    b.commit(s, n)
            else:
                assert short == [sum(n[g] for n in needs) for g in range(len(specs))]
        elif op < 0.85 and live:
            slots = rng.sample(live, rng.randint(1, len(live)))
            if any(int(b.length[s]) + 1 > 48 for s in slots):
                continue
            ga, gb = a.reserve_one_each(slots), b.reserve_one_each(slots)
            assert (ga is None) == (gb is None)
            if ga is not None:
                assert ga.tolist() == gb.tolist()
                a.commit_one_each(slots)
                b.commit_one_each(slots)
        elif live:
            s = live.pop(rng.randrange(len(live)))
            a.release(s)
            b.release(s)
        a.check()
        b.check()
        assert (a.length == b.length).all() and (a.live == b.live).all()
        assert a.free_pages() == b.free_pages() and a.free_slots == b.free_slots
        for ga, gb in zip(a.groups, b.groups):
            assert (ga.table == gb.table).all()
            assert (ga.first_live == gb.first_live).all() and (ga.next_page == gb.next_page).all()
        if live:
            assert a.table_width(live) == max(1, max(int(g.next_page[s]) for g in b.groups for s in live))


def test_native_step_layout():
    """tokens | positions | row -> request | request starts | prior lengths | slots | wanted rows |
    a slab of block-table rows per group, as the kernels read them."""
    import numpy as np
    b = books(pages=12, window=6, page_tokens=4, max_seqs=3, ctx=40)
    s0, s1 = b.admit(), b.admit()
    assert b.reserve(s0, 7) and b.reserve(s1, 2)
    b.commit(s0, 7)
    b.commit(s1, 2)
    slots = np.array([s1, s0], dtype=np.int32)
    counts = np.array([3, 1], dtype=np.int32)
    assert b.reserve_step(slots, counts) is None
    tokens = np.array([10, 11, 12, 20], dtype=np.int32)
    n_want, wants = np.array([2, 1], dtype=np.int32), np.array([0, 2, 0], dtype=np.int32)
    width = b.table_width([s0, s1])
    assert width == 2
    out = np.full(64, -7, dtype=np.int32)
    n = b.layout_step(slots, counts, tokens, n_want, wants, width, out)
    T, R, W, G = 4, 2, 3, 2
    assert n == 3 * T + (R + 1) + 2 * R + W + G * R * width
    want = ([10, 11, 12, 20] + [2, 3, 4, 7] + [0, 0, 0, 1] + [0, 3, 4] + [2, 7] + [s1, s0] + [0, 2, 3]
            + b.groups[0].table[[s1, s0], :2].reshape(-1).tolist() + b.groups[1].table[[s1, s0], :2].reshape(-1).tolist())
    assert out[:n].tolist() == want and (out[n:] == -7).all()
    # the same step laid out for 4 requests and 5 wanted rows: requests without rows, wanted row 0
    out2 = np.full(80, -7, dtype=np.int32)
    n2 = b.layout_step(slots, counts, tokens, n_want, wants, width, out2, pad_requests=4, pad_wanted=5)
    R, W = 4, 5
    assert n2 == 3 * T + (R + 1) + 2 * R + W + G * R * width
    none = [-1] * (2 * width)
    want2 = ([10, 11, 12, 20] + [2, 3, 4, 7] + [0, 0, 0, 1] + [0, 3, 4, 4, 4] + [2, 7, 0, 0] + [s1, s0, -1, -1] + [0, 2, 3, 0, 0]
             + b.groups[0].table[[s1, s0], :2].reshape(-1).tolist() + none
             + b.groups[1].table[[s1, s0], :2].reshape(-1).tolist() + none)
    assert out2[:n2].tolist() == want2 and (out2[n2:] == -7).all()
    with pytest.raises(CacheError, match="needs"):
        b.layout_step(slots, counts, tokens, n_want, wants, width, out[:10])
    with pytest.raises(CacheError, match="holds no request"):
        b.layout_step(np.array([2], dtype=np.int32), counts[:1], tokens, n_want[:1], wants, width, out)
