"""Host-side cache bookkeeping: no page lost, held twice or freed twice, under random
orders of requests; lowest-free allocation; windows give pages back."""
import random

import numpy as np
import pytest

from imparo_b200.cache import CacheError, CacheFull, CacheManager
from imparo_b200.parts.spec import PagedKV, SlotState

FULL = PagedKV(2, 16)
WIN = PagedKV(2, 16, window=10)


def _cm(page=4, pages=12, slots=3, specs=((0, (FULL,)), (1, (SlotState((2, 8)),)), (2, (WIN,)))):
    return CacheManager(list(specs), page, pages, slots, device=None)


def test_lowest_free_page_and_slot():
    cm = _cm()
    cm.add(10); cm.add(11)
    assert (cm.slot(10), cm.slot(11)) == (0, 1)
    cm.reserve(10, 9); cm.commit(10, 9)
    assert list(cm.table(10, 0)) == [0, 1, 2]
    cm.reserve(11, 4); cm.commit(11, 4)
    assert list(cm.table(11, 0)) == [3]
    cm.release(10)
    cm.add(12)
    assert cm.slot(12) == 0                      # the lowest free slot is used again
    cm.reserve(12, 6); cm.commit(12, 6)
    assert list(cm.table(12, 0)) == [0, 1]       # and the lowest free pages
    cm.check()


def test_pages_are_taken_as_a_request_grows():
    cm = _cm()
    cm.add(1)
    for n in range(1, 14):
        cm.reserve(1, 1); cm.commit(1, 1)
        assert cm.blocks_in_use(1, 0) == (n + 3) // 4
    assert cm.cached(1) == 13


def test_window_group_gives_pages_back():
    cm = _cm(pages=40)
    cm.add(1)
    for _ in range(60):
        cm.reserve(1, 1); cm.commit(1, 1)
        # a query at the next position c sees keys >= c + 1 - 10
        c = cm.cached(1)
        first = max(0, c + 1 - 10) // 4
        tab = cm.table(1, 1)
        assert all(p == -1 for p in tab[:first]) and all(p >= 0 for p in tab[first:(c + 3) // 4])
        assert cm.blocks_in_use(1, 1) <= 4
        cm.check()
    assert cm.blocks_in_use(1, 0) == 15          # the full group keeps every page
    # a long portion needs every page of the portion at once, then gives most back
    cm.add(2)
    cm.reserve(2, 33)
    assert cm.blocks_in_use(2, 1) == 9
    cm.commit(2, 33)
    assert cm.blocks_in_use(2, 1) == 3
    cm.check()


def test_full_pool_is_refused_whole():
    cm = _cm(pages=4)
    cm.add(1); cm.add(2)
    cm.reserve(1, 12); cm.commit(1, 12)
    free_before = [cm.free_pages(0), cm.free_pages(1)]
    with pytest.raises(CacheFull):
        cm.reserve(2, 8)                           # needs 2 pages in the full group, 1 is free
    assert [cm.free_pages(0), cm.free_pages(1)] == free_before
    assert cm.blocks_in_use(2, 0) == 0 and cm.blocks_in_use(2, 1) == 0
    cm.reserve(2, 4)
    cm.rollback(2)                                 # a step that did not run gives its pages back
    assert cm.free_pages(0) == free_before[0]
    cm.check()


def test_slots_run_out_and_double_release_is_an_error():
    cm = _cm(slots=2)
    cm.add(1); cm.add(2)
    with pytest.raises(CacheFull):
        cm.add(3)
    with pytest.raises(CacheError):
        cm.add(1)
    cm.release(1)
    with pytest.raises(CacheError):
        cm.release(1)
    cm.add(3)
    assert cm.slot(3) == 0
    cm.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    page = rng.choice([1, 2, 4, 16])
    pages = rng.randint(6, 40)
    cm = _cm(page=page, pages=pages, slots=4)
    live = {}
    next_id = 1
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 4:
            cm.add(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.3 and live:
            r = rng.choice(list(live)); cm.release(r); del live[r]
        elif live:
            r = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 17])
            need = cm.pages_needed(r, n)
            ok = all(need[g] <= cm.free_pages(g) for g in range(2))
            try:
                cm.reserve(r, n)
                assert ok
                if rng.random() < 0.15:
                    cm.rollback(r)
                else:
                    cm.commit(r, n); live[r] += n
            except CacheFull:
                assert not ok
        cm.check()
        for r, n in live.items():
            assert cm.cached(r) == n
            # every position a query can still see is mapped, in both groups
            tab = cm.table(r, 0)
            assert all(tab[b] >= 0 for b in range((n + page - 1) // page))
            lo = max(0, n + 1 - 10) // page
            tabw = cm.table(r, 1)
            assert all(tabw[b] >= 0 for b in range(lo, (n + page - 1) // page))
        used = sum(cm.blocks_in_use(r, 0) for r in live)
        assert used + cm.free_pages(0) == pages
    for r in list(live):
        cm.release(r)
    assert cm.free_pages(0) == pages and cm.free_pages(1) == pages and cm.free_slots() == 4
    cm.check()


def test_groups_are_formed_by_need():
    specs = [(0, (FULL,)), (1, (SlotState((2, 8)),)), (2, (WIN,)), (3, (FULL,)), (5, (WIN,)), (6, (PagedKV(1, 32),))]
    cm = CacheManager(specs, 4, 8, 2, device=None)
    assert cm.n_groups == 3
    assert cm.group_entries == [[0, 3], [2, 5], [6]]


def test_block_tables_address_rows_as_the_reference_rule_does():
    """tests/golden/kv_paging_golden.json holds what the reference's own physical_row
    (imparo-cuda/native/kv_paging.cuh:25-30) gives for shuffled block tables at its page size of 64.  The
    engine's rule, row = table[pos // page] * page + pos % page, with the table the cache manager hands to the
    kernels, must give the same rows: requests are added and released so that the manager's table for one
    request becomes each golden table."""
    import json
    import os
    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "kv_paging_golden.json")) as f:
        cases = json.load(f)["cases"]
    assert len(cases) >= 3
    for c in cases:
        page, want_table = c["page"], c["table"]
        n = len(want_table)
        cm = CacheManager([(0, (PagedKV(1, 16),))], page, n, n + 1, device=None)
        # one holder request per block, so that every block is taken; then the holders give their blocks back in
        # the order the golden table names them while request 100 grows: the lowest free block is always the next one
        for b in range(n):
            cm.add(b)
            cm.reserve(b, 1)
            cm.commit(b, 1)
            assert list(cm.table(b, 0)) == [b]
        cm.add(100)
        for b in want_table:
            cm.release(b)
            cm.reserve(100, page)
            cm.commit(100, page)
        table = [int(x) for x in cm.table(100, 0)]
        assert table == want_table
        for pos, row in zip(c["logical"], c["physical"]):
            assert table[pos // page] * page + pos % page == row
        cm.release(100)
        cm.check()
