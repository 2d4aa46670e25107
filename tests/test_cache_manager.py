"""Cache manager on the host: no page lost, held twice or freed twice under
random orders of requests; LIFO reuse; windows give pages back; state slots."""

import random

import numpy as np
import pytest
import torch

from deterministic_inference_b200.cache import CacheError, CacheManager, OutOfPages
from deterministic_inference_b200.parts import PagedKVSpec, StateSpec


def make(pages=10, page=4, reqs=6, window=None, state=False, max_len=64):
    specs = {0: PagedKVSpec(2, 8, None), 1: PagedKVSpec(2, 8, None)}
    if window:
        specs[2] = PagedKVSpec(2, 8, window)
    if state:
        specs[3] = StateSpec((5,), "float32")
    return CacheManager(specs, num_pages=pages, page_size=page, max_reqs=reqs, max_seq_len=max_len,
                        dtype=torch.float32, device="cpu")


def test_groups_by_need():
    c = make(window=6, state=True)
    assert len(c.page_groups) == 2 and len(c.state_groups) == 1
    full = c.page_groups[("paged_kv", 2, 8, None)]
    assert full.cache_ids == [0, 1] and full.pool.shape == (2, 10, 2, 2, 4, 8)
    assert c.page_groups[("paged_kv", 2, 8, 6)].pool.shape == (1, 10, 2, 2, 4, 8)
    assert c.state_groups[("state", (5,), "float32")].array.shape == (1, 6, 5)


def test_allocate_grow_release_and_lifo_reuse():
    c = make()
    g = next(iter(c.page_groups.values()))
    a = c.allocate_slot()
    c.allocate(a, 5)                        # 2 pages
    assert g.pages[a] == [1, 2] and c.num_free_pages() == 7
    c.allocate(a, 8)                        # still 2 pages
    assert g.pages[a] == [1, 2]
    c.allocate(a, 9)
    assert g.pages[a] == [1, 2, 3]
    b = c.allocate_slot()
    c.allocate(b, 4)
    assert g.pages[b] == [4]
    c.release_slot(a)
    c.check_invariants()
    d = c.allocate_slot()
    c.allocate(d, 12)
    assert g.pages[d] == [3, 2, 1]          # the pages freed last come back first
    assert 0 not in g.pages[d]              # page 0 is never handed out
    c.check_invariants()


def test_out_of_pages_is_all_or_nothing():
    c = make(pages=5)                       # 4 usable pages
    a, b = c.allocate_slot(), c.allocate_slot()
    c.allocate(a, 12)                       # 3 pages
    assert c.can_allocate(b, 4) and not c.can_allocate(b, 5) and not c.can_allocate(None, 8)
    with pytest.raises(OutOfPages):
        c.allocate(b, 8)
    assert next(iter(c.page_groups.values())).pages[b] == []
    c.check_invariants()


def test_double_free_and_foreign_free_are_caught():
    c = make()
    a = c.allocate_slot()
    c.allocate(a, 4)
    c.release_slot(a)
    with pytest.raises(CacheError, match="released twice"):
        c.release_slot(a)
    with pytest.raises(CacheError, match="not live"):
        c.allocate(a, 4)
    g = next(iter(c.page_groups.values()))
    with pytest.raises(CacheError, match="freed twice"):
        g._give_back(1)


def test_window_group_gives_pages_back_as_the_window_passes():
    c = make(pages=12, page=4, window=6)
    full = c.page_groups[("paged_kv", 2, 8, None)]
    win = c.page_groups[("paged_kv", 2, 8, 6)]
    a = c.allocate_slot()
    c.allocate(a, 16)
    assert len(win.pages[a]) == 4
    # the next query stands at position 16 and sees keys 11..16: pages 0 and 1 (positions 0..7) go
    assert c.release_passed(a, 16) == 2
    assert win.pages[a][:2] == [0, 0] and win.pages[a][2] != 0
    assert all(p != 0 for p in full.pages[a])               # the full group keeps everything
    c.check_invariants()
    # a query at 17 sees keys 12..17: page 2 (positions 8..11) goes, page 3 stays until 21
    assert c.release_passed(a, 17) == 1 and c.release_passed(a, 20) == 0
    bt = c.block_table(win, [a], 5)
    assert bt.shape == (1, 5) and list(bt[0, :3]) == [0, 0, 0]
    with pytest.raises(CacheError, match="not covered"):
        c.slot_mapping(win, a, 4, 2)
    c.release_slot(a)
    c.check_invariants()


def test_slot_mapping_and_block_table():
    c = make()
    g = next(iter(c.page_groups.values()))
    a = c.allocate_slot()
    c.allocate(a, 10)
    sm = c.slot_mapping(g, a, 3, 6)          # positions 3..8
    pl = g.pages[a]
    assert list(sm) == [pl[0] * 4 + 3, pl[1] * 4, pl[1] * 4 + 1, pl[1] * 4 + 2, pl[1] * 4 + 3, pl[2] * 4]
    assert c.block_table(g, [a, a], 4).tolist() == [pl + [0], pl + [0]]


def test_state_slots_are_zeroed_for_new_requests():
    c = make(state=True)
    arr = next(iter(c.state_groups.values())).array
    a = c.allocate_slot()
    c.reset_fresh_state()
    arr[0, a] = 7.0
    c.release_slot(a)
    b = c.allocate_slot()
    assert b == a                           # the slot comes back
    c.reset_fresh_state()
    assert float(arr[0, b].abs().sum()) == 0.0
    assert 0 not in c.live_slots            # slot 0 is never handed out


def test_sequence_longer_than_the_table_is_refused():
    c = make(pages=40, max_len=16)
    a = c.allocate_slot()
    with pytest.raises(CacheError, match="max_seq_len"):
        c.allocate(a, 17)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    c = make(pages=24, page=4, reqs=7, window=rng.choice([None, 5, 9]), max_len=80)
    live = {}                                # slot -> length
    for _ in range(400):
        op = rng.random()
        if op < 0.3 and c.num_free_slots:
            live[c.allocate_slot()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = live[s] + rng.choice([1, 1, 2, 7, 13])
            if n <= 80 and c.can_allocate(s, n):
                c.allocate(s, n)
                live[s] = n
                c.release_passed(s, n)
                for g in c.page_groups.values():          # every position a query needs is covered
                    lo = 0 if g.window is None else max(0, n - g.window + 1)
                    if n > lo:
                        c.slot_mapping(g, s, lo, n - lo)
            elif n <= 80:
                with pytest.raises(OutOfPages):
                    c.allocate(s, n)
        elif live:
            s = rng.choice(list(live))
            c.release_slot(s)
            del live[s]
        c.check_invariants()
    for s in list(live):
        c.release_slot(s)
    c.check_invariants()
    assert all(g.num_free == g.num_pages - 1 for g in c.page_groups.values())


def test_pages_for_a_byte_budget_are_shared_by_bytes_per_page_and_window_groups_are_capped():
    """Pools sized from a byte budget: groups that keep all keys get the same number of
    pages; a window group gets no more than its requests can ever hold, and what that
    saves goes to the others."""
    from deterministic_inference_b200.cache.manager import group_page_bytes, pages_for_budget
    specs = {0: PagedKVSpec(2, 32, None), 1: PagedKVSpec(2, 32, None), 2: PagedKVSpec(2, 32, 24),
             3: PagedKVSpec(4, 16, None), 4: StateSpec((8,), "float32")}
    page, dt = 16, torch.bfloat16
    per = group_page_bytes(specs, page, dt)
    full_a, win, full_b = PagedKVSpec(2, 32, None).group_key(), PagedKVSpec(2, 32, 24).group_key(), \
        PagedKVSpec(4, 16, None).group_key()
    assert per[full_a][1] == 2 * 2 * 2 * page * 32 * 2 and per[win][1] == 2 * 2 * page * 32 * 2
    budget = 10_000_000
    pages = pages_for_budget(specs, budget, page, dt, max_reqs=4, step_tokens=64)
    assert pages[full_a] == pages[full_b] and pages[win] == 1 + 4 * (-(-(24 + 64) // page) + 2)
    cost = sum(pages[k] * per[k][1] for k in pages)
    assert cost <= budget < cost + per[full_a][1] + per[full_b][1]     # one more page would not fit
    # a budget so small that the window group is not capped: all groups get the same pages
    small = pages_for_budget(specs, 20 * sum(b for _, b in per.values()), page, dt, 4, 64)
    assert small[full_a] == small[win] == small[full_b] == 20
    with pytest.raises(CacheError):
        pages_for_budget(specs, 1000, page, dt, 4, 64)
    # the manager takes the dict: each group has its own pool size, and a request's length is
    # bounded by the groups that keep all keys
    m = CacheManager(specs, pages, page, max_reqs=5, max_seq_len=4096, dtype=dt, device="cpu",
                     allocate_device=False)
    assert {g.key: g.num_pages for g in m.page_groups.values()} == pages
    assert m.usable_pages() == pages[full_a] - 1
    s = m.allocate_slot()
    m.allocate(s, 200)
    m.release_passed(s, 200)
    m.check_invariants()
    m.release_slot(s)
    m.check_invariants()
