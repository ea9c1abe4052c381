"""The cache manager on the host: no page lost, held twice or freed twice, under random request orders."""
import numpy as np
import pytest

from pulse_infer_b200.cache import CacheError, CacheManager, OutOfPages, PageAllocator, PageError
from pulse_infer_b200.parts.base import CacheSpec, StateSpec


def test_allocator_lifo_and_errors():
    a = PageAllocator(4)
    assert a.allocate(2) == [3, 2]                 # first allocation pops the highest id
    a.free([3])
    assert a.allocate(1) == [3]                    # a freed page is handed out again first
    with pytest.raises(OutOfPages):
        a.allocate(3)
    assert a.num_free == 2                         # nothing was taken by the failed call
    a.free([2])
    with pytest.raises(PageError):
        a.free([2])                                # double free
    with pytest.raises(PageError):
        a.free([9])
    with pytest.raises(PageError):
        a.free([3, 3])
    assert a.num_allocated == 1


def _manager(window=None, pages=12, slots=4, page=8, per_request=64):
    specs = [CacheSpec(2, 16, None), CacheSpec(2, 16, window), CacheSpec(2, 16, None)]
    states = [None, StateSpec((3, 5)), None]
    return CacheManager(specs, states, page, pages, slots, per_request, allocate_pools=False)


def test_groups_slots_and_state():
    cm = _manager(window=16)
    assert len(cm.groups) == 2 and cm.groups[0].cache_indices == [0, 2] and cm.groups[1].cache_indices == [1]
    assert cm.state[1].shape == (4, 3, 5)
    s = cm.open("a")
    cm.state[1][s] += 1.0
    cm.reserve("a", 20)
    assert cm.free_pages() == [9, 9] and cm.pages_needed("a", 24) == [0, 0] and cm.pages_needed("a", 25) == [1, 1]
    cm.commit("a", 20)
    assert cm.length("a") == 20
    with pytest.raises(CacheError):
        cm.open("a")
    with pytest.raises(CacheError):
        cm.commit("a", 30)                         # beyond what is reserved
    cm.close("a")
    assert cm.free_pages() == [12, 12]
    s2 = cm.open("b")
    assert s2 == s and float(cm.state[1][s2].abs().sum()) == 0.0    # the slot is reused, its state zeroed
    with pytest.raises(CacheError):
        cm.slot("a")


def test_reservation_is_atomic_and_bounded():
    cm = _manager(pages=3)
    cm.open("a")
    with pytest.raises(OutOfPages):
        cm.reserve("a", 8 * 4)
    assert cm.free_pages() == [3] and (cm.groups[0].table.row(cm.slot("a")) == -1).all()
    cm.reserve("a", 8 * 3)
    with pytest.raises(CacheError, match="beyond"):
        cm.reserve("a", 65)


def test_window_gives_pages_back_as_it_passes():
    cm = _manager(window=16, pages=12)
    cm.open("a")
    full, win = cm.groups
    for length in range(1, 65):
        cm.reserve("a", length)
        cm.commit("a", length)
        cm.check_invariants()
        held_win = int((win.table.row(cm.slot("a")) >= 0).sum())
        # keys a later query can see: length - 15 .. length; pages before that are back in the pool
        first_needed = max(0, (length - 16 + 1) // 8)
        assert held_win == (length + 7) // 8 - first_needed
        assert (win.table.row(cm.slot("a"))[:first_needed] == -1).all()
    assert int((full.table.row(cm.slot("a")) >= 0).sum()) == 8 and held_win <= 3
    cm.close("a")
    assert cm.free_pages() == [12, 12]


@pytest.mark.parametrize("seed", range(8))
def test_random_request_orders_keep_every_page_accounted(seed):
    rng = np.random.RandomState(seed)
    cm = _manager(window=24 if seed % 2 else None, pages=20, slots=4, page=8, per_request=96)
    live, next_id = {}, 0
    for _ in range(400):
        roll = rng.rand()
        if roll < 0.25 and cm.num_free_slots > 0:
            rid = f"r{next_id}"; next_id += 1
            cm.open(rid); live[rid] = 0
        elif roll < 0.85 and live:
            rid = list(live)[rng.randint(len(live))]
            grow = int(rng.choice([1, 1, 1, 2, 7, 19]))
            new_len = min(96, live[rid] + grow)
            if new_len == live[rid]:
                continue
            before = cm.free_pages()
            try:
                cm.reserve(rid, new_len)
            except OutOfPages:
                assert cm.free_pages() == before            # nothing changed
                victim = list(live)[-1]                      # make room the way the scheduler does
                cm.close(victim); del live[victim]
                cm.check_invariants()
                continue
            cm.commit(rid, new_len); live[rid] = new_len
        elif live:
            rid = list(live)[rng.randint(len(live))]
            cm.close(rid); del live[rid]
            with pytest.raises(CacheError):
                cm.close(rid)                                # closing twice is refused
        cm.check_invariants()
    for rid in list(live):
        cm.close(rid)
    cm.check_invariants()
    assert cm.free_pages() == [20] * len(cm.groups) and cm.num_free_slots == 4


def test_dirty_rows_reach_the_device_table():
    import torch
    cm = CacheManager([CacheSpec(1, 16, None)], [None], 8, 6, 3, 32, dtype=torch.float32, device="cpu")
    cm.open("a"); cm.reserve("a", 20); cm.sync_tables()
    g = cm.groups[0]
    assert g.device_table[cm.slot("a")].tolist() == g.table.row(cm.slot("a")).tolist()
    assert g.pool.shape == (1, 2, 6, 1, 8, 16)
    cm.close("a"); cm.sync_tables()
    assert (g.device_table == -1).all()
