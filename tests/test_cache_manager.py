"""The cache manager's bookkeeping: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; pages are reused."""
import numpy as np
import pytest

from crane_b200.cache import CacheError, GroupSpec, OutOfPages, PageTable


def test_admit_extend_release_and_block_table():
    t = PageTable([GroupSpec(8, 16)], max_requests=2)
    assert t.admit(1) in (0, 1)
    t.extend(1, 17)
    assert t.length(1) == 17 and t.free_pages() == 6
    bt = t.block_table(1, 0, 5)
    assert list(bt[2:]) == [-1, -1, -1] and len(set(bt[:2])) == 2 and min(bt[:2]) >= 0
    t.extend(1, 15)                       # 32 tokens: still two pages
    assert t.free_pages() == 6
    t.extend(1, 1)
    assert t.free_pages() == 5
    t.release(1)
    assert t.free_pages() == 8 and t.free_slots() == 2
    t.check()


def test_errors_are_loud():
    t = PageTable([GroupSpec(2, 16)], max_requests=1)
    t.admit(1)
    with pytest.raises(CacheError, match="already live"):
        t.admit(1)
    with pytest.raises(CacheError, match="no free state slot"):
        t.admit(2)
    with pytest.raises(OutOfPages):
        t.extend(1, 33)
    assert t.length(1) == 0 and t.free_pages() == 2      # a refused extension changes nothing
    t.release(1)
    with pytest.raises(CacheError, match="released twice"):
        t.release(1)
    with pytest.raises(CacheError):
        t.length(1)
    t.check()


def test_freed_pages_are_handed_out_first():
    t = PageTable([GroupSpec(6, 16)], max_requests=3)
    t.admit(1); t.extend(1, 32)
    first = set(t.block_table(1, 0, 2))
    t.release(1)
    t.admit(2); t.extend(2, 32)
    assert set(t.block_table(2, 0, 2)) == first           # the same pages, used again
    assert t.pages_reused() == 2


def test_window_group_gives_pages_back():
    # group 0 keeps everything, group 1 only the last 20 positions
    t = PageTable([GroupSpec(16, 8), GroupSpec(6, 8, window=20)], max_requests=1)
    t.admit(7)
    for _ in range(12):
        t.extend(7, 10)
        t.check()
    assert t.length(7) == 120
    assert t.free_pages(0) == 1                            # 15 pages for 120 tokens
    bt = t.block_table(7, 1, 16)
    # the next token (position 120) reads positions >= 101: blocks 12.. are needed
    assert all(b == -1 for b in bt[:11]) and all(b >= 0 for b in bt[13:15])
    assert t.free_pages(1) >= 6 - 5
    t.release(7)
    assert t.free_pages(0) == 16 and t.free_pages(1) == 6
    t.check()


def test_window_pages_cover_the_portion_being_written():
    t = PageTable([GroupSpec(8, 4, window=6)], max_requests=1)
    t.admit(1)
    t.extend(1, 10)        # positions 0..9
    t.extend(1, 9)         # portion 10..18: its first token reads from position 5 = block 1
    bt = t.block_table(1, 0, 8)
    assert bt[0] == -1 and all(b >= 0 for b in bt[1:5])


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_the_books_straight(seed):
    rng = np.random.default_rng(seed)
    groups = [GroupSpec(40, 16), GroupSpec(24, 8, window=int(rng.integers(9, 60)))]
    t = PageTable(groups, max_requests=5)
    live, next_id = {}, 1
    for _ in range(600):
        r = rng.random()
        if r < 0.25 and t.free_slots() > 0:
            t.admit(next_id)
            live[next_id] = 0
            next_id += 1
        elif r < 0.85 and live:
            rid = int(rng.choice(list(live)))
            n = int(rng.integers(1, 50))
            need = [t.pages_needed(rid, n, g) for g in range(2)]
            fits = all(need[g] <= t.free_pages(g) for g in range(2))
            assert t.try_extend(rid, n) == fits
            if fits:
                live[rid] += n
            assert t.length(rid) == live[rid]
        elif live:
            rid = int(rng.choice(list(live)))
            t.release(rid)
            del live[rid]
        t.check()
        # what a request may read is held: every block of the full group, the window's blocks
        for rid, n in live.items():
            bt = t.block_table(rid, 0, 64)
            assert all(b >= 0 for b in bt[: (n + 15) // 16])
            w = groups[1].window
            btw = t.block_table(rid, 1, 128)
            first = max(0, n - w + 1) // 8
            assert all(b >= 0 for b in btw[first: (n + 7) // 8])
    for rid in list(live):
        t.release(rid)
    t.check()
    assert t.free_pages(0) == 40 and t.free_pages(1) == 24 and t.free_slots() == 5
    assert t.pages_reused() > 0


def test_pools_shape_keys_and_values_independently():
    """A mixer may keep values wider or narrower than its keys: the group key,
    the bytes a page costs and (on a device) the pools' shapes follow."""
    from crane_b200.cache.pools import bytes_per_page, group_layers
    from crane_b200.parts import CacheNeed
    needs = [CacheNeed("kv", kv_heads=2, head_dim=16), CacheNeed("kv", kv_heads=2, head_dim=16, v_head_dim=40),
             CacheNeed("none"), CacheNeed("kv", kv_heads=2, head_dim=16), CacheNeed("kv", kv_heads=1, head_dim=24, v_head_dim=8)]
    keys, of_layer = group_layers(needs)
    assert keys == [(2, 16, 0, 16), (2, 16, 0, 40), (1, 24, 0, 8)] and of_layer == [0, 1, -1, 0, 2]
    assert bytes_per_page(needs, 8, 2) == [2 * (2 * 8 * 32 * 2), 2 * 8 * 56 * 2, 1 * 8 * 32 * 2]
    assert needs[0].value_dim == 16 and needs[1].value_dim == 40
