"""The cache manager on the host: no page lost, held twice or freed twice, under random orders."""
import random

import pytest

from xinfer_b200.cache import CacheError, CacheGroup, CacheManager


def test_pages_are_taken_per_token_and_returned():
    cm = CacheManager([CacheGroup(16, 8)], max_requests=4)
    s = cm.open_request()
    assert cm.length(s) == 0 and cm.table(s) == []
    assert cm.extend(s, 5) and cm.table(s) == [0]
    assert cm.extend(s, 5) and cm.table(s) == [0]          # asking again takes nothing
    cm.advance(s, 5)
    assert cm.extend(s, 16) and cm.table(s) == [0]
    assert cm.extend(s, 17) and cm.table(s) == [0, 1]
    cm.advance(s, 17)
    assert cm.free_pages() == 6
    cm.close_request(s)
    assert cm.free_pages() == 8 and cm.live_requests() == 0
    cm.check_consistent()


def test_reuse_is_first_in_first_out():
    cm = CacheManager([CacheGroup(8, 4)], max_requests=4)
    a, b = cm.open_request(), cm.open_request()
    assert cm.extend(a, 16) and cm.extend(b, 8)
    assert cm.table(a) == [0, 1] and cm.table(b) == [2]
    cm.close_request(a)                      # pages 1, 0 go to the back of the free list
    c = cm.open_request()
    assert c == a                            # lowest free slot
    assert cm.extend(c, 24)
    assert cm.table(c) == [3, 1, 0]
    cm.check_consistent()


def test_all_or_nothing_and_exhaustion():
    cm = CacheManager([CacheGroup(16, 3)], max_requests=2)
    a, b = cm.open_request(), cm.open_request()
    assert cm.extend(a, 32)
    assert not cm.can_extend(b, 33) and not cm.extend(b, 33)
    assert cm.table(b) == [] and cm.free_pages() == 1
    assert cm.extend(b, 16)
    assert not cm.extend(a, 33)
    with pytest.raises(CacheError):
        cm.open_request()
    cm.check_consistent()


def test_misuse_is_refused():
    cm = CacheManager([CacheGroup(16, 4)], max_requests=2)
    s = cm.open_request()
    cm.extend(s, 10)
    with pytest.raises(CacheError):
        cm.advance(s, 40)                    # pages were never taken
    cm.advance(s, 10)
    with pytest.raises(CacheError):
        cm.advance(s, 5)                     # a request never shrinks
    cm.close_request(s)
    with pytest.raises(CacheError):
        cm.close_request(s)                  # freed twice
    with pytest.raises(CacheError):
        cm.length(s)
    assert not cm.extend(s, 4)
    assert cm.free_pages() == 4
    with pytest.raises(CacheError):
        CacheManager([], 1)
    with pytest.raises(CacheError):
        CacheManager([CacheGroup(0, 4)], 1)


def test_window_group_gives_pages_back_once_the_window_has_passed():
    # group 0 keeps all keys, group 1 a window of 20 tokens; both 8-token pages
    cm = CacheManager([CacheGroup(8, 16), CacheGroup(8, 16, window=20)], max_requests=2)
    s = cm.open_request()
    assert cm.extend(s, 40)
    assert len(cm.table(s, 0)) == 5 and len(cm.table(s, 1)) == 5
    cm.advance(s, 40)
    # the next query (position 40) reads keys 21..40: pages 0 and 1 (keys 0..15) are behind it
    assert cm.table(s, 1) == [-1, -1, 2, 3, 4]
    assert cm.table(s, 0) == [0, 1, 2, 3, 4]
    assert cm.free_pages(1) == 13 and cm.free_pages(0) == 11
    for n in range(41, 60):
        assert cm.extend(s, n)
        cm.advance(s, n)
        first_key = n - 20 + 1
        t = cm.table(s, 1)
        assert all((p == -1) == ((i + 1) * 8 <= first_key) for i, p in enumerate(t)), (n, t)
    cm.check_consistent()
    cm.close_request(s)
    assert cm.free_pages(0) == 16 and cm.free_pages(1) == 16


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    groups = [CacheGroup(rng.choice([4, 8, 16]), rng.randint(6, 24)),
              CacheGroup(rng.choice([4, 8, 16]), rng.randint(6, 24), window=rng.randint(3, 40))]
    cm = CacheManager(groups, max_requests=5)
    live = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 5:
            live[cm.open_request()] = 0
        elif op < 0.35 and live:
            s = rng.choice(list(live))
            cm.close_request(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            n = live[s] + rng.randint(1, 30)
            if cm.extend(s, n):
                if rng.random() < 0.9:       # sometimes pages are taken but the step never runs
                    cm.advance(s, n)
                    live[s] = n
            else:
                assert not cm.can_extend(s, n)
        cm.check_consistent()
        assert cm.live_requests() == len(live)
        for s, n in live.items():
            assert cm.length(s) == n
            for g, grp in enumerate(groups):
                t = cm.table(s, g)
                assert len(t) * grp.page_size >= n
                held = [p for p in t if p >= 0]
                assert len(held) == len(set(held))
                if grp.window:  # everything a later query can read is still held
                    first = max(0, n - grp.window + 1) // grp.page_size
                    assert all(p >= 0 for p in t[first:])
    for s in list(live):
        cm.close_request(s)
    assert [cm.free_pages(g) for g in range(2)] == [g.num_pages for g in groups]


def test_the_log_of_freed_pages():
    """With the log on, every page that goes back (a closed request, a window that has passed) is
    reported exactly once; with it off nothing is kept."""
    from xinfer_b200.cache.manager import CacheGroup, CacheManager
    cm = CacheManager([CacheGroup(4, 16, None), CacheGroup(4, 16, 6)], 2)
    a = cm.open_request()
    assert cm.extend(a, 10) and cm.drain_freed() == []
    cm.advance(a, 10)
    assert cm.drain_freed() == []          # the log is off
    cm.log_freed(True)
    assert cm.extend(a, 21)
    cm.advance(a, 21)                      # the windowed group lets go of what lies wholly before position 16
    freed = cm.drain_freed()
    assert freed and all(g == 1 for g, _ in freed) and cm.drain_freed() == []
    held = [p for p in cm.table(a, 0)] + [p for p in cm.table(a, 1) if p >= 0]
    cm.close_request(a)
    rest = cm.drain_freed()
    assert sorted(p for g, p in rest if g == 0) == sorted(cm_pages for cm_pages in held[:6])
    assert len(rest) == len(held) and len(set(rest)) == len(rest)
    cm.check_consistent()
