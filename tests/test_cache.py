"""The cache manager on the host: no page lost, held twice or freed twice, under random orders (no GPU)."""
import random

import pytest

from purhie_b200.cache import CacheManager, CacheNeed, CheckError, OutOfPages, OutOfSlots, PageAllocator, SlotAllocator
from purhie_b200.native import InferenceError


def test_allocator_hands_out_each_page_once_and_reuses_the_last_freed():
    a = PageAllocator(4)
    p = a.alloc(3)
    assert sorted(p) == [0, 1, 2] and a.num_free == 1
    with pytest.raises(OutOfPages):
        a.alloc(2)
    assert a.num_free == 1                      # a refused allocation takes nothing
    a.free([p[1]])
    assert a.alloc(1) == [p[1]]                 # reuse starts with the page freed last
    a.free(p)
    with pytest.raises(CheckError):
        a.free([p[0]])                          # freed twice
    a.check()


def test_reference_counts_keep_a_shared_page():
    a = PageAllocator(2)
    (p,) = a.alloc(1)
    a.share(p)
    assert a.free([p]) == [] and a.num_free == 1
    assert a.free([p]) == [p] and a.num_free == 2


def test_slots():
    s = SlotAllocator(2)
    x, y = s.alloc(), s.alloc()
    with pytest.raises(OutOfSlots):
        s.alloc()
    s.free(x)
    with pytest.raises(CheckError):
        s.free(x)
    assert s.alloc() == x
    s.check()


def needs_two_groups():
    full = CacheNeed.pages(2, 16)
    win = CacheNeed.pages(2, 16, window=24)
    return [full, win, CacheNeed(), win, CacheNeed.state((4,))]


def test_groups_are_formed_by_geometry_and_policy():
    m = CacheManager(needs_two_groups(), page_size=8, num_pages=[10, 6], max_requests=3)
    assert [(g["window"], g["entries"]) for g in m.groups] == [(None, [0]), (24, [1, 3])]
    assert m.state_entries == [4]
    assert m.entry_group == {0: 0, 1: 1, 3: 1}


def test_values_narrower_than_keys_get_a_group_and_pages_of_their_own_size():
    """A mixer may keep values that are not as wide as its keys (compressed values): such entries form a group of
    their own, and a page of that group holds kv_heads x page_size x (key width + value width) elements per entry
    (`page_stride`: an entry's pages lie side by side, the entries of a group one after the other)."""
    needs = [CacheNeed.pages(2, 16), CacheNeed.pages(2, 16, value_dim=4), CacheNeed.pages(2, 16, value_dim=4),
             CacheNeed.pages(2, 16, value_dim=16)]
    m = CacheManager(needs, page_size=8, num_pages=[5, 7], max_requests=2)
    groups = m.info()["groups"]
    assert [(g["entries"], g["head_dim"], g["value_dim"]) for g in groups] == [([0, 3], 16, 16), ([1, 2], 16, 4)]
    assert groups[0]["page_stride"] == 2 * 8 * (16 + 16)
    assert groups[1]["page_stride"] == 2 * 8 * (16 + 4)
    m.add_request("a")
    m.reserve("a", 20)
    m.advance("a", 20)
    assert m.free_pages() == [2, 4]
    m.release("a")
    m.check()


def test_pages_grow_one_block_at_a_time_and_window_pages_return():
    m = CacheManager(needs_two_groups(), page_size=8, num_pages=[16, 16], max_requests=2)
    m.add_request("a")
    total = 0
    for n in (5, 3, 1, 20, 1, 1, 40, 2):
        m.reserve("a", n)
        assert len(m.block_table("a", 0)) == -(-(total + n) // 8)
        m.advance("a", n)
        total += n
        m.check()
        # full group keeps everything; the window group keeps only blocks a later query can see
        assert all(p >= 0 for p in m.block_table("a", 0))
        first_needed = max(0, total - 24 + 1) // 8
        t = m.block_table("a", 1)
        assert all(p == -1 for p in t[:first_needed]) and all(p >= 0 for p in t[first_needed:])
    assert m.groups[1]["used"] == len(m.block_table("a", 1)) - max(0, total - 24 + 1) // 8
    slots = m.token_slots("a", 0, 60, 4)
    assert len(set(slots)) == 4
    with pytest.raises(RuntimeError):
        m.token_slots("a", 1, 0, 1)             # that page was given back
    m.release("a")
    assert m.free_pages() == [16, 16] and m.free_slots == 2
    m.check()


def test_reserve_is_all_or_nothing_and_unreserve_restores():
    m = CacheManager([CacheNeed.pages(1, 16), CacheNeed.pages(1, 16, window=8)], page_size=4, num_pages=[8, 2],
                     max_requests=2)
    m.add_request("a")
    with pytest.raises(OutOfPages):
        m.reserve("a", 12)                      # the window group has 2 pages only
    assert m.free_pages() == [8, 2]
    m.reserve("a", 8)
    m.unreserve("a")
    assert m.free_pages() == [8, 2] and m.length("a") == 0
    m.check()


def test_truncate_gives_back_whole_pages_past_the_length():
    m = CacheManager([CacheNeed.pages(1, 16)], page_size=4, num_pages=8, max_requests=1)
    m.add_request("a")
    m.reserve("a", 14); m.advance("a", 14)
    m.truncate("a", 5)
    assert m.length("a") == 5 and len(m.block_table("a", 0)) == 2 and m.free_pages() == [6]
    with pytest.raises(InferenceError):
        m.truncate("a", 9)
    m.check()


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    m = CacheManager(needs_two_groups(), page_size=4, num_pages=[24, 12], max_requests=4)
    live, ever = {}, 0
    for _ in range(600):
        r = rng.random()
        if r < 0.15 and len(live) < 4:
            rid = f"r{ever}"; ever += 1
            m.add_request(rid); live[rid] = 0
        elif r < 0.25 and live:
            rid = rng.choice(sorted(live))
            m.release(rid); del live[rid]
        elif live:
            rid = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 13])
            before = m.free_pages()
            try:
                m.reserve(rid, n)
            except OutOfPages:
                assert m.free_pages() == before
                if rng.random() < 0.5:
                    m.release(rid); del live[rid]
                continue
            if rng.random() < 0.1:
                m.unreserve(rid)
            else:
                m.advance(rid, n); live[rid] += n
                assert m.length(rid) == live[rid]
        m.check()
        with pytest.raises(OutOfSlots) if len(live) == 4 else _null():
            if len(live) == 4:
                m.add_request("overflow")
    for rid in list(live):
        m.release(rid)
    assert m.free_pages() == [24, 12]
    m.check()


class _null:
    def __enter__(self): return self
    def __exit__(self, *a): return False


def test_slots_of_a_long_portion_are_those_of_its_tokens_one_by_one():
    """Long portions are mapped page by page; the result is what mapping every token alone gives, also across pages
    that a window has passed (which must raise either way)."""
    cm = CacheManager([CacheNeed.pages(1, 8, None), CacheNeed.pages(1, 8, 40)], 16, [64, 64], 2)
    cm.add_request("a")
    cm.reserve("a", 300)
    for g in (0, 1):
        for start, n in ((0, 300), (5, 200), (17, 64), (100, 199), (299, 1)):
            one_by_one = sum((cm.token_slots("a", g, p, 1) for p in range(start, start + n)), [])
            assert cm.token_slots("a", g, start, n) == one_by_one
    cm.advance("a", 300)
    cm.reserve("a", 80)                                       # the window group has given back its first pages
    assert cm.token_slots("a", 1, 300, 80) == sum((cm.token_slots("a", 1, p, 1) for p in range(300, 380)), [])
    with pytest.raises(RuntimeError):
        cm.token_slots("a", 1, 0, 100)
