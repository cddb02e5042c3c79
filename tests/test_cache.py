"""The cache books: no page lost, held twice or freed twice, under random orders (no GPU)."""
import numpy as np
import pytest

from hk_b200.cache import CacheBooks, CacheError, ContextFull, OutOfPages, PagePool, TooManyRequests


def test_pool_take_give_and_double_free():
    p = PagePool(3)
    a, b, c = p.take(), p.take(), p.take()
    assert sorted([a, b, c]) == [0, 1, 2] and p.free_count == 0
    with pytest.raises(OutOfPages):
        p.take()
    p.give(b)
    with pytest.raises(CacheError):
        p.give(b)                      # freed twice
    with pytest.raises(CacheError):
        p.give(7)                      # never existed
    assert p.take() == b               # last freed, first reused


def test_extend_takes_pages_as_positions_need_them():
    books = CacheBooks([None], page_tokens=4, num_pages=6, max_requests=2, max_context=24)
    s = books.open()
    books.extend(s, 3)
    assert books.groups[0].pool.free_count == 5
    books.extend(s, 1)                 # fills the page
    assert books.groups[0].pool.free_count == 5
    books.extend(s, 1)                 # position 4 opens page 1
    assert books.groups[0].pool.free_count == 4 and int(books.length[s]) == 5
    assert (books.groups[0].table[s, :2] >= 0).all() and books.groups[0].table[s, 2] == -1
    books.audit()
    books.close(s)
    assert books.groups[0].pool.free_count == 6
    books.audit()
    with pytest.raises(CacheError):
        books.close(s)                 # not live any more


def test_out_of_pages_and_context_full_change_nothing():
    books = CacheBooks([None, None], page_tokens=4, num_pages=3, max_requests=3, max_context=16)
    a, b = books.open(), books.open()
    books.extend(a, 8)
    before = (books.free_pages(), int(books.length[b]), books.groups[0].table.copy())
    with pytest.raises(OutOfPages):
        books.extend(b, 5)             # needs 2, 1 free
    assert (books.free_pages(), int(books.length[b])) == before[:2]
    assert (books.groups[0].table == before[2]).all()
    books.extend(b, 4)
    with pytest.raises(ContextFull):
        books.extend(a, 9)             # 17 > 16
    books.audit()
    books.open()
    with pytest.raises(TooManyRequests):
        books.open()


def test_window_group_gives_pages_back_as_the_window_passes():
    # group 0 keeps everything, group 1 a window of 6 positions; 4-token pages
    books = CacheBooks([None, 6], page_tokens=4, num_pages=8, max_requests=1, max_context=32)
    s = books.open()
    books.extend(s, 10)                # positions 0..9, pages 0..2 in both groups
    assert books.free_pages() == [5, 5]
    # next query sits at 10 and reads keys 5..10: page 0 (positions 0..3) has passed
    books.extend(s, 1)
    assert books.free_pages() == [5, 6] and books.groups[1].table[s, 0] == -1
    books.extend(s, 1)                 # query at 11 reads 6..11: nothing new passes, position 11 fits page 2
    assert books.free_pages() == [5, 6]
    books.extend(s, 1)                 # query at 12 reads 7..12, takes page 3
    assert books.free_pages() == [4, 5]
    books.extend(s, 1)                 # query at 13 reads 8..13: page 1 (4..7) passes
    assert books.free_pages() == [4, 6]
    books.audit()
    # a long portion keeps its own pages until the next extend
    books.extend(s, 12)                # up to position 25
    assert int(books.length[s]) == 26
    books.audit()
    books.extend(s, 1)                 # query at 26 reads 21..26: pages 0..4 have passed
    g = books.groups[1]
    assert int(g.first_page[s]) == 5 and (g.table[s, :5] == -1).all() and (g.table[s, 5:7] >= 0).all()
    books.close(s)
    assert books.free_pages() == [8, 8]
    books.audit()


def test_truncate_gives_back_the_tail():
    books = CacheBooks([None], page_tokens=4, num_pages=8, max_requests=1, max_context=32)
    s = books.open()
    books.extend(s, 14)
    books.truncate(s, 5)
    assert books.free_pages() == [6] and int(books.length[s]) == 5
    books.extend(s, 4)
    assert books.free_pages() == [5]
    books.audit()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed):
    rng = np.random.default_rng(seed)
    windows = [None, int(rng.integers(3, 20))] if seed % 2 else [None]
    books = CacheBooks(windows, page_tokens=int(rng.choice([1, 4, 8, 16])), num_pages=int(rng.integers(6, 40)),
                       max_requests=5, max_context=200)
    live = []
    for _ in range(600):
        op = rng.random()
        try:
            if op < 0.15 and len(live) < 5:
                live.append(books.open())
            elif op < 0.25 and live:
                books.close(live.pop(int(rng.integers(len(live)))))
            elif op < 0.30 and live and windows == [None]:
                s = live[int(rng.integers(len(live)))]
                books.truncate(s, int(rng.integers(0, int(books.length[s]) + 1)))
            elif live:
                s = live[int(rng.integers(len(live)))]
                books.extend(s, int(rng.integers(1, 30)) if rng.random() < 0.3 else 1)
        except (OutOfPages, ContextFull, TooManyRequests):
            pass
        books.audit()
        for g in books.groups:
            for s in live:
                n = int(books.length[s])
                # the next query sits at position n and reads keys from n - window + 1 on
                lo = 0 if g.window is None else max(0, n - g.window + 1) // books.page_tokens
                assert int(g.first_page[s]) <= lo, "a page that can still be read was given back"
                need = range(lo, -(-n // books.page_tokens))
                assert all(g.table[s, i] >= 0 for i in need), "a position that can still be read has no page"
    for s in live:
        books.close(s)
    books.audit()
    assert all(f == g.pool.num_pages for f, g in zip(books.free_pages(), books.groups))


def test_pages_passed_says_what_release_would_give_back():
    books = CacheBooks([None, 10], page_tokens=4, num_pages=16, max_requests=2, max_context=64)
    s = books.open()
    books.extend(s, 30)                      # 8 pages in both groups
    # the next query sits at position 30 and reads keys from 21 on: logical pages 0..4 of the windowed group are passed
    assert books.pages_passed(s) == [0, 5]
    assert books.release_passed(s) == 5 and books.pages_passed(s) == [0, 0]
    books.audit()
