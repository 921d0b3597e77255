"""Page bookkeeping of the paged cache (q27b_pager_*): host code, runs without a GPU."""
import numpy as np
import pytest

PAGE = 256


def pages_of(table_row):
    return [int(x) for x in table_row if x >= 0]


def check_invariants(p, seqs, n_pages):
    """Every page is free or held; a page held by two sequences sits at the same index in both (a shared
    prefix) and below it their tables agree; free + distinct held pages = the pool."""
    table, lens = p.tables(seqs) if seqs else (np.zeros((0, p.max_pages), np.int32), np.zeros((0,), np.int32))
    held = set()
    for b, s in enumerate(seqs):
        pg = pages_of(table[b])
        assert len(pg) == (int(lens[b]) + PAGE - 1) // PAGE
        assert len(set(pg)) == len(pg)
        assert all(0 <= x < n_pages for x in pg)
        assert all(x == -1 for x in table[b, len(pg):])
        held |= set(pg)
    for a in range(len(seqs)):
        for b in range(a + 1, len(seqs)):
            pa, pb = pages_of(table[a]), pages_of(table[b])
            for x in set(pa) & set(pb):
                i = pa.index(x)
                assert pb.index(x) == i and pa[:i] == pb[:i]
    assert p.free_pages() + len(held) == n_pages


def test_extend_cut_close(q27):
    n_pages = 12
    p = q27.Pager(n_pages, 4, 8)
    a = p.open()
    assert p.length(a) == 0 and p.free_pages() == n_pages
    p.extend(a, 1)
    p.extend(a, PAGE)          # still one page
    assert p.free_pages() == n_pages - 1
    p.extend(a, PAGE + 1)
    t0, _ = p.tables([a])
    p.extend(a, 5 * PAGE)
    t1, l1 = p.tables([a])
    assert l1[0] == 5 * PAGE and list(t1[0, :2]) == list(t0[0, :2])  # pages never move
    check_invariants(p, [a], n_pages)
    # cut back: the rows below the new length stay where they are (src/model.h:177-180), the rest is free again
    p.cut(a, 2 * PAGE + 7)
    t2, l2 = p.tables([a])
    assert l2[0] == 2 * PAGE + 7 and list(t2[0, :3]) == list(t1[0, :3]) and t2[0, 3] == -1
    assert p.free_pages() == n_pages - 3
    p.extend(a, 3 * PAGE)      # same page again for the rest of page 2, nothing new
    assert p.free_pages() == n_pages - 3
    p.cut(a, 0)
    assert p.free_pages() == n_pages and p.length(a) == 0
    p.extend(a, 10)
    p.close(a)
    assert p.free_pages() == n_pages and p.length(a) == -1
    with pytest.raises(q27.Q27Error):
        p.extend(a, 10)        # closed


def test_out_of_pages_changes_nothing(q27):
    p = q27.Pager(4, 3, 8)
    a, b = p.open(), p.open()
    p.extend(a, 3 * PAGE)
    p.extend(b, PAGE)
    before = p.tables([a, b])
    with pytest.raises(q27.Q27Error) as e:
        p.extend(b, 2 * PAGE + 1)   # needs two more pages, none is free
    assert e.value.code == q27.UNSUPPORTED
    after = p.tables([a, b])
    assert (before[0] == after[0]).all() and (before[1] == after[1]).all() and p.free_pages() == 0
    with pytest.raises(q27.Q27Error):
        p.extend(a, 9 * PAGE)       # more than max_pages_per_seq
    with pytest.raises(q27.Q27Error):
        p.extend(a, PAGE)           # shorter than it is: that is cut
    with pytest.raises(q27.Q27Error):
        p.cut(a, 3 * PAGE + 1)
    c = p.open()
    with pytest.raises(q27.Q27Error):
        p.open()                    # all slots in use
    p.close(c)


def test_fork_shares_full_pages(q27):
    n_pages = 16
    p = q27.Pager(n_pages, 4, 8)
    a = p.open()
    p.extend(a, 3 * PAGE + 100)
    ta, _ = p.tables([a])
    # prefix ends inside page 2: pages 0 and 1 are shared, page 2 is copied
    b, cp = p.fork(a, 2 * PAGE + 50)
    tb, lb = p.tables([b])
    assert lb[0] == 2 * PAGE + 50 and list(tb[0, :2]) == list(ta[0, :2])
    assert cp == (int(ta[0, 2]), int(tb[0, 2]), 50) and tb[0, 2] != ta[0, 2]
    assert p.free_pages() == n_pages - 4 - 1
    check_invariants(p, [a, b], n_pages)
    # prefix ends on a page boundary: nothing to copy
    c, cp2 = p.fork(a, 2 * PAGE)
    assert cp2 is None and p.free_pages() == n_pages - 5
    p.extend(c, 2 * PAGE + 1)  # its own new page
    check_invariants(p, [a, b, c], n_pages)
    # closing the original keeps the shared pages alive for the forks
    p.close(a)
    assert p.free_pages() == n_pages - 2 - 1 - 1
    check_invariants(p, [b, c], n_pages)
    # a sequence cut back into a shared page may not write there before it has a copy of its own
    p.cut(c, PAGE + 10)
    with pytest.raises(q27.Q27Error) as e:
        p.extend(c, PAGE + 11)
    assert e.value.code == q27.UNSUPPORTED
    tc0, _ = p.tables([c])
    cp3 = p.unshare(c)
    tc1, _ = p.tables([c])
    assert cp3 == (int(tc0[0, 1]), int(tc1[0, 1]), 10) and tc1[0, 1] != tc0[0, 1]
    assert p.unshare(c) is None
    p.extend(c, PAGE + 11)
    check_invariants(p, [b, c], n_pages)
    p.close(b)
    p.close(c)
    assert p.free_pages() == n_pages


def test_random_walk_keeps_the_books(q27):
    rng = np.random.default_rng(7)
    n_pages, max_pages = 40, 10
    p = q27.Pager(n_pages, 6, max_pages)
    live = []
    for step in range(600):
        op = rng.integers(0, 6)
        try:
            if op == 0 and len(live) < 6:
                live.append(p.open())
            elif op == 1 and live:
                s = live[rng.integers(len(live))]
                p.extend(s, min(max_pages * PAGE, p.length(s) + int(rng.integers(0, 3 * PAGE))))
            elif op == 2 and live:
                s = live[rng.integers(len(live))]
                p.cut(s, int(rng.integers(0, p.length(s) + 1)))
            elif op == 3 and live:
                s = live.pop(rng.integers(len(live)))
                p.close(s)
            elif op == 4 and live and len(live) < 6:
                s = live[rng.integers(len(live))]
                n, _ = p.fork(s, int(rng.integers(0, p.length(s) + 1)))
                live.append(n)
            elif op == 5 and live:
                p.unshare(live[rng.integers(len(live))])
        except q27.Q27Error as e:
            assert e.code == q27.UNSUPPORTED  # out of pages, or a shared last page: the books must still add up
        check_invariants(p, live, n_pages)
    for s in live:
        p.close(s)
    assert p.free_pages() == n_pages
