"""CPU tests of the paged cache's block manager (nimllm_kvpool_*, host bookkeeping only:
created with on_device=0 it makes no CUDA call).  The policy it replaces is the reference's
reset of the whole cache when the next turn does not fit (src/chat.nim:86-91)."""
import random

import numpy as np
import pytest

from nimllm_b200 import _lib
from nimllm_b200.attention import PagedKvPool


def _pool(n_pages=8, page_rows=32, max_seqs=4, max_pages=4):
    return PagedKvPool(2, n_pages, page_rows, 3, 64, max_seqs, max_pages, on_device=False)


def test_create_rejects_bad_arguments():
    for kw in [dict(page_rows=48), dict(n_pages=0), dict(max_seqs=0), dict(max_pages=0)]:
        with pytest.raises(_lib.NimllmAttnError):
            _pool(**kw)


def test_reserve_grows_page_by_page_and_never_shrinks():
    p = _pool()
    assert p.free_pages == 8 and (p.table_host() == -1).all()
    p.reserve(1, 1)
    assert p.seq_pages(1) == 1 and p.seq_rows(1) == 1 and p.free_pages == 7
    p.reserve(1, 32)            # still the first page
    assert p.seq_pages(1) == 1 and p.free_pages == 7
    p.reserve(1, 33)            # crosses into a second page
    assert p.seq_pages(1) == 2 and p.free_pages == 6
    p.reserve(1, 5)             # a smaller request changes nothing
    assert p.seq_pages(1) == 2 and p.seq_rows(1) == 33
    t = p.table_host()
    assert (t[1, :2] >= 0).all() and (t[1, 2:] == -1).all() and (t[[0, 2, 3]] == -1).all()
    p.reserve(0, 0)             # zero rows hold no page
    assert p.seq_pages(0) == 0


def test_a_full_pool_refuses_the_one_request_and_changes_nothing():
    p = _pool(n_pages=5)
    p.reserve(0, 96)            # 3 pages
    p.reserve(1, 40)            # 2 pages
    before = p.table_host()
    with pytest.raises(_lib.NimllmAttnError, match="free"):
        p.reserve(2, 1)
    with pytest.raises(_lib.NimllmAttnError, match="free"):
        p.reserve(1, 128)       # wants 2 more, none free: not even partially granted
    assert (p.table_host() == before).all() and p.seq_rows(1) == 40 and p.free_pages == 0
    p.release(0)                # the caller's eviction choice; sequence 1 keeps its cache
    assert p.free_pages == 3 and p.seq_rows(0) == 0 and (p.table_host()[0] == -1).all()
    assert (p.table_host()[1] == before[1]).all()
    p.reserve(1, 128)
    assert p.seq_pages(1) == 4 and p.free_pages == 1


def test_per_sequence_limit_and_bad_slots():
    p = _pool()
    with pytest.raises(_lib.NimllmAttnError, match="pages"):
        p.reserve(0, 4 * 32 + 1)
    for seq in (-1, 4):
        with pytest.raises(_lib.NimllmAttnError):
            p.reserve(seq, 1)
        with pytest.raises(_lib.NimllmAttnError):
            p.release(seq)
    with pytest.raises(_lib.NimllmAttnError):
        p.table()               # host-only pool has no device table
    with pytest.raises(_lib.NimllmAttnError):
        p.k(0)
    p.sync()                    # a no-op without device memory


def test_random_traffic_keeps_every_page_owned_exactly_once():
    rng = random.Random(7)
    n_pages, max_seqs, max_pages, page_rows = 37, 6, 12, 16
    p = PagedKvPool(1, n_pages, page_rows, 1, 64, max_seqs, max_pages, on_device=False)
    rows = [0] * max_seqs
    for _ in range(2000):
        s = rng.randrange(max_seqs)
        if rng.random() < 0.2:
            p.release(s)
            rows[s] = 0
        else:
            want = rows[s] + rng.randrange(1, 40)
            need = -(-want // page_rows)
            held = -(-rows[s] // page_rows)
            fits = need <= max_pages and need - held <= p.free_pages
            if fits:
                p.reserve(s, want)
                rows[s] = want
            else:
                with pytest.raises(_lib.NimllmAttnError):
                    p.reserve(s, want)
        t = p.table_host()
        held = t[t >= 0]
        assert len(held) == len(set(held.tolist())), "a page is held twice"
        assert len(held) + p.free_pages == n_pages, "a page leaked"
        assert held.size == 0 or held.max() < n_pages
        for q in range(max_seqs):
            k = -(-rows[q] // page_rows)
            assert p.seq_rows(q) == rows[q] and p.seq_pages(q) == k
            assert (t[q, :k] >= 0).all() and (t[q, k:] == -1).all()
    assert isinstance(p.table_host(), np.ndarray)
