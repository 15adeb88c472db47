"""GPU test of the paged cache's block manager driving the two paged entry points: a session of
several conversations (multi-token turns, single-token decode steps, one conversation ending and
a new one taking over its pages) gives bit-identical attention outputs to the same session on a
contiguous cache per conversation -- where the reference would have reset the whole cache
(src/chat.nim:86-91)."""
import numpy as np
import pytest
import torch

from gpu_util import host
from nimllm_b200 import _lib
from nimllm_b200 import attention as A

pytestmark = pytest.mark.gpu


def test_pool_memory_is_zeroed_and_views_are_per_layer():
    p = A.PagedKvPool(3, 5, 32, 2, 64, 2, 4)
    k0, k2, v1 = p.k(0), p.k(2), p.v(1)
    assert k0.shape == (5, 2, 32, 64) and k0.dtype == torch.bfloat16
    assert k2.data_ptr() - k0.data_ptr() == 2 * k0.numel() * 2
    assert not k0.any() and not k2.any() and not v1.any()
    t = p.table()
    assert t.shape == (2, 4) and t.dtype == torch.int32 and (t == -1).all()
    assert p.table(1).data_ptr() - t.data_ptr() == 4 * 4
    with pytest.raises(_lib.NimllmAttnError):
        p.k(3)
    p.close()


def test_session_on_the_pool_equals_contiguous_caches():
    Hq, Hkv, D, n_layer, page_rows, cap = 9, 3, 64, 2, 32, 256
    S = 3                                                       # sequence slots
    geom = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
    pool = A.PagedKvPool(n_layer, 14, page_rows, Hkv, D, S, cap // page_rows)
    kc = torch.zeros(n_layer, S, Hkv, cap, D, device="cuda").bfloat16()
    vc = torch.zeros_like(kc)
    flat = dict(seq_stride=Hkv * cap * D, head_stride=cap * D, max_seq=cap)
    cos, sin = A.rope_tables(2 * cap, D, 10000.0)              # idle slots rotate at positions cap .. cap+n
    g = torch.Generator(device="cuda").manual_seed(123)
    lens = np.zeros(S, np.int32)

    def step(n, live=(1, 1, 1)):
        """Every live slot appends n tokens and attends with the query of its last one; an idle
        slot's rows are sent to positions past the table (both caches drop them)."""
        live = np.array(live, bool)
        for s in np.flatnonzero(live):
            pool.reserve(int(s), int(lens[s]) + n)
        pool.sync()
        pos = torch.from_numpy(np.where(live, lens, cap).astype(np.int32)).cuda()
        new_len = torch.from_numpy(np.where(live, lens + n, lens).astype(np.int32)).cuda()
        for layer in range(n_layer):
            acts = [torch.randn(S, n, h * D, generator=g, device="cuda").bfloat16() for h in (Hq, Hkv, Hkv)]
            q1, k1, v1 = (a.clone() for a in acts)
            A.rope_append(q1, k1, v1, cos, sin, seq_pos=pos, k_cache=kc[layer], v_cache=vc[layer], **geom, **flat)
            want = A.decode_batch(q1[:, -1].contiguous(), kc[layer], vc[layer], max_len=cap, seq_len=new_len,
                                  seq_stride=flat["seq_stride"], head_stride=flat["head_stride"], **geom)
            q2, k2, v2 = (a.clone() for a in acts)
            A.rope_append_paged(q2, k2, v2, cos, sin, pool.k(layer), pool.v(layer), pool.table(), seq_pos=pos, **geom)
            got = A.decode_paged(q2[:, -1].contiguous(), pool.k(layer), pool.v(layer), pool.table(), max_len=cap,
                                 seq_len=new_len, **geom)
            torch.cuda.synchronize()
            np.testing.assert_array_equal(host(got)[live], host(want)[live])
            assert np.isfinite(host(got)).all()
        lens[:] = host(new_len)

    step(70)                                                    # first turns: multi-token appends across pages
    for _ in range(30):
        step(1)                                                 # decode steps, crossing a page end on the way
    assert [pool.seq_pages(s) for s in range(S)] == [4, 4, 4] and pool.free_pages == 2
    pool.release(1)                                             # conversation 1 ends; the others keep their history
    kc[:, 1] = 0; vc[:, 1] = 0; lens[1] = 0
    assert pool.free_pages == 6
    step(90, live=(0, 1, 0))                                    # a new conversation in slot 1 reuses freed pages
    step(33)                                                    # 133, 123, 133 rows: 5 + 4 + 5 pages, the pool is full
    assert pool.free_pages == 0
    with pytest.raises(_lib.NimllmAttnError, match="free"):
        pool.reserve(2, 256)                                    # refused alone ...
    step(1)                                                     # ... and everybody carries on
    assert sum(pool.seq_pages(s) for s in range(S)) == 14
    pool.close()
