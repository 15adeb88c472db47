"""GPU parity of the paged-cache decode: the same sequences stored contiguously and scattered over
randomly assigned pages must give bit-identical results (same kernel arithmetic, only the
addresses differ), and both match the float64 ground truth; appends through the page table land
in the right rows."""
import numpy as np
import pytest
import torch

from gpu_util import bf16_bits, host
from nimllm_b200 import attention as A
from oracle import oracle as O
from util import TOL_BF16, assert_close

pytestmark = pytest.mark.gpu


def _paged_copy(kc, vc, lens, page_rows, gen):
    """kc, vc [B, Hkv, cap, D] -> pages [n_pages, Hkv, page_rows, D] in shuffled order + table."""
    B, Hkv, cap, D = kc.shape
    per_seq = [int((L + page_rows - 1) // page_rows) for L in lens]
    max_pages = max(max(per_seq), 1)
    n_pages = sum(per_seq) + 3                                  # a few pages stay unused
    order = torch.randperm(n_pages, generator=gen).tolist()
    kp = torch.full((n_pages, Hkv, page_rows, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    vp = torch.full_like(kp, float("nan"))
    table = torch.full((B, max_pages), -1, dtype=torch.int32)
    nxt = 0
    for b in range(B):
        for pg in range(per_seq[b]):
            idx = order[nxt]; nxt += 1
            table[b, pg] = idx
            r0 = pg * page_rows
            r1 = min(r0 + page_rows, cap)
            kp[idx, :, :r1 - r0] = kc[b, :, r0:r1]
            vp[idx, :, :r1 - r0] = vc[b, :, r0:r1]
    table[table < 0] = 0                                        # unread entries must still be valid indices
    return kp, vp, table.cuda()


@pytest.mark.parametrize("Hq,Hkv,D", [(9, 3, 64), (32, 8, 128), (8, 1, 128), (4, 4, 64)])
@pytest.mark.parametrize("page_rows", [32, 256])
def test_paged_equals_contiguous_and_ground_truth(Hq, Hkv, D, page_rows):
    lens = np.array([1, 31, 32, 33, 255, 256, 257, 1000, 0, 4096, 5, 2049], np.int32)
    B, cap = len(lens), 4096
    g = torch.Generator(device="cuda").manual_seed(31 + page_rows + D)
    kc = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    vc = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    q = torch.randn(B, Hq * D, generator=g, device="cuda").bfloat16()
    sl = torch.from_numpy(lens).cuda()
    geom = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=cap, seq_len=sl)
    # chunk_rows = 0 on a bf16 cache: the same balanced kernel the paged entry point runs
    flat, flat_rec = A.decode_batch(q, kc, vc, seq_stride=Hkv * cap * D, head_stride=cap * D, partials=True, **geom)
    kp, vp, table = _paged_copy(kc, vc, lens, page_rows, torch.Generator().manual_seed(5))
    paged, paged_rec = A.decode_paged(q, kp, vp, table, partials=True, **geom)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(paged), host(flat))
    np.testing.assert_array_equal(host(paged_rec)[:, :D + 2], host(flat_rec)[:, :D + 2])
    assert np.isfinite(host(paged)).all()                      # no NaN page was touched
    bits = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    ref = O.decode_batch(host(q), bits(kc), bits(vc), np.arange(B, dtype=np.int64) * Hkv * cap * D,
                         np.full(B, cap * D, np.int64), lens, Hq, Hkv, D, 1 / np.sqrt(D), acc64=True)
    assert_close(host(paged), ref, TOL_BF16, "paged decode vs fp64 ground truth")


def test_paged_append_then_decode():
    """A new token per sequence goes through the paged append, then the paged decode attends it:
    equal to doing the same on a contiguous cache."""
    Hq, Hkv, D, page_rows, cap = 9, 3, 64, 64, 512
    lens = np.array([63, 64, 65, 200, 0, 511], np.int32)        # rows already cached; the new token is row lens[b]
    B = len(lens)
    g = torch.Generator(device="cuda").manual_seed(77)
    kc = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    vc = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    for b in range(B):                                          # rows at and past the length are not history
        kc[b, :, lens[b]:] = 0; vc[b, :, lens[b]:] = 0
    kp, vp, table = _paged_copy(kc, vc, lens + 1, page_rows, torch.Generator().manual_seed(9))
    kp = torch.nan_to_num(kp); vp = torch.nan_to_num(vp)
    cos, sin = A.rope_tables(cap, D, 10000.0)
    pos = torch.from_numpy(lens).cuda()
    acts = [torch.randn(B, 1, n * D, generator=g, device="cuda") for n in (Hq, Hkv, Hkv)]
    q1, k1, v1 = (a.clone() for a in acts)
    A.rope_append(q1, k1, v1, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, seq_pos=pos, k_cache=kc, v_cache=vc,
                  seq_stride=Hkv * cap * D, head_stride=cap * D, max_seq=cap)
    flat = A.decode_batch(q1.view(B, Hq * D), kc, vc, n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=cap, seq_len=pos + 1,
                          seq_stride=Hkv * cap * D, head_stride=cap * D)
    q2, k2, v2 = (a.clone() for a in acts)
    A.rope_append_paged(q2, k2, v2, cos, sin, kp, vp, table, n_head=Hq, n_kv_head=Hkv, head_dim=D, seq_pos=pos)
    paged = A.decode_paged(q2.view(B, Hq * D), kp, vp, table, n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=cap,
                           seq_len=pos + 1)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(host(paged), host(flat))


def test_paged_append_of_several_tokens_crosses_pages_and_stays_in_the_pool():
    """Appends of n = 70 tokens starting near page ends: every row must land in its own page (the
    pool afterwards equals a paged copy of the contiguous cache), rows past the table and rows
    whose table entry is unassigned (-1) or outside the pool are dropped, guard pages stay intact."""
    Hq, Hkv, D, page_rows, cap, n = 4, 2, 64, 32, 256, 70
    pos0 = np.array([0, 30, 63, 150, 200], np.int32)            # 200 + 70 > 256: the tail is past the table
    B = len(pos0)
    g = torch.Generator(device="cuda").manual_seed(78)
    kc = torch.zeros(B, Hkv, cap, D, device="cuda").bfloat16()
    vc = torch.zeros_like(kc)
    max_pages = cap // page_rows
    n_pool = B * max_pages + 2                                   # two guard pages nobody owns
    perm = torch.randperm(B * max_pages, generator=torch.Generator().manual_seed(10)).to(torch.int32)
    table = perm.view(B, max_pages).cuda()
    table[3, 6] = -1                                             # rows 192..223 of sequence 3: unassigned
    table[1, 2] = n_pool + 5                                     # rows 64..95 of sequence 1: outside the pool
    kp = torch.zeros(n_pool, Hkv, page_rows, D, device="cuda").bfloat16()
    vp = torch.zeros_like(kp)
    kp[-2:] = 7.0; vp[-2:] = 7.0
    cos, sin = A.rope_tables(cap + n, D, 10000.0)
    pos = torch.from_numpy(pos0).cuda()
    acts = [torch.randn(B, n, h * D, generator=g, device="cuda").bfloat16() for h in (Hq, Hkv, Hkv)]
    q1, k1, v1 = (a.clone() for a in acts)
    A.rope_append(q1, k1, v1, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, seq_pos=pos, k_cache=kc, v_cache=vc,
                  seq_stride=Hkv * cap * D, head_stride=cap * D, max_seq=cap)
    q2, k2, v2 = (a.clone() for a in acts)
    A.rope_append_paged(q2, k2, v2, cos, sin, kp, vp, table, n_head=Hq, n_kv_head=Hkv, head_dim=D, seq_pos=pos)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(bf16_bits(q1), bf16_bits(q2))
    np.testing.assert_array_equal(bf16_bits(k1), bf16_bits(k2))
    tab = table.cpu().numpy()
    for b in range(B):
        for r in range(max_pages):
            pg = int(tab[b, r])
            want_k = kc[b, :, r * page_rows:(r + 1) * page_rows]
            want_v = vc[b, :, r * page_rows:(r + 1) * page_rows]
            if pg < 0 or pg >= n_pool:
                continue                                          # dropped rows: nothing to compare, nothing written
            np.testing.assert_array_equal(bf16_bits(kp[pg]), bf16_bits(want_k))
            np.testing.assert_array_equal(bf16_bits(vp[pg]), bf16_bits(want_v))
    assert (kp[-2:] == 7.0).all() and (vp[-2:] == 7.0).all()
    # the page whose table entry was redirected received nothing either
    orphan = int(perm.view(B, max_pages)[1, 2])
    assert not kp[orphan].any() and not vp[orphan].any()


def test_paged_argument_checks():
    z = torch.zeros(2, 2 * 64, dtype=torch.bfloat16, device="cuda")
    pages = torch.zeros(4, 1, 48, 64, dtype=torch.bfloat16, device="cuda")          # 48 rows: not a power of two
    table = torch.zeros(2, 2, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="page_rows"):
        A.decode_paged(z, pages, pages, table, n_head=2, n_kv_head=1, head_dim=64, max_len=64)
    pages = torch.zeros(4, 1, 64, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="cannot hold"):
        A.decode_paged(z, pages, pages, table, n_head=2, n_kv_head=1, head_dim=64, max_len=1000)
