"""GPU parity of the reference-named launchers and of the fused RoPE/append kernel."""
import numpy as np
import pytest
import torch

from gpu_util import bf16_bits, dev, host, wrap_ptr
from nimllm_b200 import _lib, attention as A
from oracle import oracle as O
from util import TOL_F32, assert_close, normal

pytestmark = pytest.mark.gpu


def test_legacy_launchers_match_oracle():
    L = _lib.lib()
    S, Hq, Hkv, D = 37, 9, 3, 64
    E, Ekv = Hq * D, Hkv * D
    x = normal(400, 0, (S, E))
    cos, sin = O.rope_tables(S, D, 10000.0)
    d, dcos, dsin = dev(x), dev(cos), dev(sin)      # named: a temporary would be freed before the launch
    L.gpu_rope_fwd(d.data_ptr(), dcos.data_ptr(), dsin.data_ptr(), S, E, Hq, D)
    ref = O.rope_fwd(x.copy(), cos, sin, Hq, D)
    assert_close(host(d), ref, 1e-6, "gpu_rope_fwd")

    head = torch.zeros(S, D, device="cuda")
    L.gpu_extract_head(d.data_ptr(), head.data_ptr(), 4, S, E, D)
    np.testing.assert_array_equal(host(head), host(d)[:, 4 * D:5 * D])
    kk = dev(normal(400, 1, (S, Ekv)))
    L.gpu_extract_kv_head(kk.data_ptr(), head.data_ptr(), 7, 3, S, Ekv, D)
    np.testing.assert_array_equal(host(head), host(kk)[:, 2 * D:3 * D])
    dst = torch.zeros(S, E, device="cuda")
    L.gpu_insert_head(head.data_ptr(), dst.data_ptr(), 5, S, E, D)
    np.testing.assert_array_equal(host(dst)[:, 5 * D:6 * D], host(head))
    assert not host(dst)[:, :5 * D].any()

    sc = normal(400, 2, (S, S))
    dsc = dev(sc)
    L.gpu_causal_mask(dsc.data_ptr(), 0.125, S)
    ref = sc.copy(); O.lib().oracle_causal_mask(ref, 0.125, S)
    np.testing.assert_array_equal(host(dsc), ref)
    y = torch.zeros(S, S, device="cuda")
    L.gpu_softmax_fwd(dsc.data_ptr(), y.data_ptr(), S, S)
    assert_close(host(y), O.softmax_fwd(ref), 1e-6, "gpu_softmax_fwd")
    for cols in (1, 31, 32, 33, 300, 1025):
        xs = normal(401, cols, (3, cols), 2.0)
        ys = torch.zeros(3, cols, device="cuda")
        dxs = dev(xs)
        L.gpu_softmax_fwd(dxs.data_ptr(), ys.data_ptr(), 3, cols)
        assert_close(host(ys), O.softmax_fwd(xs), 1e-6, f"softmax cols={cols}")
    z = torch.zeros(S * S, device="cuda")
    dsc2 = dev(sc)
    L.gpu_scale(dsc2.data_ptr(), 0.3, z.data_ptr(), S * S)
    np.testing.assert_array_equal(host(z), (sc * np.float32(0.3)).reshape(-1))
    torch.cuda.synchronize()


@pytest.mark.parametrize("causal", [1, 0])
def test_gpu_flash_attn_fwd_single_head(causal):
    """The reference's unused fused entry (src/kernels.cu:750): dense [S, hd], one head."""
    S, D = 45, 64
    q = normal(402, 0, (S, D)); k = normal(402, 1, (S, D)); v = normal(402, 2, (S, D))
    o = torch.zeros(S, D, device="cuda")
    dq, dk, dv = dev(q), dev(k), dev(v)
    _lib.lib().gpu_flash_attn_fwd(dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), o.data_ptr(), S, D, 0.125, causal)
    torch.cuda.synchronize()
    if causal:
        ref = O.prefill_f64(q[None], k[None], v[None], 1, 1, D, 0.125)[0]
    else:
        s = (q.astype(np.float64) @ k.astype(np.float64).T) * 0.125
        p = np.exp(s - s.max(1, keepdims=True)); p /= p.sum(1, keepdims=True)
        ref = p @ v.astype(np.float64)
    assert_close(host(o), ref, TOL_F32, "gpu_flash_attn_fwd")


@pytest.mark.parametrize("act,cache", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                       (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_rope_append_batch_with_positions(act, cache):
    B, n, Hq, Hkv, D, max_seq = 3, 2, 8, 2, 128, 40
    pos = np.array([0, 17, 38], np.int32)
    q = normal(403, 0, (B, n, Hq * D)); k = normal(403, 1, (B, n, Hkv * D)); v = normal(403, 2, (B, n, Hkv * D))
    if act == torch.bfloat16:
        q, k, v = [O.from_bf16(O.to_bf16(x)) for x in (q, k, v)]
    cos, sin = A.rope_tables(max_seq, D, 500000.0)
    kc = torch.zeros(B, Hkv, max_seq, D, dtype=cache, device="cuda"); vc = torch.zeros_like(kc)
    dq, dk, dv = dev(q, act), dev(k, act), dev(v, act)
    A.rope_append(dq, dk, dv, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, seq_pos=dev(pos), k_cache=kc,
                  v_cache=vc, seq_stride=Hkv * max_seq * D, head_stride=max_seq * D, max_seq=max_seq)
    torch.cuda.synchronize()
    ocos, osin = O.rope_tables(max_seq, D, 500000.0)
    tol = 1e-6 if act == torch.float32 else 8e-3
    for b in range(B):
        p = int(pos[b])
        qr = O.rope_fwd(q[b].copy(), ocos[p:], osin[p:], Hq, D)
        kr = O.rope_fwd(k[b].copy(), ocos[p:], osin[p:], Hkv, D)
        assert_close(host(dq[b]), qr, tol, "q rotated")
        assert_close(host(dk[b]), kr, tol, "k written back")
        ck, cv = host(kc[b]), host(vc[b])          # [Hkv, max_seq, D]
        ctol = 1e-6 if (act == torch.float32 and cache == torch.float32) else 8e-3
        for t in range(n):
            if p + t < max_seq:
                assert_close(ck[:, p + t].reshape(-1), kr[t], ctol, "cache K row")
                assert_close(cv[:, p + t].reshape(-1), v[b, t], ctol, "cache V row")
        untouched = np.ones(max_seq, bool); untouched[p:p + n] = False
        assert not ck[:, untouched].any() and not cv[:, untouched].any()
    # the last sequence's second token (position 39) fits; position 40 would not be stored
    assert host(kc[2])[:, 39].any()


def test_rope_append_exact_cast_and_shard_rows():
    """fp32 -> bf16 cache rounding is round-to-nearest-even, and a KV-sequence shard keeps
    only rows [cache_row0, cache_row0 + max_seq)."""
    B, Hkv, D, rows = 1, 2, 64, 8
    v = normal(404, 0, (B, 1, Hkv * D)); k = normal(404, 1, (B, 1, Hkv * D))
    for pos, stored in ((13, True), (5, False), (16, False)):
        kc = torch.zeros(B, Hkv, rows, D, dtype=torch.bfloat16, device="cuda"); vc = torch.zeros_like(kc)
        A.rope_append(None, dev(k), dev(v), None, None, n_head=0, n_kv_head=Hkv, head_dim=D, pos0=pos, k_cache=kc,
                      v_cache=vc, seq_stride=Hkv * rows * D, head_stride=rows * D, cache_row0=8, max_seq=rows)
        torch.cuda.synchronize()
        if stored:
            np.testing.assert_array_equal(bf16_bits(vc[0, :, pos - 8]).reshape(-1), O.to_bf16(v.reshape(-1)))
            np.testing.assert_array_equal(bf16_bits(kc[0, :, pos - 8]).reshape(-1), O.to_bf16(k.reshape(-1)))
        else:
            assert not host(kc).any() and not host(vc).any()


def test_kvcache_handle_api():
    """nimllm_kvcache_* : layout, zero fill, reset, pos bookkeeping (src/model.nim:729-746)."""
    L = _lib.lib()
    h = L.nimllm_kvcache_create(2, 3, 2, 16, 64, _lib.F32)
    assert h
    assert L.nimllm_kvcache_seq_stride(h) == 2 * 16 * 64 and L.nimllm_kvcache_head_stride(h) == 16 * 64
    assert L.nimllm_kvcache_pos(h) == 0
    k1 = L.nimllm_kvcache_k(h, 1); k0 = L.nimllm_kvcache_k(h, 0)
    assert k1 - k0 == 3 * 2 * 16 * 64 * 4
    assert L.nimllm_kvcache_k(h, 2) is None
    # append through the ABI into layer 1, then read the block back with a plain copy
    k = normal(405, 0, (3, 1, 128)); v = normal(405, 1, (3, 1, 128))
    dk, dv = dev(k), dev(v)
    _lib.check(L.nimllm_rope_append(None, 0, dk.data_ptr(), dv.data_ptr(), _lib.F32, 0, None, None, None, 5,
                                    k1, L.nimllm_kvcache_v(h, 1), _lib.F32, None, L.nimllm_kvcache_seq_stride(h),
                                    L.nimllm_kvcache_head_stride(h), 0, 16, 3, 1, 2, 64, None))
    L.nimllm_kvcache_set_pos(h, 6)
    assert L.nimllm_kvcache_pos(h) == 6
    torch.cuda.synchronize()
    back = wrap_ptr(k1, (3, 2, 16, 64))
    np.testing.assert_array_equal(host(back)[:, :, 5].reshape(3, 128), k.reshape(3, 128))
    assert not host(back)[:, :, :5].any()
    _lib.check(L.nimllm_kvcache_reset(h, None))
    torch.cuda.synchronize()
    assert not host(wrap_ptr(k1, (3, 2, 16, 64))).any() and L.nimllm_kvcache_pos(h) == 0
    L.nimllm_kvcache_destroy(h)
