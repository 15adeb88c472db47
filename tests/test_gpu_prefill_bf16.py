"""GPU parity of the tcgen05 causal prefill kernel (bf16, D = 128), through the C ABI,
against float64 ground truth computed on the same bf16-rounded inputs (bound 2e-2)."""
import numpy as np
import pytest
import torch

from gpu_util import host
from nimllm_b200 import attention as A
from oracle import oracle as O
from util import SEED_C4, TOL_BF16, assert_close

pytestmark = pytest.mark.gpu
D = 128
BASE = 500000.0


def _inputs(seed, B, S, Hq, Hkv):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, S, Hq * D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv * D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv * D, generator=g, device="cuda").bfloat16()
    return q, k, v


def _rotated_reference(q, k, S, Hq, Hkv, pos0=0):
    """RoPE in fp32 on the bf16 inputs, rounded to bf16 as the kernels store / stage them."""
    qf, kf = host(q).copy(), host(k).copy()
    cos, sin = O.rope_tables(pos0 + S, D, BASE)
    for b in range(qf.shape[0]):
        O.rope_fwd(qf[b], cos[pos0:], sin[pos0:], Hq, D)
        O.rope_fwd(kf[b], cos[pos0:], sin[pos0:], Hkv, D)
    return O.from_bf16(O.to_bf16(qf)), O.from_bf16(O.to_bf16(kf))


def _status_ok():
    """No bounded wait inside a bf16 prefill launch has given up (sticky per-device word, cleared here)."""
    return A.prefill_status(reset=True) == 0


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 1, 1), (1, 256, 4, 1), (2, 384, 8, 2), (1, 300, 4, 2),
                                        (1, 1, 4, 4), (1, 129, 2, 1), (1, 1000, 8, 2), (3, 512, 4, 4)])
@pytest.mark.parametrize("rope,save_cache", [(False, False), (True, False), (True, True)])
def test_prefill_bf16_shapes(B, S, Hq, Hkv, rope, save_cache):
    q, k, v = _inputs(500 + S, B, S, Hq, Hkv)
    q0, k0 = q.clone(), k.clone()
    cos, sin = A.rope_tables(S, D, BASE) if rope else (None, None)
    lse = torch.zeros(B, Hq, S, device="cuda")
    out = A.attn_forward(q, k, v, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, save_cache=save_cache, lse=lse)
    torch.cuda.synchronize()
    assert _status_ok()
    if rope:
        qf, kf = _rotated_reference(q0, k0, S, Hq, Hkv)
        np.testing.assert_array_equal(host(k), kf)               # K rotated in place, bit-exact bf16
        if save_cache:
            np.testing.assert_array_equal(host(q), qf)           # saveCache: post-RoPE Q left for backward()
    else:
        qf, kf = host(q0), host(k0)
    ref = O.prefill_f64(qf, kf, host(v), Hq, Hkv, D, 1 / np.sqrt(D))
    assert_close(host(out), ref, TOL_BF16, "prefill bf16")
    # log-sum-exp of the last row of the last head
    b, h, i = B - 1, Hq - 1, S - 1
    kvh = h // (Hq // Hkv)
    s = (qf[b, i, h * D:(h + 1) * D].astype(np.float64) @ kf[b, :, kvh * D:(kvh + 1) * D].astype(np.float64).T) / np.sqrt(D)
    assert abs(host(lse)[b, h, i] - (np.log(np.exp(s - s.max()).sum()) + s.max())) < 2e-2


def test_prefill_fills_bf16_cache_and_decode_continues():
    """Prefill fills the KV cache (K rotated, V raw); a decode step on the cache then equals
    the next row of a longer causal attention."""
    B, S, Hq, Hkv = 2, 260, 8, 2
    q, k, v = _inputs(600, B, S + 1, Hq, Hkv)
    cos, sin = A.rope_tables(S + 1, D, BASE)
    qf, kf = _rotated_reference(q, k, S + 1, Hq, Hkv)
    ref = O.prefill_f64(qf, kf, host(v), Hq, Hkv, D, 1 / np.sqrt(D))
    kv = A.KvCache(1, B, Hkv, S + 8, D, torch.bfloat16)
    qp, kp, vp = q[:, :S].contiguous(), k[:, :S].contiguous(), v[:, :S].contiguous()
    out = A.attn_forward(qp, kp, vp, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, kv=kv, save_cache=False)
    kv.pos = S
    assert_close(host(out), ref[:, :S], TOL_BF16, "prefill rows")
    np.testing.assert_array_equal(host(kv.k[0, :, :, :S]).transpose(0, 2, 1, 3).reshape(B, S, Hkv * D), kf[:, :S])
    np.testing.assert_array_equal(host(kv.v[0, :, :, :S]).transpose(0, 2, 1, 3).reshape(B, S, Hkv * D), host(v)[:, :S])
    qn, kn, vn = q[:, S].float().contiguous(), k[:, S].float().contiguous(), v[:, S].float().contiguous()
    step = A.attn_forward_cached(kv, 0, qn, kn, vn, cos, sin, n_head=Hq)
    assert_close(host(step), ref[:, S], TOL_BF16, "decode step after prefill")


def test_c4_shape_sampled_rows_and_determinism():
    """Full C4 shape (4 x 8192, 32q/8kv): sampled (batch, head, row) outputs against float64
    ground truth, and bit-identical results on a second run."""
    B, S, Hq, Hkv = 4, 8192, 32, 8
    q, k, v = _inputs(SEED_C4, B, S, Hq, Hkv)
    q0 = q.clone()
    cos, sin = A.rope_tables(S, D, BASE)
    out = A.attn_forward(q, k, v, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, save_cache=False)
    torch.cuda.synchronize()
    assert _status_ok()
    # k is now rotated; a second run must not rotate it again: pass no tables for K by
    # running on rotated copies through the no-RoPE path
    qf_all = None
    rows = [0, 1, 127, 128, 255, 256, 4095, 4096, 8191]
    for b, h in [(0, 0), (1, 13), (3, 31)]:
        kvh = h // 4
        qh = q0[b:b + 1, :, h * D:(h + 1) * D].contiguous()
        qrot, _ = _rotated_reference(qh, k[b:b + 1, :, kvh * D:(kvh + 1) * D].contiguous() * 0, S, 1, 1)
        kh = host(k[b:b + 1, :, kvh * D:(kvh + 1) * D])
        vh = host(v[b:b + 1, :, kvh * D:(kvh + 1) * D])
        for i in rows:
            ref = O.prefill_f64(qrot, kh, vh, 1, 1, D, 1 / np.sqrt(D), row0=i, row1=i + 1)[0, 0]
            assert_close(host(out[b, i, h * D:(h + 1) * D]), ref, TOL_BF16, f"b={b} h={h} row={i}")
    # determinism: same rotated K, Q rotated in the prologue again from the original values
    out2 = A.attn_forward(q0.clone(), k, v, None, None, n_head=Hq, n_kv_head=Hkv, head_dim=D, save_cache=False)
    q_rot = q0.clone()
    out3 = A.attn_forward(q_rot, k.clone(), v, None, None, n_head=Hq, n_kv_head=Hkv, head_dim=D, save_cache=False)
    assert torch.equal(out2, out3)


def test_unsupported_head_dim_is_an_error_not_a_fallback():
    q = torch.zeros(1, 128, 32, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(Exception, match="head_dim"):
        A.attn_forward(q, q.clone(), q.clone(), None, None, n_head=1, n_kv_head=1, head_dim=32)


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 128, 3, 1), (2, 384, 9, 3), (1, 300, 6, 3), (1, 1000, 9, 3), (1, 1, 3, 3)])
@pytest.mark.parametrize("rope,save_cache", [(False, False), (True, True)])
def test_prefill_bf16_head_dim_64(B, S, Hq, Hkv, rope, save_cache):
    """The reference's own model shape (9 q / 3 kv heads of 64, RoPE base 10000) in bf16."""
    d, base = 64, 10000.0
    g = torch.Generator(device="cuda").manual_seed(900 + S)
    q = torch.randn(B, S, Hq * d, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, S, Hkv * d, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, S, Hkv * d, generator=g, device="cuda").bfloat16()
    q0, k0 = host(q).copy(), host(k).copy()
    cos, sin = A.rope_tables(S, d, base) if rope else (None, None)
    out = A.attn_forward(q, k, v, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=d, save_cache=save_cache)
    torch.cuda.synchronize()
    assert _status_ok()
    if rope:
        ct, st = O.rope_tables(S, d, base)
        for b in range(B):
            O.rope_fwd(q0[b], ct, st, Hq, d)
            O.rope_fwd(k0[b], ct, st, Hkv, d)
        q0, k0 = O.from_bf16(O.to_bf16(q0)), O.from_bf16(O.to_bf16(k0))
        np.testing.assert_array_equal(host(k), k0)
        np.testing.assert_array_equal(host(q), q0)           # save_cache leaves the rotated Q
    ref = O.prefill_f64(q0, k0, host(v), Hq, Hkv, d, 1 / np.sqrt(d))
    assert_close(host(out), ref, TOL_BF16, "prefill bf16, head_dim 64")
