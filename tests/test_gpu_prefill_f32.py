"""GPU parity of the fp32 path (C ABI) against the CPU oracle, the committed golden
vectors and -- where oracle/_ref is present -- the reference's own compiled kernels."""
import os

import numpy as np
import pytest
import torch

from gpu_util import dev, host
from nimllm_b200 import _lib, attention as A
from oracle import oracle as O
from util import SEED_C1, TOL_F32, assert_close, normal

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_f64_golden.npz")


def _c1_flow(seed, S, n_pre, Hq, Hkv, D, base, chunk_rows=0):
    """Configuration C1's flow: causal prefill of n_pre tokens (filling the cache), then one
    cached decode step per remaining token.  Returns out [S, Hq*D] and the cache."""
    q = normal(seed, 0, (S, Hq * D)); k = normal(seed, 1, (S, Hkv * D)); v = normal(seed, 2, (S, Hkv * D))
    cos, sin = A.rope_tables(S, D, base)
    kv = A.KvCache(1, 1, Hkv, S, D, torch.float32)
    dq, dk, dv = dev(q), dev(k), dev(v)
    out = torch.zeros(S, Hq * D, device="cuda")
    out[:n_pre] = A.attn_forward(dq[:n_pre], dk[:n_pre], dv[:n_pre], cos, sin, n_head=Hq, n_kv_head=Hkv,
                                 head_dim=D, kv=kv, save_cache=True)
    kv.pos = n_pre
    for t in range(n_pre, S):
        out[t] = A.attn_forward_cached(kv, 0, dq[t:t + 1], dk[t:t + 1], dv[t:t + 1], cos, sin, n_head=Hq,
                                       chunk_rows=chunk_rows)[0]
        kv.pos += 1
    torch.cuda.synchronize()
    return (q, k, v), host(out), host(dq), host(dk), kv


def _oracle_flow(q, k, v, S, n_pre, Hq, Hkv, D, base):
    cos, sin = O.rope_tables(S, D, base)
    out = np.zeros((S, Hq * D), np.float32)
    o, q_rot, k_rot = O.attn_forward(q[:n_pre], k[:n_pre], v[:n_pre], cos, sin, Hq, Hkv, D)
    out[:n_pre] = o
    kv = O.KvCache(Hkv, D, S)
    kv.fill(k_rot, v[:n_pre])
    for t in range(n_pre, S):
        out[t] = O.attn_forward_cached(kv, q[t], k[t], v[t], cos, sin, Hq)
    return out, q_rot, k_rot, kv


def test_c1_prefill_128_then_32_decode_steps():
    S, n_pre, Hq, Hkv, D, base = 160, 128, 9, 3, 64, 10000.0
    (q, k, v), out, q_after, k_after, kv = _c1_flow(SEED_C1, S, n_pre, Hq, Hkv, D, base)
    ref, q_rot, k_rot, okv = _oracle_flow(q, k, v, S, n_pre, Hq, Hkv, D, base)
    assert_close(out, ref, TOL_F32, "C1 attnOut vs oracle")
    # saveCache contract: q and k hold their post-RoPE values (src/model.nim:494-495,534)
    assert_close(q_after[:n_pre], q_rot, 1e-6, "q rotated in place")
    assert_close(k_after[:n_pre], k_rot, 1e-6, "k rotated in place")
    # final cache contents: K rotated, V raw, rows 0..159 (src/model.nim:797-815)
    assert_close(host(kv.k[0, 0]), okv.k, 1e-6, "cache K")
    np.testing.assert_array_equal(host(kv.v[0, 0]), okv.v)
    g = np.load(GOLD)
    assert_close(out[g["c1_rows"]], g["c1_out"], TOL_F32, "C1 attnOut vs float64 golden")


@pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built")
def test_c1_against_reference_compiled_kernels():
    """The reference's own kernels + cuBLAS under the restated Nim loop, same seeded inputs:
    pins the oracle AND is the parity target of the fp32 bound."""
    S, n_pre, Hq, Hkv, D, base = 160, 128, 9, 3, 64, 10000.0
    (q, k, v), out, _, _, kv = _c1_flow(SEED_C1, S, n_pre, Hq, Hkv, D, base)
    cos, sin = O.rope_tables(S, D, base)
    ref = np.zeros((S, Hq * D), np.float32)
    o, q_rot, k_rot = O.ref_attn_forward(q[:n_pre], k[:n_pre], v[:n_pre], cos, sin, Hq, Hkv, D)
    ref[:n_pre] = o
    R = O.ref_lib()
    h = R.ref_kvcache_create(Hkv, D, S, Hq, cos, sin)
    assert R.ref_kvcache_fill(h, k_rot, np.ascontiguousarray(v[:n_pre]), n_pre) == 0
    for t in range(n_pre, S):
        row = np.zeros(Hq * D, np.float32)
        assert R.ref_attn_forward_cached(h, np.ascontiguousarray(q[t]), np.ascontiguousarray(k[t]),
                                         np.ascontiguousarray(v[t]), row, Hq) == 0
        ref[t] = row
    rk = np.zeros((Hkv, S, D), np.float32); rv = np.zeros_like(rk)
    assert R.ref_kvcache_download(h, rk, rv) == 0
    R.ref_kvcache_destroy(h)
    assert_close(out, ref, TOL_F32, "C1 attnOut vs the reference's kernels")
    assert_close(host(kv.k[0, 0]), rk, 1e-6, "cache K vs reference")
    np.testing.assert_array_equal(host(kv.v[0, 0]), rv)
    # and the CPU restatement is pinned by the same run
    oref, _, _, _ = _oracle_flow(q, k, v, S, n_pre, Hq, Hkv, D, base)
    assert_close(oref, ref, 2e-5, "oracle vs the reference's kernels")


@pytest.mark.parametrize("S,Hq,Hkv,D,base", [(1, 9, 3, 64, 10000.0), (17, 9, 3, 64, 10000.0),
                                             (33, 8, 2, 128, 500000.0), (72, 8, 2, 128, 500000.0),
                                             (40, 4, 4, 64, 100000.0), (250, 9, 3, 64, 10000.0)])
def test_prefill_shapes(S, Hq, Hkv, D, base):
    q = normal(200 + S, 0, (S, Hq * D)); k = normal(200 + S, 1, (S, Hkv * D)); v = normal(200 + S, 2, (S, Hkv * D))
    cos, sin = A.rope_tables(S, D, base)
    lse = torch.zeros(1, Hq, S, device="cuda")
    out = A.attn_forward(dev(q), dev(k), dev(v), cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, lse=lse)
    ocos, osin = O.rope_tables(S, D, base)
    ref, q_rot, k_rot = O.attn_forward(q, k, v, ocos, osin, Hq, Hkv, D)
    assert_close(host(out), ref, TOL_F32, "prefill fp32")
    # log-sum-exp of row i of head h, from the rotated inputs in float64
    h, i = Hq - 1, S - 1
    kvh = h // (Hq // Hkv)
    s = (q_rot[i, h * D:(h + 1) * D].astype(np.float64) @ k_rot[:, kvh * D:(kvh + 1) * D].astype(np.float64).T) / np.sqrt(D)
    assert abs(host(lse)[0, h, i] - np.log(np.exp(s - s.max()).sum()) - s.max()) < 1e-4


def test_golden_llama_and_mha_shapes():
    g = np.load(GOLD)
    for name in ("llama", "mha"):
        seed, S, Hq, Hkv, D = [int(x) for x in g[f"{name}_meta"]]
        base = float(g[f"{name}_base"])
        (q, k, v), out, _, k_after, kv = _c1_flow(seed, S, S * 4 // 5, Hq, Hkv, D, base, chunk_rows=64)
        assert_close(out[g[f"{name}_rows"]], g[f"{name}_out"], TOL_F32, f"{name} vs float64 golden")


def test_batched_prefill_with_position_offset():
    """B > 1 and pos0 > 0 (a continuation chunk's RoPE rows); not in the reference (batch 1)."""
    B, S, Hq, Hkv, D, pos0 = 3, 21, 8, 2, 64, 11
    q = normal(300, 0, (B, S, Hq * D)); k = normal(300, 1, (B, S, Hkv * D)); v = normal(300, 2, (B, S, Hkv * D))
    cos, sin = A.rope_tables(pos0 + S, D, 10000.0)
    out = host(A.attn_forward(dev(q), dev(k), dev(v), cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, pos0=pos0))
    ocos, osin = O.rope_tables(pos0 + S, D, 10000.0)
    for b in range(B):
        ref, _, _ = O.attn_forward(q[b], k[b], v[b], ocos[pos0:], osin[pos0:], Hq, Hkv, D)
        assert_close(out[b], ref, TOL_F32, f"batch {b}")


@pytest.mark.parametrize("B,S,Hq,Hkv,D", [(6, 200, 16, 4, 64), (5, 130, 24, 8, 128), (8, 100, 20, 5, 32), (3, 449, 9, 3, 64)])
def test_register_tiled_kernel_on_launches_that_fill_the_gpu(B, S, Hq, Hkv, D):
    """Launches of at least one 64-row query tile per two SMs run the register-tiled fp32 kernel: ragged last
    tiles, a diagonal inside every tile, all three head sizes, batch > 1; output and log-sum-exp."""
    q = normal(400 + S, 0, (B, S, Hq * D)); k = normal(400 + S, 1, (B, S, Hkv * D)); v = normal(400 + S, 2, (B, S, Hkv * D))
    cos, sin = A.rope_tables(S, D, 10000.0)
    lse = torch.zeros(B, Hq, S, device="cuda")
    out = host(A.attn_forward(dev(q), dev(k), dev(v), cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, lse=lse))
    ocos, osin = O.rope_tables(S, D, 10000.0)
    lse_h = host(lse)
    for b in range(B):
        ref, q_rot, k_rot = O.attn_forward(q[b], k[b], v[b], ocos, osin, Hq, Hkv, D)
        assert_close(out[b], ref, TOL_F32, f"tiled prefill fp32, batch {b}")
        for h, i in ((0, 0), (Hq - 1, S - 1), (Hq // 2, 63), (1, 64)):
            kvh = h // (Hq // Hkv)
            sc = (q_rot[i, h * D:(h + 1) * D].astype(np.float64) @ k_rot[:i + 1, kvh * D:(kvh + 1) * D].astype(np.float64).T) / np.sqrt(D)
            assert abs(lse_h[b, h, i] - np.log(np.exp(sc - sc.max()).sum()) - sc.max()) < 1e-4
