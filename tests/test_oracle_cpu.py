"""CPU tests of the oracle (oracle/attn_oracle.c): against the committed golden vectors,
against float64 NumPy restatements, and through the properties the decode path relies on."""
import hashlib
import os

import numpy as np
import pytest

from oracle import oracle as O
from util import TOL_F32, assert_close, normal, rel_err

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "attn_f64_golden.npz")


def _case(g, name):
    seed, S, Hq, Hkv, D = [int(x) for x in g[f"{name}_meta"]]
    q = normal(seed, 0, (S, Hq * D)); k = normal(seed, 1, (S, Hkv * D)); v = normal(seed, 2, (S, Hkv * D))
    h = hashlib.sha256()
    for a in (q, k, v):
        h.update(a.tobytes())
    assert h.hexdigest() == bytes(g[f"{name}_sha"]).decode(), "seeded inputs drifted from the fixture"
    return q, k, v, S, Hq, Hkv, D, float(g[f"{name}_base"]), g[f"{name}_rows"]


@pytest.mark.parametrize("name", ["c1", "llama", "mha"])
def test_forward_matches_f64_golden(name):
    g = np.load(GOLD)
    q, k, v, S, Hq, Hkv, D, base, rows = _case(g, name)
    cos, sin = O.rope_tables(S, D, base)
    out, q_rot, k_rot = O.attn_forward(q, k, v, cos, sin, Hq, Hkv, D)
    # the fixture takes cos/sin in float64 of the fp32 angle; one ulp of a 160-radian fp32 angle
    # is 1.5e-5, so the stated fp32 bound (1e-4) is the meaningful one here
    assert_close(out[rows], g[f"{name}_out"], TOL_F32, f"{name} attnOut")
    assert_close(k_rot[rows], g[f"{name}_krot"], TOL_F32, f"{name} rotated K")


@pytest.mark.parametrize("name", ["c1", "llama"])
def test_prefill_then_cached_decode_matches_golden(name):
    """Prefill on the first rows, then one forwardCached step per remaining row."""
    g = np.load(GOLD)
    q, k, v, S, Hq, Hkv, D, base, rows = _case(g, name)
    n_pre = S * 4 // 5
    cos, sin = O.rope_tables(S, D, base)
    out = np.zeros((S, Hq * D), np.float32)
    o, _, k_rot = O.attn_forward(q[:n_pre], k[:n_pre], v[:n_pre], cos, sin, Hq, Hkv, D)
    out[:n_pre] = o
    kv = O.KvCache(Hkv, D, S)
    kv.fill(k_rot, v[:n_pre])
    for t in range(n_pre, S):
        out[t] = O.attn_forward_cached(kv, q[t], k[t], v[t], cos, sin, Hq)
    assert kv.pos == S
    assert_close(out[rows], g[f"{name}_out"], TOL_F32, f"{name} prefill+decode")
    krows = kv.k.transpose(1, 0, 2).reshape(S, Hkv * D)
    assert_close(krows[rows], g[f"{name}_krot"], TOL_F32, f"{name} cache K")
    np.testing.assert_array_equal(kv.v.transpose(1, 0, 2).reshape(S, Hkv * D), v)


def test_rope_tables_formula():
    cos, sin = O.rope_tables(300, 64, 10000.0)
    pos = np.arange(300, dtype=np.float64)[:, None]
    f = np.arange(32, dtype=np.float64)[None, :]
    theta = pos / 10000.0 ** (2 * f / 64)
    # fp32 angles: absolute error grows with the position (ulp of theta)
    assert np.abs(cos - np.cos(theta)).max() < 3e-5
    assert np.abs(sin - np.sin(theta)).max() < 3e-5
    assert cos[0].tolist() == [1.0] * 32 and sin[0].tolist() == [0.0] * 32


def test_softmax_rows():
    x = normal(5, 0, (7, 301), 3.0)
    y = O.softmax_fwd(x)
    e = np.exp(x.astype(np.float64) - x.max(1, keepdims=True))
    ref = e / e.sum(1, keepdims=True)
    assert_close(y, ref, 1e-6, "softmax")
    # one column and a power-of-two width (thread-count edge cases of the reference kernel)
    assert O.softmax_fwd(np.array([[3.0]], np.float32))[0, 0] == 1.0
    assert abs(O.softmax_fwd(normal(6, 0, (2, 256))).sum(1) - 1).max() < 1e-6


def test_masked_scores_vanish_exactly():
    """-1e9 masking (src/kernels.cu:255) equals exclusion: exp underflows to exactly 0."""
    S, D = 9, 64
    q = normal(7, 0, (S, D)); k = normal(7, 1, (S, D)); v = normal(7, 2, (S, D))
    cos, sin = O.rope_tables(S, D, 10000.0)
    out, _, _ = O.attn_forward(q, k, v, cos, sin, 1, 1, D, apply_rope=False)
    ref = O.prefill_f64(q[None], k[None], v[None], 1, 1, D, 1 / np.sqrt(D))[0]
    assert_close(out, ref, 1e-5, "masking")
    assert_close(out[0], v[0], 1e-6, "row 0 attends itself only")


def _ragged(seed, B, Hq, Hkv, D, lens, bf16=False):
    cap = int(max(lens))
    off = np.zeros(B, np.int64); hs = np.zeros(B, np.int64)
    total = 0
    for b in range(B):
        off[b] = total; hs[b] = max(int(lens[b]), 1) * D
        total += Hkv * hs[b]
    k = normal(seed, 10, (total,)); v = normal(seed, 11, (total,)); q = normal(seed, 12, (B, Hq * D))
    if bf16:
        k, v = O.to_bf16(k), O.to_bf16(v)
    return q, k, v, off, hs, np.asarray(lens, np.int32), cap


def test_decode_batch_f32_vs_f64_and_bf16():
    B, Hq, Hkv, D = 5, 9, 3, 64
    q, k, v, off, hs, lens, _ = _ragged(11, B, Hq, Hkv, D, [1, 2, 63, 64, 130])
    o32 = O.decode_batch(q, k, v, off, hs, lens, Hq, Hkv, D, 0.125)
    o64 = O.decode_batch(q, k, v, off, hs, lens, Hq, Hkv, D, 0.125, acc64=True)
    assert_close(o32, o64, 1e-5, "decode fp32 vs fp64")
    # length 1: the output is the single V row of the KV head
    np.testing.assert_allclose(o64[0, :D], v[off[0]:off[0] + D], rtol=1e-6)
    kb, vb = O.to_bf16(k), O.to_bf16(v)
    ob = O.decode_batch(q, kb, vb, off, hs, lens, Hq, Hkv, D, 0.125, acc64=True)
    ow = O.decode_batch(q, O.from_bf16(kb), O.from_bf16(vb), off, hs, lens, Hq, Hkv, D, 0.125, acc64=True)
    np.testing.assert_array_equal(ob, ow)


def test_zero_length_sequence_gives_zeros():
    q, k, v, off, hs, lens, _ = _ragged(12, 2, 4, 2, 64, [0, 3])
    o, m, l = O.decode_batch(q, k, v, off, hs, lens, 4, 2, 64, 0.125, want_ml=True)
    assert not o[0].any() and l[0].max() == 0 and np.isneginf(m[0]).all()


@pytest.mark.parametrize("n_parts", [1, 2, 3, 8])
def test_split_kv_combine_equals_unsplit(n_parts):
    """Splitting the KV rows into contiguous shards and merging (m, l, o) equals the
    unsplit softmax -- the property split-KV and KV-sequence sharding rest on."""
    B, Hq, Hkv, D, L = 3, 8, 2, 128, 257
    q, k, v, off, hs, lens, _ = _ragged(13, B, Hq, Hkv, D, [L] * B)
    full = O.decode_batch(q, k, v, off, hs, lens, Hq, Hkv, D, 0.09, acc64=True)
    W = D + 4
    parts = np.zeros((n_parts, B * Hq, W), np.float32)
    bounds = np.linspace(0, L, n_parts + 1).astype(int)
    for p in range(n_parts):
        r0, r1 = bounds[p], bounds[p + 1]
        o, m, l = O.decode_batch(q, k, v, off + r0 * D, hs, np.full(B, r1 - r0, np.int32), Hq, Hkv, D, 0.09,
                                 acc64=True, want_ml=True)
        parts[p, :, :D] = o.reshape(B * Hq, D); parts[p, :, D] = m.reshape(-1); parts[p, :, D + 1] = l.reshape(-1)
    out, m, l = O.combine(parts, D)
    assert_close(out.reshape(B, Hq * D), full, 1e-5, "combine")


def test_combine_ignores_empty_parts():
    D, W = 64, 68
    parts = np.zeros((3, 2, W), np.float32)
    parts[0, :, :D] = 1.0; parts[0, :, D] = 0.5; parts[0, :, D + 1] = 2.0
    parts[1, :, D] = -np.inf  # empty shard: l = 0
    parts[2, :, :D] = 3.0; parts[2, :, D] = 0.5; parts[2, :, D + 1] = 2.0
    out, m, l = O.combine(parts, D)
    np.testing.assert_allclose(out, 2.0, rtol=1e-6)
    np.testing.assert_allclose(l, 4.0, rtol=1e-6)


def test_bf16_rounding_is_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.4e38, 1e-40], np.float32)
    import torch
    ref = torch.tensor(x).bfloat16().view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(O.to_bf16(x), ref)


def test_legacy_pieces_restate_reference_kernels():
    S, E, H, D = 6, 192, 3, 64
    x = normal(14, 0, (S, E))
    dst = np.zeros((S, D), np.float32)
    O.lib().oracle_extract_kv_head(x, dst, 7, 3, S, E, D)      # q head 7 of kvRepeat 3 -> KV head 2
    np.testing.assert_array_equal(dst, x[:, 2 * D:3 * D])
    back = np.zeros_like(x)
    O.lib().oracle_insert_head(dst, back, 1, S, E, D)
    np.testing.assert_array_equal(back[:, D:2 * D], dst)
    sc = normal(14, 1, (5, 5)); ref = sc.copy()
    O.lib().oracle_causal_mask(sc, 0.125, 5)
    assert (sc[np.triu_indices(5, 1)] == np.float32(-1e9)).all()
    np.testing.assert_array_equal(sc[np.tril_indices(5)], (ref * np.float32(0.125))[np.tril_indices(5)])


def test_attention_backward_matches_autograd_of_an_independent_formulation():
    """The restated backward (src/model.nim:639-685) against float64 autograd through a plain
    softmax(QK^T)V with rotate-half RoPE written independently in torch."""
    import torch
    from oracle import oracle as O
    S, Hq, Hkv, D = 37, 6, 2, 32
    G = Hq // Hkv
    rng = np.random.default_rng(5)
    q = rng.standard_normal((S, Hq * D)).astype(np.float32)
    k = rng.standard_normal((S, Hkv * D)).astype(np.float32)
    v = rng.standard_normal((S, Hkv * D)).astype(np.float32)
    dout = rng.standard_normal((S, Hq * D)).astype(np.float32)
    cos, sin = O.rope_tables(S, D, 10000.0)

    def rope(x, n_head):
        x = x.view(S, n_head, D)
        c = torch.from_numpy(cos).double()[:, None, :]; s_ = torch.from_numpy(sin).double()[:, None, :]
        x0, x1 = x[..., :D // 2], x[..., D // 2:]
        return torch.cat([x0 * c - x1 * s_, x0 * s_ + x1 * c], dim=-1)

    tq = torch.from_numpy(q).double().requires_grad_(); tk = torch.from_numpy(k).double().requires_grad_()
    tv = torch.from_numpy(v).double().requires_grad_()
    qr, kr = rope(tq, Hq), rope(tk, Hkv)
    vv = tv.view(S, Hkv, D)
    outs = []
    mask = torch.tril(torch.ones(S, S, dtype=torch.bool))
    for h in range(Hq):
        sc = (qr[:, h] @ kr[:, h // G].T) / np.sqrt(D)
        p = torch.softmax(sc.masked_fill(~mask, float("-inf")), dim=-1)
        outs.append(p @ vv[:, h // G])
    out = torch.stack(outs, dim=1).reshape(S, Hq * D)
    out.backward(torch.from_numpy(dout).double())

    q_rot, k_rot = q.copy(), k.copy()
    O.rope_fwd(q_rot, cos, sin, Hq, D); O.rope_fwd(k_rot, cos, sin, Hkv, D)
    for acc64, tol in ((True, 2e-6), (False, 2e-5)):
        dq, dk, dv = O.attn_backward(q_rot, k_rot, v, dout, cos, sin, Hq, Hkv, D, acc64=acc64)
        for name, got, want in (("dq", dq, tq.grad), ("dk", dk, tk.grad), ("dv", dv, tv.grad)):
            want = want.numpy()
            err = np.abs(got - want).max() / np.abs(want).max()
            assert err <= tol, f"{name} acc64={acc64}: {err:.3e}"
