"""GPU parity of the decode kernels, called through the C ABI, against the CPU oracle."""
import numpy as np
import pytest
import torch

from gpu_util import bf16_bits, dev, host, ragged_cache
from nimllm_b200 import attention as A
from oracle import oracle as O
from util import SEED_C3, SEED_C5, TOL_BF16, TOL_F32, assert_close, normal, rng

pytestmark = pytest.mark.gpu


# Which kernel serves a call follows from its arguments: an fp32 cache or more than 8 query heads
# per KV head -> the fp32-FMA kernel; a bf16 cache with an explicit chunk_rows -> the mma.sync kernel
# on the chunk grid; a bf16 cache with chunk_rows = 0 -> the balanced mma.sync kernel.


def _run(seed, lens, Hq, Hkv, D, kv_dtype, chunk_rows, q_dtype=torch.float32, pad_rows=3):
    B = len(lens)
    k, v, off, hs = ragged_cache(seed, lens, Hkv, D, kv_dtype, normal, pad_rows)
    q = normal(seed, 12, (B, Hq * D))
    if q_dtype == torch.bfloat16:
        q = O.from_bf16(O.to_bf16(q))
    scale = 1.0 / np.sqrt(D)
    out, rec = A.decode_batch(dev(q, q_dtype), dev(k, kv_dtype), dev(v, kv_dtype), n_head=Hq, n_kv_head=Hkv,
                              head_dim=D, max_len=int(max(max(lens), 1)), seq_len=dev(np.asarray(lens, np.int32)),
                              kv_off=dev(off), head_stride=int(hs[0]), scale=scale, chunk_rows=chunk_rows,
                              partials=True)
    torch.cuda.synchronize()
    ref32 = O.decode_batch(q, k, v, off, hs, np.asarray(lens, np.int32), Hq, Hkv, D, scale)
    ref64, m, l = O.decode_batch(q, k, v, off, hs, np.asarray(lens, np.int32), Hq, Hkv, D, scale, acc64=True,
                                 want_ml=True)
    return host(out), host(rec), ref32, ref64, m, l


LENS = [1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 129, 200, 255, 256, 257, 300]


@pytest.mark.parametrize("Hq,Hkv,D", [(9, 3, 64), (8, 2, 128), (4, 4, 64), (2, 1, 128), (16, 2, 64), (5, 1, 64)])
@pytest.mark.parametrize("chunk_rows", [0, 64, 128])
def test_generic_fp32_cache_matches_reference_arithmetic(Hq, Hkv, D, chunk_rows):
    out, rec, ref32, ref64, m, l = _run(101, LENS, Hq, Hkv, D, torch.float32, chunk_rows)
    assert_close(out, ref32, TOL_F32, "decode fp32 vs oracle fp32")
    assert_close(out, ref64, TOL_F32, "decode fp32 vs oracle fp64")
    assert_close(rec[:, :D].reshape(out.shape), ref64, TOL_F32, "partials o")
    # m + log(l) is the log-sum-exp of the scaled scores, whatever the split
    np.testing.assert_allclose(rec[:, D] + np.log(rec[:, D + 1]), (m + np.log(l)).reshape(-1), atol=2e-4)


@pytest.mark.parametrize("Hq,Hkv,D", [(9, 3, 64), (32, 8, 128), (8, 8, 64), (8, 1, 128), (16, 2, 64),      # mma.sync kernels
                                      (18, 2, 64), (16, 1, 128), (9, 1, 64), (20, 2, 128)])                    # > 8 heads per KV head: fp32 FMA
@pytest.mark.parametrize("chunk_rows", [0, 64, 192])
def test_bf16_cache_matches_f64_ground_truth(Hq, Hkv, D, chunk_rows):
    out, rec, ref32, ref64, m, l = _run(102, LENS, Hq, Hkv, D, torch.bfloat16, chunk_rows, q_dtype=torch.bfloat16)
    assert_close(out, ref64, TOL_BF16, "decode bf16 vs fp64 ground truth")
    np.testing.assert_allclose(rec[:, D] + np.log(rec[:, D + 1]), (m + np.log(l)).reshape(-1), atol=3e-2)


BAL_LENS = [0, 1, 31, 32, 33, 0, 700, 64, 2049, 5, 0, 4096, 16, 333, 1025, 0]


@pytest.mark.parametrize("Hq,Hkv,D", [(9, 3, 64), (32, 8, 128), (8, 8, 64), (8, 1, 128), (16, 2, 64), (3, 1, 128)])
@pytest.mark.parametrize("lens", [LENS, BAL_LENS, [4096], [40000, 3], [0, 0]], ids=["short", "ragged", "one", "long", "empty"])
def test_balanced_kernel_matches_f64_ground_truth(Hq, Hkv, D, lens):
    """The balanced kernel cuts the flattened batch into equal spans per warp: pieces of a pair
    held by several warps, whole pairs inside one warp, empty sequences and warps with nothing
    to do all occur in these cases."""
    out, rec, ref32, ref64, m, l = _run(106, lens, Hq, Hkv, D, torch.bfloat16, 0, q_dtype=torch.bfloat16)
    assert_close(out, ref64, TOL_BF16, "balanced decode vs fp64 ground truth")
    assert_close(rec[:, :D].reshape(out.shape), out, 1e-6, "records carry the output")
    live = np.repeat(np.asarray(lens) > 0, Hq)
    np.testing.assert_allclose((rec[:, D] + np.log(rec[:, D + 1]))[live], (m + np.log(l)).reshape(-1)[live], atol=3e-2)
    assert not out[~(np.asarray(lens) > 0)].any() and not rec[~live, D + 1].any()


def test_balanced_kernel_uniform_cache():
    Hq, Hkv, D, B, L, cap = 8, 2, 128, 5, 1000, 1024
    kv = O.from_bf16(O.to_bf16(normal(107, 0, (2, B, Hkv, cap, D))))
    q = O.from_bf16(O.to_bf16(normal(107, 1, (B, Hq * D))))
    kw = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=L, seq_stride=Hkv * cap * D, head_stride=cap * D)
    out = A.decode_batch(dev(q, torch.bfloat16), dev(kv[0], torch.bfloat16), dev(kv[1], torch.bfloat16), **kw)
    off = np.arange(B, dtype=np.int64) * Hkv * cap * D
    ref = O.decode_batch(q, kv[0].reshape(-1), kv[1].reshape(-1), off, np.full(B, cap * D, np.int64),
                         np.full(B, L, np.int32), Hq, Hkv, D, 1.0 / np.sqrt(D), acc64=True)
    assert_close(host(out), ref, TOL_BF16, "balanced, seq_len = NULL")


def test_mma_kernel_is_tight_when_p_is_exact():
    """With one attended row p = 1 exactly, so the tensor-core kernel must return that V row
    bit-exactly (bf16 -> fp32): checks fragment layouts without rounding noise."""
    Hq, Hkv, D = 8, 2, 128
    lens = [1] * 6
    k, v, off, hs = ragged_cache(103, lens, Hkv, D, torch.bfloat16, normal, 0)
    q = normal(103, 12, (6, Hq * D))
    for chunk_rows in (64, 0):                                   # chunk grid, balanced
        out = A.decode_batch(dev(q), dev(k, torch.bfloat16), dev(v, torch.bfloat16), n_head=Hq, n_kv_head=Hkv,
                             head_dim=D, max_len=1, seq_len=dev(np.asarray(lens, np.int32)), kv_off=dev(off),
                             head_stride=int(hs[0]), chunk_rows=chunk_rows)
        out = host(out).reshape(6, Hq, D)
        for b in range(6):
            for h in range(Hq):
                np.testing.assert_array_equal(out[b, h], v[off[b] + (h // 4) * hs[b]: off[b] + (h // 4) * hs[b] + D])


def test_zero_length_and_missing_seq_len():
    Hq, Hkv, D = 9, 3, 64
    lens = [0, 5, 0, 70]
    for dt in (torch.float32, torch.bfloat16):
        out, rec, ref32, ref64, m, l = _run(104, lens, Hq, Hkv, D, dt, 64)
        assert not out[0].any() and not out[2].any()
        assert_close(out, ref64, TOL_BF16 if dt == torch.bfloat16 else TOL_F32, "zero-length rows")
    # seq_len = NULL: every sequence attends max_len rows of a uniform cache
    B, L = 3, 77
    kv = normal(105, 0, (2, B, Hkv, 80, D))
    q = normal(105, 1, (B, Hq * D))
    out = A.decode_batch(dev(q), dev(kv[0]), dev(kv[1]), n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=L,
                         seq_stride=Hkv * 80 * D, head_stride=80 * D)
    off = np.arange(B, dtype=np.int64) * Hkv * 80 * D
    ref = O.decode_batch(q, kv[0].reshape(-1), kv[1].reshape(-1), off, np.full(B, 80 * D, np.int64),
                         np.full(B, L, np.int32), Hq, Hkv, D, 0.125)
    assert_close(host(out), ref, TOL_F32, "uniform cache")


def test_split_invariance_and_determinism_c3_shape():
    """Full C3-shaped batch (256 ragged sequences, 9q/3kv, D=64, bf16): results do not
    depend on the chunking beyond fp32 merge noise, repeat bit-exactly, and a sample of
    sequences matches the float64 ground truth."""
    B, Hq, Hkv, D = 256, 9, 3, 64
    lens = rng(SEED_C3, 0).integers(512, 4097, B).astype(np.int32)
    gen = torch.Generator(device="cuda").manual_seed(SEED_C3)
    outs = {}
    # every sequence gets a [Hkv, 4096, D] block (uniform strides), ragged seq_len inside
    cap = 4096
    kc = torch.randn(B, Hkv, cap, D, generator=gen, device="cuda").bfloat16()
    vc = torch.randn(B, Hkv, cap, D, generator=gen, device="cuda").bfloat16()
    q = torch.randn(B, Hq * D, generator=gen, device="cuda").bfloat16()
    args = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=4096, seq_len=dev(lens),
                seq_stride=Hkv * cap * D, head_stride=cap * D)
    for chunk in (0, 256, 1024, 4096):
        outs[chunk] = host(A.decode_batch(q, kc, vc, chunk_rows=chunk, **args))
    again = host(A.decode_batch(q, kc, vc, chunk_rows=0, **args))
    np.testing.assert_array_equal(outs[0], again)
    for chunk in (256, 1024, 4096):
        # the bf16 rounding of P depends on the running maximum, hence on the split
        assert_close(outs[chunk], outs[0], TOL_BF16, f"chunk {chunk} vs auto")
    sample = [0, 17, 255, int(np.argmax(lens)), int(np.argmin(lens))]
    kb, vb = bf16_bits(kc[sample]).reshape(-1), bf16_bits(vc[sample]).reshape(-1)
    soff = np.arange(len(sample), dtype=np.int64) * Hkv * cap * D
    ref = O.decode_batch(host(q[sample]), kb, vb, soff, np.full(len(sample), cap * D, np.int64), lens[sample],
                         Hq, Hkv, D, 0.125, acc64=True)
    for chunk in outs:
        assert_close(outs[chunk][sample], ref, TOL_BF16, f"C3 sample vs fp64, chunk {chunk}")


def test_kv_sequence_shards_combine_to_unsharded_c5_shape():
    """C5 shape at reduced length (32q/8kv, D=128, bf16): N contiguous KV shards, each
    decoded to (o, m, l) records, merged by nimllm_attn_combine == the unsharded decode."""
    B, Hq, Hkv, D, L = 2, 32, 8, 128, 8192
    gen = torch.Generator(device="cuda").manual_seed(SEED_C5)
    kc = torch.randn(B, Hkv, L, D, generator=gen, device="cuda").bfloat16()
    vc = torch.randn(B, Hkv, L, D, generator=gen, device="cuda").bfloat16()
    q = torch.randn(B, Hq * D, generator=gen, device="cuda").bfloat16()
    base = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
    full = host(A.decode_batch(q, kc, vc, max_len=L, seq_stride=Hkv * L * D, head_stride=L * D, **base))
    for N in (2, 4, 8):
        rows = L // N
        recs = []
        for r in range(N):
            off = dev(np.arange(B, dtype=np.int64) * Hkv * L * D + r * rows * D)
            _, rec = A.decode_batch(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, partials=True, **base)
            recs.append(rec)
        merged = host(A.combine(torch.stack(recs), D)).reshape(B, Hq * D)
        # P is rounded to bf16 relative to the running maximum, which depends on where the rows
        # are cut: sharded and unsharded agree to a fraction of the bf16 bound, not to fp32 noise
        assert_close(merged, full, 5e-3, f"{N} shards vs unsharded", elem_tol=2e-2)
    kb, vb = bf16_bits(kc).reshape(-1), bf16_bits(vc).reshape(-1)
    ref = O.decode_batch(host(q), kb, vb, np.arange(B, dtype=np.int64) * Hkv * L * D, np.full(B, L * D, np.int64),
                         np.full(B, L, np.int32), Hq, Hkv, D, 1 / np.sqrt(D), acc64=True)
    assert_close(full, ref, TOL_BF16, "C5-shaped decode vs fp64")


def test_combine_matches_oracle():
    D, W, n_parts, rows = 64, 68, 5, 37
    parts = normal(106, 0, (n_parts, rows, W))
    parts[:, :, D + 1] = np.abs(parts[:, :, D + 1]) + 0.1
    parts[2, 3:9, D + 1] = 0.0            # empty shards
    parts[2, 3:9, D] = -np.inf
    out, rec = A.combine(dev(parts), D, partials=True)
    ref, m, l = O.combine(parts, D)
    assert_close(host(out), ref, 1e-5, "combine o")
    rec = host(rec)
    np.testing.assert_allclose(rec[:, D] + np.log(rec[:, D + 1]), m + np.log(l), atol=1e-5)
