"""Generates tests/golden/attn_f64_golden.npz: attention outputs computed by an
independent float64 NumPy formulation (no code shared with oracle/ or the CUDA library)
on inputs regenerated from fixed Philox seeds.  Only sampled output rows are stored; a
SHA-256 of the inputs guards against drift of the generator.

    python tests/golden/make_golden.py

The reference's own tests hold no vector for multi-token attention (its checks stop at the
Q projection or at S = 1), so these fixtures pin the mathematics; the reference's
arithmetic is pinned by running its own compiled kernels beside the library in the GPU
tests (tests/test_gpu_prefill_f32.py, tests/test_gpu_model_c2.py), not by a stored file.
"""
import hashlib
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from util import SEED_C1, normal  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

CASES = {
    # name: (seed, S, Hq, Hkv, D, rope base, sampled rows)
    "c1": (SEED_C1, 160, 9, 3, 64, 10000.0, [0, 1, 7, 31, 32, 63, 64, 100, 127, 128, 129, 140, 159]),
    "llama": (SEED_C1 + 100, 72, 8, 2, 128, 500000.0, [0, 5, 31, 32, 33, 64, 71]),
    "mha": (SEED_C1 + 200, 40, 4, 4, 64, 100000.0, [0, 15, 16, 39]),
}


def inputs(seed, S, Hq, Hkv, D):
    q = normal(seed, 0, (S, Hq * D))
    k = normal(seed, 1, (S, Hkv * D))
    v = normal(seed, 2, (S, Hkv * D))
    return q, k, v


def digest(*arrays):
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def rope64(x, H, D, base):
    """Rotate-half RoPE in float64 with the reference's fp32 angle (theta is computed in
    fp32 by the reference, src/model.nim:160; cos/sin of it are taken in float64 here)."""
    S = x.shape[0]
    half = D // 2
    pos = np.arange(S, dtype=np.float32)[:, None]
    f = np.arange(half, dtype=np.float32)[None, :]
    inv = np.power(np.float32(base), np.float32(2.0) * f / np.float32(D), dtype=np.float32)
    theta = (pos / inv).astype(np.float32).astype(np.float64)
    c, s = np.cos(theta)[:, None, :], np.sin(theta)[:, None, :]
    x = x.astype(np.float64).reshape(S, H, D)
    x0, x1 = x[..., :half], x[..., half:]
    return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], -1).reshape(S, H * D)


def attention64(q, k, v, Hq, Hkv, D, base):
    S = q.shape[0]
    G = Hq // Hkv
    qr, kr = rope64(q, Hq, D, base), rope64(k, Hkv, D, base)
    vv = v.astype(np.float64)
    out = np.zeros((S, Hq * D))
    mask = np.tril(np.ones((S, S), bool))
    for h in range(Hq):
        kvh = h // G
        Q = qr[:, h * D:(h + 1) * D]; K = kr[:, kvh * D:(kvh + 1) * D]; V = vv[:, kvh * D:(kvh + 1) * D]
        s = (Q @ K.T) / np.sqrt(np.float64(D))
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(1, keepdims=True))
        p /= p.sum(1, keepdims=True)
        out[:, h * D:(h + 1) * D] = p @ V
    return out, kr


def main():
    blob = {}
    for name, (seed, S, Hq, Hkv, D, base, rows) in CASES.items():
        q, k, v = inputs(seed, S, Hq, Hkv, D)
        out, kr = attention64(q, k, v, Hq, Hkv, D, base)
        blob[f"{name}_meta"] = np.array([seed, S, Hq, Hkv, D], np.int64)
        blob[f"{name}_base"] = np.array(base, np.float64)
        blob[f"{name}_rows"] = np.array(rows, np.int64)
        blob[f"{name}_out"] = out[rows].astype(np.float32)
        blob[f"{name}_krot"] = kr[rows].astype(np.float32)
        blob[f"{name}_sha"] = np.frombuffer(digest(q, k, v).encode(), np.uint8)
    np.savez_compressed(os.path.join(HERE, "attn_f64_golden.npz"), **blob)
    print("wrote attn_f64_golden.npz", {k: v.shape for k, v in blob.items()})


if __name__ == "__main__":
    main()
