"""GPU parity of the attention backward (fp32) through the C ABI: against the CPU restatement of
the reference's backward loop (fp32 and float64 accumulation) and against that loop run through the
reference's own compiled kernels + cuBLAS."""
import numpy as np
import pytest
import torch

from gpu_util import host
from nimllm_b200 import attention as A
from oracle import oracle as O
from util import TOL_F32, assert_close, normal

pytestmark = pytest.mark.gpu


def _forward(q, k, v, cos, sin, Hq, Hkv, D):
    """Library forward with save_cache: rotated q, k stay in the buffers; out and lse come back."""
    B, S = q.shape[0], q.shape[1]
    lse = torch.zeros(B, Hq, S, device="cuda")
    out = A.attn_forward(q, k, v, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, save_cache=True, lse=lse)
    return out, lse


@pytest.mark.parametrize("B,S,Hq,Hkv,D", [(1, 128, 9, 3, 64), (2, 77, 4, 2, 32), (1, 300, 8, 2, 128), (1, 1, 3, 3, 64),
                                           (3, 33, 6, 1, 64),
                                           # launches large enough for the 64 x 64 register-tiled kernels: grouped heads
                                           # (per-head partial sums) and one query head per KV head, ragged last tiles
                                           (2, 300, 9, 3, 64), (2, 200, 10, 10, 64), (1, 449, 12, 4, 64)])
@pytest.mark.parametrize("rope", [True, False])
def test_backward_matches_oracle(B, S, Hq, Hkv, D, rope):
    q0 = normal(700 + S, 0, (B, S, Hq * D)); k0 = normal(700 + S, 1, (B, S, Hkv * D))
    v0 = normal(700 + S, 2, (B, S, Hkv * D)); dout = normal(700 + S, 3, (B, S, Hq * D))
    q, k, v = (torch.from_numpy(x).cuda() for x in (q0, k0, v0))
    cos, sin = A.rope_tables(S, D, 10000.0) if rope else (None, None)
    out, lse = _forward(q, k, v, cos, sin, Hq, Hkv, D)
    dq, dk, dv = A.attn_backward(q, k, v, out, torch.from_numpy(dout).cuda(), lse, cos, sin,
                                 n_head=Hq, n_kv_head=Hkv, head_dim=D)
    again = A.attn_backward(q, k, v, out, torch.from_numpy(dout).cuda(), lse, cos, sin,
                            n_head=Hq, n_kv_head=Hkv, head_dim=D)
    torch.cuda.synchronize()
    for a, b in zip((dq, dk, dv), again):
        np.testing.assert_array_equal(host(a), host(b))            # fixed summation order
    ct, st = O.rope_tables(S, D, 10000.0)
    for b in range(B):
        qr, kr = q0[b].copy(), k0[b].copy()
        if rope:
            O.rope_fwd(qr, ct, st, Hq, D); O.rope_fwd(kr, ct, st, Hkv, D)
        for acc64 in (False, True):
            rq, rk, rv = O.attn_backward(qr, kr, v0[b], dout[b], ct, st, Hq, Hkv, D, apply_rope=rope, acc64=acc64)
            if S == 1:
                # one key: dS is exactly 0 in the reference's formulation; here delta = dO.o is taken
                # from the rounded forward output, which leaves rounding noise instead of zeros
                np.testing.assert_allclose(host(dq[b]), rq, atol=1e-5)
            else:
                assert_close(host(dq[b]), rq, TOL_F32, f"dq acc64={acc64}")
            if S == 1:
                np.testing.assert_allclose(host(dk[b]), rk, atol=1e-5)
            else:
                assert_close(host(dk[b]), rk, TOL_F32, f"dk acc64={acc64}")
            assert_close(host(dv[b]), rv, TOL_F32, f"dv acc64={acc64}")


def test_backward_against_reference_compiled_kernels():
    """C1's shape (9 q / 3 kv heads of 64, 128 tokens): the same gradients from the reference's
    kernels + cuBLAS in the reference's launch order, from the oracle and from this library."""
    if not O.ref_available():
        pytest.skip("the reference's kernels were not compiled into oracle/_ref")
    S, Hq, Hkv, D = 128, 9, 3, 64
    q0 = normal(801, 0, (S, Hq * D)); k0 = normal(801, 1, (S, Hkv * D)); v0 = normal(801, 2, (S, Hkv * D))
    dout = normal(801, 3, (S, Hq * D))
    ct, st = O.rope_tables(S, D, 10000.0)
    qr, kr = q0.copy(), k0.copy()
    O.rope_fwd(qr, ct, st, Hq, D); O.rope_fwd(kr, ct, st, Hkv, D)
    ref = O.ref_attn_backward(qr, kr, v0, dout, ct, st, Hq, Hkv, D)
    ora = O.attn_backward(qr, kr, v0, dout, ct, st, Hq, Hkv, D)
    q, k, v = (torch.from_numpy(x).cuda().unsqueeze(0) for x in (q0, k0, v0))
    cos, sin = A.rope_tables(S, D, 10000.0)
    out, lse = _forward(q, k, v, cos, sin, Hq, Hkv, D)
    got = A.attn_backward(q, k, v, out, torch.from_numpy(dout).cuda().unsqueeze(0), lse, cos, sin,
                          n_head=Hq, n_kv_head=Hkv, head_dim=D)
    torch.cuda.synchronize()
    for name, r, o, g in zip(("dq", "dk", "dv"), ref, ora, got):
        assert_close(o, r, TOL_F32, f"oracle vs reference kernels, {name}")
        assert_close(host(g[0]), r, TOL_F32, f"library vs reference kernels, {name}")


def test_backward_argument_checks():
    S, Hq, Hkv, D = 16, 2, 1, 64
    z = torch.zeros(1, S, Hq * D, device="cuda"); zk = torch.zeros(1, S, Hkv * D, device="cuda")
    lse = torch.zeros(1, Hq, S, device="cuda")
    with pytest.raises(RuntimeError, match="lse"):
        A.attn_backward(z, zk, zk, z, z, None, None, None, n_head=Hq, n_kv_head=Hkv, head_dim=D)
    z48 = torch.zeros(1, S, Hq * 48, device="cuda"); zk48 = torch.zeros(1, S, Hkv * 48, device="cuda")
    with pytest.raises(RuntimeError, match="head_dim"):
        A.attn_backward(z48, zk48, zk48, z48, z48, lse, None, None, n_head=Hq, n_kv_head=Hkv, head_dim=48)
