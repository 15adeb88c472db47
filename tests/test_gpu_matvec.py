"""GPU parity of the decode projections (tests marked gpu): the quantised mat-vecs behind the
reference's own launcher names, the fused q/k/v projection + RoPE + cache append, and the output
projection + residual, all through the C ABI, against the CPU restatement of the reference's
arithmetic (fp32 bound 1e-4) and against the reference's own compiled kernels."""
import ctypes as C

import numpy as np
import pytest
import torch

from gpu_util import bf16_bits, dev, host
from nimllm_b200 import _lib, attention as A
from oracle import oracle as O
from util import TOL_F32, assert_close, normal

pytestmark = pytest.mark.gpu

SHAPES = [(576, 576), (192, 576), (1536, 576), (576, 1536), (1024, 4096), (40, 96), (7, 32), (33, 2080)]


def _weights(seed, rows, cols, kind):
    w = normal(seed, 0, (rows, cols), 0.02)
    if kind in ("q4_0", "q8_0"):
        blocks = O.quantize(w, kind)
        return blocks, O.dequantize(blocks, kind, (rows, cols)), torch.from_numpy(blocks).cuda()
    if kind == "bf16":
        wr = O.from_bf16(O.to_bf16(w))
        return None, wr, dev(wr, torch.bfloat16)
    return None, w, dev(w)


W_TYPE = {"f32": _lib.W_F32, "bf16": _lib.W_BF16, "q8_0": _lib.W_Q8_0, "q4_0": _lib.W_Q4_0}


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
def test_legacy_quantised_matvec_matches_oracle_and_reference_kernels(rows, cols, kind):
    blocks, wd, wdev = _weights(300 + rows, rows, cols, kind)
    x = normal(301, 1, (cols,))
    y = torch.zeros(rows, device="cuda")
    fn = getattr(_lib.lib(), "gpu_matvec_" + kind)
    fn(wdev.data_ptr(), dev(x).data_ptr(), y.data_ptr(), rows, cols)
    torch.cuda.synchronize()
    assert_close(host(y), O.matvec_q(blocks, kind, x, rows, cols), TOL_F32, f"{kind} matvec vs the restated kernel (fp32)")
    assert_close(host(y), O.matvec_q(blocks, kind, x, rows, cols, acc64=True), TOL_F32, f"{kind} matvec vs float64")
    # The reference's own compiled kernels are run only where they are well defined: k_matvec_q4_0
    # writes its per-warp sums over the first floats of the shared copy of x while other warps may
    # still read them (no barrier after the loop, src/kernels.cu:981), so its results depend on
    # timing and are left out; k_matvec_q8_0 stores 256 partial sums into `cols` floats of shared
    # memory (src/kernels.cu:1041-1043), which is out of bounds for cols < 256 -- never run here.
    if O.ref_available() and kind == "q8_0" and cols >= 256:
        R = O.ref_lib()
        yr = torch.zeros(rows, device="cuda")
        R.gpu_matvec_q8_0.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        R.gpu_matvec_q8_0.restype = None
        R.gpu_matvec_q8_0(wdev.data_ptr(), dev(x).data_ptr(), yr.data_ptr(), rows, cols)
        torch.cuda.synchronize()
        assert_close(host(y), host(yr), TOL_F32, "q8_0 matvec vs the reference's compiled kernel")


def test_q4_quantiser_of_the_oracle_is_the_reference_quantiser():
    """Pins the test inputs: the CPU quantiser used to make Q4_0 matrices gives the bytes the
    reference's own gpu_quantize_q4_0 gives (src/kernels.cu:904-932, 990-994)."""
    if not O.ref_available():
        pytest.skip("the reference's kernels were not compiled into oracle/_ref")
    R = O.ref_lib()
    w = normal(302, 0, (64, 576), 0.02)
    out = torch.zeros(w.size // 32 * 18, dtype=torch.uint8, device="cuda")
    R.gpu_quantize_q4_0.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
    R.gpu_quantize_q4_0.restype = None
    R.gpu_quantize_q4_0(dev(w).data_ptr(), out.data_ptr(), w.size)
    torch.cuda.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy(), O.quantize(w, "q4_0"))


@pytest.mark.parametrize("kind", ["f32", "bf16", "q8_0", "q4_0"])
@pytest.mark.parametrize("B", [1, 2, 3, 8, 11])
def test_matvec_batched_with_residual(kind, B):
    rows, cols = 576, 1536
    blocks, wd, wdev = _weights(310, rows, cols, kind)
    x = normal(311, 1, (B, cols)); r = normal(311, 2, (B, rows))
    y = A.matvec(wdev, dev(x), rows, w_type=W_TYPE[kind], residual=dev(r))
    torch.cuda.synchronize()
    ref = (x.astype(np.float64) @ wd.astype(np.float64).T + r).astype(np.float32)
    assert_close(host(y), ref, TOL_F32, f"{kind} matvec + residual, batch {B}")


@pytest.mark.parametrize("rows,cols", SHAPES)
@pytest.mark.parametrize("kind", ["q4_0", "q8_0"])
def test_staged_kernels_on_ragged_shapes(rows, cols, kind):
    """Batches of eight and more go through the kernels that stage weights in shared memory: row
    segments that start off a 16-byte boundary, matrices whose last bytes lie past the last 16-byte
    boundary (7 x 32 Q4_0 = 126 bytes), odd block counts per row, an odd number of rows, a second
    partial batch tile."""
    blocks, wd, wdev = _weights(320 + rows, rows, cols, kind)
    B = 11
    x = normal(321, 1, (B, cols))
    y = A.matvec(wdev, dev(x), rows, w_type=W_TYPE[kind])
    torch.cuda.synchronize()
    ref = (x.astype(np.float64) @ wd.astype(np.float64).T).astype(np.float32)
    assert_close(host(y), ref, TOL_F32, f"{kind} staged matvec {rows}x{cols}")
    assert A.matvec_status() == 0


@pytest.mark.parametrize("kind", ["f32", "bf16", "q8_0", "q4_0"])
@pytest.mark.parametrize("Hq,Hkv,D,n_embd", [(9, 3, 64, 576), (32, 8, 128, 4096), (4, 4, 64, 256)])
@pytest.mark.parametrize("B,cache_dtype", [(1, torch.float32), (5, torch.bfloat16), (8, torch.float32), (10, torch.bfloat16)])
def test_qkv_rope_append_matches_unfused_reference_arithmetic(kind, Hq, Hkv, D, n_embd, B, cache_dtype):
    """q = wq x, k = wk x, v = wv x in float64 on the (de)quantised weights, then the reference's
    RoPE (restated, fp32) and append: rotated q out, rotated K / raw V in the right cache rows."""
    base, cap = 10000.0, 96
    _, wq, wq_d = _weights(320, Hq * D, n_embd, kind)
    _, wk, wk_d = _weights(321, Hkv * D, n_embd, kind)
    _, wv, wv_d = _weights(322, Hkv * D, n_embd, kind)
    x = normal(323, 0, (B, n_embd))
    pos = (np.arange(B) * 7 % cap).astype(np.int32)
    cos, sin = A.rope_tables(cap, D, base)
    kc = torch.zeros(B, Hkv, cap, D, dtype=cache_dtype, device="cuda"); vc = torch.zeros_like(kc)
    q, k, v = A.qkv_rope_append(dev(x), wq_d, wk_d, wv_d, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, w_type=W_TYPE[kind],
                                seq_pos=dev(pos), k_cache=kc, v_cache=vc, seq_stride=Hkv * cap * D, head_stride=cap * D,
                                max_seq=cap, want_kv=True)
    torch.cuda.synchronize()
    x64 = x.astype(np.float64)
    qr = (x64 @ wq.astype(np.float64).T).astype(np.float32)
    kr = (x64 @ wk.astype(np.float64).T).astype(np.float32)
    vr = (x64 @ wv.astype(np.float64).T).astype(np.float32)
    oc, osn = O.rope_tables(cap, D, base)
    for b in range(B):
        O.rope_fwd(qr[b:b + 1], oc[pos[b]:], osn[pos[b]:], Hq, D)
        O.rope_fwd(kr[b:b + 1], oc[pos[b]:], osn[pos[b]:], Hkv, D)
    assert_close(host(q), qr, TOL_F32, "q"); assert_close(host(k), kr, TOL_F32, "k"); assert_close(host(v), vr, TOL_F32, "v")
    kcache, vcache = host(kc), host(vc)
    tol = TOL_F32 if cache_dtype == torch.float32 else 8e-3          # bf16 rounding of the cached row
    for b in range(B):
        assert_close(kcache[b, :, pos[b]], kr[b].reshape(Hkv, D), tol, "cached K row")
        assert_close(vcache[b, :, pos[b]], vr[b].reshape(Hkv, D), tol, "cached V row")
        mask = np.ones(cap, bool); mask[pos[b]] = False
        assert not kcache[b][:, mask].any() and not vcache[b][:, mask].any()      # nothing else was touched


def test_fused_step_equals_the_unfused_library_calls():
    """qkv_rope_append -> decode -> wo_residual against matvec x3 -> rope_append -> decode -> matvec + add."""
    Hq, Hkv, D, n_embd, B, cap = 9, 3, 64, 576, 4, 64
    ws = [dev(normal(330 + i, 0, s, 0.05)) for i, s in enumerate([(Hq * D, n_embd), (Hkv * D, n_embd), (Hkv * D, n_embd), (n_embd, Hq * D)])]
    x_in, x_norm = dev(normal(334, 0, (B, n_embd))), dev(normal(334, 1, (B, n_embd)))
    pos = torch.tensor([5, 0, 33, 62], dtype=torch.int32, device="cuda")
    cos, sin = A.rope_tables(cap, D, 10000.0)
    hist = normal(335, 0, (2, B, Hkv, cap, D))
    geom = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
    outs = []
    for fused in (True, False):
        kc, vc = dev(hist[0]).clone(), dev(hist[1]).clone()
        cache = dict(k_cache=kc, v_cache=vc, seq_stride=Hkv * cap * D, head_stride=cap * D, max_seq=cap)
        if fused:
            q = A.qkv_rope_append(x_norm, ws[0], ws[1], ws[2], cos, sin, seq_pos=pos, **geom, **cache)
        else:
            q, k, v = (A.matvec(w, x_norm, w.shape[0]) for w in ws[:3])
            A.rope_append(q.view(B, 1, -1), k.view(B, 1, -1), v.view(B, 1, -1), cos, sin, seq_pos=pos, **geom, **cache)
        attn = A.decode_batch(q, kc, vc, max_len=cap, seq_len=pos + 1, seq_stride=Hkv * cap * D, head_stride=cap * D, **geom)
        outs.append(host(A.wo_residual(attn, ws[3], x_in) if fused else A.matvec(ws[3], attn, n_embd) + x_in))
    assert_close(outs[0], outs[1], 1e-5, "fused vs unfused decode step")


def test_matvec_argument_checks():
    z = torch.zeros(64, device="cuda")
    with pytest.raises(RuntimeError, match="cols"):
        A.matvec(torch.zeros(40, dtype=torch.uint8, device="cuda"), z.view(1, 64)[:, :40].contiguous(), 1, w_type=_lib.W_Q4_0)
    with pytest.raises(RuntimeError, match="aligned"):
        A.matvec(torch.zeros(4 * 64 + 1, device="cuda")[1:], z.view(1, 64), 4)
