"""The C++ host mirror (nimllm_b200/host): KvCache / initKvCache / resetKvCache and the two
attention blocks named after src/model.nim, driven through its ctypes shim on configuration C1."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from gpu_util import dev, host, wrap_ptr
from nimllm_b200 import build
from oracle import oracle as O
from util import SEED_C1, TOL_F32, assert_close, normal

pytestmark = pytest.mark.gpu


def _host_lib():
    H = C.CDLL(build.build_host())
    H.nimllm_host_session_create.restype = C.c_void_p
    H.nimllm_host_session_create.argtypes = [C.c_int] * 5 + [C.c_float, C.c_size_t]
    for name, args, res in [("nimllm_host_session_destroy", [C.c_void_p], None),
                            ("nimllm_host_kv_pos", [C.c_void_p], C.c_int),
                            ("nimllm_host_kv_set_pos", [C.c_void_p, C.c_int], None),
                            ("nimllm_host_kv_reset", [C.c_void_p], None),
                            ("nimllm_host_kv_k", [C.c_void_p, C.c_int], C.c_void_p),
                            ("nimllm_host_kv_v", [C.c_void_p, C.c_int], C.c_void_p),
                            ("nimllm_host_attn_forward", [C.c_void_p] * 5 + [C.c_int] * 3, C.c_int),
                            ("nimllm_host_attn_forward_cached", [C.c_void_p, C.c_int] + [C.c_void_p] * 4, C.c_int),
                            ("nimllm_host_attn_step_cached", [C.c_void_p, C.c_int] + [C.c_void_p] * 4 + [C.c_int] + [C.c_void_p] * 3, C.c_int),
                            ("nimllm_host_free_step", [C.c_void_p], None)]:
        fn = getattr(H, name); fn.argtypes = args; fn.restype = res
    return H


def test_c1_through_the_cpp_host_layer():
    H = _host_lib()
    S, n_pre, Hq, Hkv, D, base, n_layer = 160, 128, 9, 3, 64, 10000.0, 2
    q = normal(SEED_C1, 0, (S, Hq * D)); k = normal(SEED_C1, 1, (S, Hkv * D)); v = normal(SEED_C1, 2, (S, Hkv * D))
    sess = H.nimllm_host_session_create(n_layer, Hq, Hkv, D, S, base, 8 << 20)
    assert sess
    try:
        dq, dk, dv = dev(q), dev(k), dev(v)
        out = torch.zeros(S, Hq * D, device="cuda")
        layer = 1
        assert H.nimllm_host_attn_forward(sess, dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), out.data_ptr(), n_pre, 1,
                                          layer) == 0
        assert H.nimllm_host_kv_pos(sess) == n_pre
        for t in range(n_pre, S):
            rc = H.nimllm_host_attn_forward_cached(sess, layer, dq[t].data_ptr(), dk[t].data_ptr(), dv[t].data_ptr(),
                                                   out[t].data_ptr())
            assert rc == 0
            H.nimllm_host_kv_set_pos(sess, t + 1)          # the caller's kv.pos += newTokens (src/model.nim:890)
            H.nimllm_host_free_step(sess)                  # chat.nim:98,123 freeStepAllocations()
        torch.cuda.synchronize()

        cos, sin = O.rope_tables(S, D, base)
        ref = np.zeros((S, Hq * D), np.float32)
        o, q_rot, k_rot = O.attn_forward(q[:n_pre], k[:n_pre], v[:n_pre], cos, sin, Hq, Hkv, D)
        ref[:n_pre] = o
        okv = O.KvCache(Hkv, D, S); okv.fill(k_rot, v[:n_pre])
        for t in range(n_pre, S):
            ref[t] = O.attn_forward_cached(okv, q[t], k[t], v[t], cos, sin, Hq)
        assert_close(host(out), ref, TOL_F32, "C1 through the C++ host layer")
        assert_close(host(dq)[:n_pre], q_rot, 1e-6, "q rotated in place (saveCache)")
        kc = host(wrap_ptr(H.nimllm_host_kv_k(sess, layer), (Hkv, S, D)))
        assert_close(kc, okv.k, 1e-6, "cache K of the written layer")
        assert not host(wrap_ptr(H.nimllm_host_kv_k(sess, 0), (Hkv, S, D))).any()      # other layer untouched
        H.nimllm_host_kv_reset(sess)
        torch.cuda.synchronize()
        assert H.nimllm_host_kv_pos(sess) == 0
        assert not host(wrap_ptr(H.nimllm_host_kv_k(sess, layer), (Hkv, S, D))).any()
    finally:
        H.nimllm_host_session_destroy(sess)


@pytest.mark.parametrize("kind", ["f32", "q8_0"])
def test_decode_steps_with_projections_through_the_cpp_host_layer(kind):
    """forwardCached()'s attention part with its projections (src/model.nim:775-849) through the C++ mirror:
    24 tokens decoded one by one from an empty cache; every step's xOut = xResid + wo * attention against
    the oracle run on the same (dequantised) weights."""
    from nimllm_b200 import _lib
    H = _host_lib()
    steps, Hq, Hkv, D, base = 24, 9, 3, 64, 10000.0
    E, Ekv = Hq * D, Hkv * D
    mats = {}
    wdev = {}
    for i, (name, rows) in enumerate((("wq", E), ("wk", Ekv), ("wv", Ekv), ("wo", E))):
        w = normal(700 + i, 0, (rows, E), 0.05)
        if kind == "q8_0":
            blocks = O.quantize(w, "q8_0")
            mats[name] = O.dequantize(blocks, "q8_0", (rows, E))
            wdev[name] = torch.from_numpy(blocks).cuda()
        else:
            mats[name] = w
            wdev[name] = dev(w)
    wtype = _lib.W_Q8_0 if kind == "q8_0" else _lib.W_F32
    xn = normal(710, 0, (steps, E)); xr = normal(710, 1, (steps, E))
    sess = H.nimllm_host_session_create(1, Hq, Hkv, D, 64, base, 8 << 20)
    assert sess
    try:
        dxn, dxr = dev(xn), dev(xr)
        out = torch.zeros(steps, E, device="cuda")
        for t in range(steps):
            rc = H.nimllm_host_attn_step_cached(sess, 0, wdev["wq"].data_ptr(), wdev["wk"].data_ptr(), wdev["wv"].data_ptr(),
                                                wdev["wo"].data_ptr(), wtype, dxn[t].data_ptr(), dxr[t].data_ptr(), out[t].data_ptr())
            assert rc == 0
            H.nimllm_host_kv_set_pos(sess, t + 1)
            H.nimllm_host_free_step(sess)
        torch.cuda.synchronize()
        cos, sin = O.rope_tables(64, D, base)
        okv = O.KvCache(Hkv, D, 64)
        ref = np.zeros((steps, E), np.float32)
        f64 = lambda a: a.astype(np.float64)
        for t in range(steps):
            q = (f64(mats["wq"]) @ f64(xn[t])).astype(np.float32)
            k = (f64(mats["wk"]) @ f64(xn[t])).astype(np.float32)
            v = (f64(mats["wv"]) @ f64(xn[t])).astype(np.float32)
            attn = O.attn_forward_cached(okv, q, k, v, cos, sin, Hq)
            ref[t] = (f64(mats["wo"]) @ f64(attn) + f64(xr[t])).astype(np.float32)
        assert_close(host(out), ref, TOL_F32, f"decode steps with {kind} projections through the C++ host layer")
    finally:
        H.nimllm_host_session_destroy(sess)
