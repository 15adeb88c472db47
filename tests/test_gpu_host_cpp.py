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
