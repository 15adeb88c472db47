"""ctypes/numpy front end of the CPU oracle (oracle/attn_oracle.c) and of the
compiled-reference harness (oracle/_ref/libnimllm_ref.so).

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
_REF = None

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
i64p = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
u16p = np.ctypeslib.ndpointer(dtype=np.uint16, flags="C_CONTIGUOUS")


def build(force: bool = False) -> None:
    """Compile liboracle.so (and oracle/_ref when the reference tree is present)."""
    so = os.path.join(_HERE, "liboracle.so")
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, os.path.join(_HERE, "liboracle.so")])
    ref = os.path.join(_HERE, "_ref", "libnimllm_ref_pts.so")      # the later of the two outputs of `make ref`
    root = os.environ.get("REFERENCE_ROOT", "/root/reference")     # the same variable oracle/Makefile reads
    if os.path.exists(os.path.join(root, "src", "kernels.cu")) and (force or not os.path.exists(ref)):
        subprocess.check_call(["make", "-s", "-C", _HERE, "ref", f"REFERENCE_ROOT={root}"])


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        build()
        L = C.CDLL(os.path.join(_HERE, "liboracle.so"))
        L.oracle_rope_tables.argtypes = [f32p, f32p, C.c_int, C.c_int, C.c_float]
        L.oracle_rope_fwd.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.oracle_softmax_fwd.argtypes = [f32p, f32p, C.c_int, C.c_int]
        L.oracle_causal_mask.argtypes = [f32p, C.c_float, C.c_int]
        L.oracle_scale.argtypes = [f32p, C.c_float, f32p, C.c_int]
        L.oracle_extract_head.argtypes = [f32p, f32p] + [C.c_int] * 4
        L.oracle_extract_kv_head.argtypes = [f32p, f32p] + [C.c_int] * 5
        L.oracle_insert_head.argtypes = [f32p, f32p] + [C.c_int] * 4
        L.oracle_attn_forward.argtypes = [f32p, f32p, f32p, f32p, f32p, f32p] + [C.c_int] * 5
        L.oracle_kv_append.argtypes = [f32p, f32p, f32p, f32p] + [C.c_int] * 5
        L.oracle_attn_backward.argtypes = [f32p] * 9 + [C.c_int] * 6
        L.oracle_rope_bwd.argtypes = [f32p, f32p, f32p, C.c_int, C.c_int, C.c_int, C.c_int]
        L.oracle_attn_forward_cached.argtypes = [f32p] * 7 + [C.c_int, f32p] + [C.c_int] * 4
        L.oracle_decode_batch.argtypes = [f32p, C.c_void_p, C.c_void_p, i64p, i64p, i32p, f32p,
                                          C.c_int, C.c_int, C.c_int, C.c_int, C.c_float,
                                          C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        L.oracle_prefill_f64.argtypes = [f32p, f32p, f32p, f32p] + [C.c_int] * 5 + [C.c_float, C.c_int, C.c_int]
        L.oracle_combine.argtypes = [f32p, C.c_int, C.c_int, C.c_int, C.c_int, f32p, C.c_void_p, C.c_void_p]
        L.oracle_f32_to_bf16.argtypes = [f32p, u16p, C.c_int64]
        L.oracle_bf16_to_f32.argtypes = [u16p, f32p, C.c_int64]
        u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")
        L.oracle_quantize_q4_0.argtypes = [f32p, u8p, C.c_int64]
        L.oracle_quantize_q8_0.argtypes = [f32p, u8p, C.c_int64]
        L.oracle_dequantize.argtypes = [u8p, C.c_int, f32p, C.c_int64]
        L.oracle_matvec_q.argtypes = [u8p, C.c_int, f32p, f32p, C.c_int, C.c_int, C.c_int]
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_threads.argtypes = [C.c_int]
        _LIB = L
    return _LIB


# ----------------------------------------------------------------- numpy API

def quantize(w, kind):
    """w [rows, cols] float32 -> packed Q4_0 (18 bytes per 32 weights, the reference's quantiser,
    src/kernels.cu:904-932) or Q8_0 (34 bytes per 32) blocks as a flat uint8 array."""
    w = np.ascontiguousarray(w, np.float32)
    q4 = kind == "q4_0"
    out = np.empty(w.size // 32 * (18 if q4 else 34), np.uint8)
    (lib().oracle_quantize_q4_0 if q4 else lib().oracle_quantize_q8_0)(w.reshape(-1), out, w.size)
    return out


def dequantize(blocks, kind, shape):
    out = np.empty(int(np.prod(shape)), np.float32)
    lib().oracle_dequantize(np.ascontiguousarray(blocks), int(kind == "q4_0"), out, out.size)
    return out.reshape(shape)


def matvec_q(blocks, kind, x, rows, cols, acc64=False):
    """The reference's k_matvec_q4_0 / k_matvec_q8_0 arithmetic (src/kernels.cu:941-1051) on the CPU."""
    y = np.empty(rows, np.float32)
    lib().oracle_matvec_q(np.ascontiguousarray(blocks), int(kind == "q4_0"), np.ascontiguousarray(x, np.float32), y, rows, cols,
                          int(acc64))
    return y


def rope_tables(max_pos: int, head_dim: int, base: float):
    cos = np.empty((max_pos, head_dim // 2), np.float32)
    sin = np.empty_like(cos)
    lib().oracle_rope_tables(cos, sin, max_pos, head_dim, base)
    return cos, sin


def rope_fwd(data, cos, sin, n_head, head_dim):
    """In place on data [S, n_head*head_dim]; cos/sin rows 0..S-1 are used."""
    S, n_embd = data.shape
    lib().oracle_rope_fwd(data, np.ascontiguousarray(cos), np.ascontiguousarray(sin), S, n_embd, n_head, head_dim)
    return data


def softmax_fwd(x):
    y = np.empty_like(x)
    lib().oracle_softmax_fwd(x, y, x.shape[0], x.shape[1])
    return y


def attn_forward(q, k, v, cos, sin, Hq, Hkv, D, apply_rope=True):
    """Reference forward() attention block. Returns (out, q_rot, k_rot)."""
    q = np.array(q, np.float32, order="C"); k = np.array(k, np.float32, order="C")
    v = np.ascontiguousarray(v, np.float32)
    S = q.shape[0]
    out = np.zeros((S, Hq * D), np.float32)
    lib().oracle_attn_forward(q, k, v, np.ascontiguousarray(cos), np.ascontiguousarray(sin), out, S, Hq, Hkv, D, int(apply_rope))
    return out, q, k


def attn_backward(q_rot, k_rot, v, dout, cos, sin, Hq, Hkv, D, apply_rope=True, acc64=False):
    """Reference backward() attention block (src/model.nim:639-685) for one sequence: returns
    (dq, dk, dv) given the post-RoPE q, k the forward saved, raw v and the gradient of attnOut."""
    q_rot = np.ascontiguousarray(q_rot, np.float32); k_rot = np.ascontiguousarray(k_rot, np.float32)
    v = np.ascontiguousarray(v, np.float32); dout = np.ascontiguousarray(dout, np.float32)
    S = q_rot.shape[0]
    dq = np.zeros((S, Hq * D), np.float32); dk = np.zeros((S, Hkv * D), np.float32); dv = np.zeros((S, Hkv * D), np.float32)
    lib().oracle_attn_backward(q_rot, k_rot, v, dout, np.ascontiguousarray(cos), np.ascontiguousarray(sin), dq, dk, dv,
                               S, Hq, Hkv, D, int(apply_rope), int(acc64))
    return dq, dk, dv


class KvCache:
    """One layer of the reference's KvCache (src/model.nim:70-73,729-746) on the host."""

    def __init__(self, Hkv, D, max_seq):
        self.k = np.zeros((Hkv, max_seq, D), np.float32)
        self.v = np.zeros((Hkv, max_seq, D), np.float32)
        self.pos = 0
        self.Hkv, self.D, self.max_seq = Hkv, D, max_seq

    def reset(self):
        self.k[:] = 0; self.v[:] = 0; self.pos = 0

    def fill(self, k_rot, v):
        n = k_rot.shape[0]
        lib().oracle_kv_append(np.ascontiguousarray(k_rot, np.float32), np.ascontiguousarray(v, np.float32),
                               self.k, self.v, 0, n, self.Hkv, self.D, self.max_seq)
        self.pos = n


def attn_forward_cached(kv: KvCache, q, k_new, v_new, cos, sin, Hq):
    """Reference forwardCached() attention block, newTokens == 1. Returns out [Hq*D]."""
    q = np.array(q, np.float32, order="C").reshape(-1)
    k_new = np.array(k_new, np.float32, order="C").reshape(-1)
    v_new = np.ascontiguousarray(v_new, np.float32).reshape(-1)
    out = np.zeros(Hq * kv.D, np.float32)
    lib().oracle_attn_forward_cached(q, k_new, v_new, np.ascontiguousarray(cos), np.ascontiguousarray(sin),
                                     kv.k, kv.v, kv.pos, out, Hq, kv.Hkv, kv.D, kv.max_seq)
    kv.pos += 1
    return out


def decode_batch(q, k, v, kv_off, head_stride, seq_len, Hq, Hkv, D, scale, acc64=False, want_ml=False):
    """Batched ragged decode (read side). k, v: flat float32 or uint16 (bf16 bits) arrays."""
    q = np.ascontiguousarray(q, np.float32)
    B = q.shape[0]
    bf16 = k.dtype == np.uint16
    assert k.dtype == v.dtype and k.dtype in (np.uint16, np.float32)
    out = np.zeros((B, Hq * D), np.float32)
    m = np.zeros((B, Hq), np.float32) if want_ml else None
    l = np.zeros((B, Hq), np.float32) if want_ml else None
    lib().oracle_decode_batch(q, k.ctypes.data, v.ctypes.data, np.ascontiguousarray(kv_off, np.int64),
                              np.ascontiguousarray(head_stride, np.int64), np.ascontiguousarray(seq_len, np.int32),
                              out, B, Hq, Hkv, D, scale, int(bf16), int(acc64),
                              m.ctypes.data if want_ml else None, l.ctypes.data if want_ml else None)
    return (out, m, l) if want_ml else out


def prefill_f64(q, k, v, Hq, Hkv, D, scale, row0=0, row1=None):
    """Causal attention with float64 accumulation on rotated inputs [B,S,*]; rows [row0,row1)."""
    q = np.ascontiguousarray(q, np.float32); k = np.ascontiguousarray(k, np.float32); v = np.ascontiguousarray(v, np.float32)
    B, S, _ = q.shape
    row1 = S if row1 is None else row1
    out = np.zeros((B, row1 - row0, Hq * D), np.float32)
    lib().oracle_prefill_f64(q, k, v, out, B, S, Hq, Hkv, D, scale, row0, row1)
    return out


def combine(parts, D):
    """parts [n_parts, rows, W] (o[D], m, l, pad) -> (out [rows, D], m, l)."""
    parts = np.ascontiguousarray(parts, np.float32)
    n, rows, W = parts.shape
    out = np.zeros((rows, D), np.float32)
    m = np.zeros(rows, np.float32); l = np.zeros(rows, np.float32)
    lib().oracle_combine(parts, n, rows, D, W, out, m.ctypes.data, l.ctypes.data)
    return out, m, l


def to_bf16(x):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().oracle_f32_to_bf16(x.reshape(-1), y.reshape(-1), x.size)
    return y


def from_bf16(x):
    x = np.ascontiguousarray(x, np.uint16)
    y = np.empty(x.shape, np.float32)
    lib().oracle_bf16_to_f32(x.reshape(-1), y.reshape(-1), x.size)
    return y


def num_threads() -> int:
    return lib().oracle_num_threads()


# ------------------------------------------------- compiled reference (GPU)

def ref_available() -> bool:
    return os.path.exists(os.path.join(_HERE, "_ref", "libnimllm_ref.so"))


_REF_PTS = None


def ref_pts_lib():
    """The same sources built with nvcc --default-stream per-thread (oracle/Makefile): the
    reference's launches go to a stream that can be captured into a CUDA graph.  None when absent."""
    global _REF_PTS
    path = os.path.join(_HERE, "_ref", "libnimllm_ref_pts.so")
    if _REF_PTS is None and os.path.exists(path):
        _REF_PTS = _bind_ref(C.CDLL(path))
    return _REF_PTS


def ref_lib() -> C.CDLL:
    """The reference's compiled kernels + the restated Nim host loop. Needs a GPU to call."""
    global _REF
    if _REF is None:
        _REF = _bind_ref(C.CDLL(os.path.join(_HERE, "_ref", "libnimllm_ref.so")))
    return _REF


def _bind_ref(R):
    if True:
        R.ref_attn_forward.argtypes = [f32p] * 6 + [C.c_int] * 5
        R.ref_attn_backward.argtypes = [f32p] * 9 + [C.c_int] * 4
        R.ref_kvcache_create.restype = C.c_void_p
        R.ref_kvcache_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, f32p, f32p]
        R.ref_kvcache_reset.argtypes = [C.c_void_p]
        R.ref_kvcache_destroy.argtypes = [C.c_void_p]
        R.ref_kvcache_pos.argtypes = [C.c_void_p]
        R.ref_kvcache_fill.argtypes = [C.c_void_p, f32p, f32p, C.c_int]
        R.ref_attn_forward_cached.argtypes = [C.c_void_p, f32p, f32p, f32p, f32p, C.c_int]
        R.ref_kvcache_download.argtypes = [C.c_void_p, f32p, f32p]
        R.ref_attn_forward_dev.argtypes = [C.c_void_p] * 7 + [C.c_int] * 5
        R.ref_decode_batch_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, i64p, i64p, i32p,
                                           C.c_void_p, C.c_void_p] + [C.c_int] * 5
        R.ref_model_create.restype = C.c_void_p
        R.ref_model_create.argtypes = [C.c_int] * 9 + [np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS")]
        R.ref_model_set_attn.argtypes = [C.c_void_p] * 5
        R.ref_model_reset.argtypes = [C.c_void_p]
        R.ref_model_destroy.argtypes = [C.c_void_p]
        R.ref_model_step.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, f32p]
        R.ref_model_prefill_lib.argtypes = [C.c_void_p, i32p, C.c_int, C.c_void_p, f32p]
        R.ref_model_set_proj.argtypes = [C.c_void_p] * 3
        R.ref_model_step_graph.argtypes = [C.c_void_p, C.c_int, f32p, C.c_void_p]
        R.ref_model_graph_available.restype = C.c_int
    return R


def ref_attn_backward(q_rot, k_rot, v, dout, cos, sin, Hq, Hkv, D):
    """backward()'s attention block run through the reference's compiled kernels + cuBLAS."""
    q_rot = np.ascontiguousarray(q_rot, np.float32); k_rot = np.ascontiguousarray(k_rot, np.float32)
    v = np.ascontiguousarray(v, np.float32); dout = np.ascontiguousarray(dout, np.float32)
    S = q_rot.shape[0]
    dq = np.zeros((S, Hq * D), np.float32); dk = np.zeros((S, Hkv * D), np.float32); dv = np.zeros((S, Hkv * D), np.float32)
    rc = ref_lib().ref_attn_backward(q_rot, k_rot, v, dout, np.ascontiguousarray(cos[:S]), np.ascontiguousarray(sin[:S]),
                                     dq, dk, dv, S, Hq, Hkv, D)
    if rc:
        raise RuntimeError("reference harness failed")
    return dq, dk, dv


def ref_attn_forward(q, k, v, cos, sin, Hq, Hkv, D, apply_rope=True):
    q = np.array(q, np.float32, order="C"); k = np.array(k, np.float32, order="C")
    v = np.ascontiguousarray(v, np.float32)
    S = q.shape[0]
    out = np.zeros((S, Hq * D), np.float32)
    rc = ref_lib().ref_attn_forward(q, k, v, np.ascontiguousarray(cos[:S]), np.ascontiguousarray(sin[:S]), out, S, Hq, Hkv, D, int(apply_rope))
    if rc:
        raise RuntimeError("reference harness failed")
    return out, q, k
