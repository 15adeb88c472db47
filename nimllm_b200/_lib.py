"""ctypes binding of libnimllm_attn.so -- the same prototypes a Nim {.importc, cdecl.}
block declares (include/nimllm_attn.h).  Loading fails loudly when the library has not
been built: there is no CPU or PyTorch fallback for any entry point."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnimllm_attn.so")

F32, BF16 = 0, 1
W_F32, W_BF16, W_Q8_0, W_Q4_0 = 0, 1, 2, 3

_lib = None

vp, i32, i64, f32, sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

PROTOTYPES = {
    # name: (restype, argtypes)
    "nimllm_attn_last_error": (C.c_char_p, []),
    "nimllm_attn_version": (i32, []),
    "nimllm_rope_tables_host": (i32, [vp, vp, i32, i32, f32]),
    "nimllm_kvcache_create": (vp, [i32, i32, i32, i32, i32, i32]),
    "nimllm_kvcache_destroy": (None, [vp]),
    "nimllm_kvcache_reset": (i32, [vp, vp]),
    "nimllm_kvcache_k": (vp, [vp, i32]),
    "nimllm_kvcache_v": (vp, [vp, i32]),
    "nimllm_kvcache_pos": (i32, [vp]),
    "nimllm_kvcache_set_pos": (None, [vp, i32]),
    "nimllm_kvcache_seq_stride": (i64, [vp]),
    "nimllm_kvcache_head_stride": (i64, [vp]),
    "nimllm_rope_append": (i32, [vp, i32, vp, vp, i32, i32, vp, vp, vp, i32, vp, vp, i32, vp, i64, i64,
                                 i32, i32, i32, i32, i32, i32, vp]),
    "nimllm_rope_append_paged": (i32, [vp, i32, vp, vp, i32, i32, vp, vp, vp, i32, vp, vp, i32, vp, i32, i32, i32,
                                       i32, i32, i32, i32, vp]),
    "nimllm_kvpool_create": (vp, [i32, i32, i32, i32, i32, i32, i32, i32, i32]),
    "nimllm_kvpool_destroy": (None, [vp]),
    "nimllm_kvpool_reserve": (i32, [vp, i32, i32]),
    "nimllm_kvpool_release": (i32, [vp, i32]),
    "nimllm_kvpool_sync": (i32, [vp, vp]),
    "nimllm_kvpool_free_pages": (i32, [vp]),
    "nimllm_kvpool_seq_pages": (i32, [vp, i32]),
    "nimllm_kvpool_seq_rows": (i32, [vp, i32]),
    "nimllm_kvpool_table_host": (vp, [vp]),
    "nimllm_kvpool_table": (vp, [vp, i32]),
    "nimllm_kvpool_k": (vp, [vp, i32]),
    "nimllm_kvpool_v": (vp, [vp, i32]),
    "nimllm_attn_decode_plan": (i32, [vp, i32, i32, i32, i32, vp, i32, vp]),
    "nimllm_attn_decode_workspace_bytes": (sz, [i32, i32, i32, i32, i32, i32]),
    "nimllm_attn_decode": (i32, [vp, i32, vp, vp, i32, vp, i64, i64, vp, i32, vp, i32, vp, i32, i32, i32,
                                 i32, f32, i32, vp, sz, vp]),
    "nimllm_attn_decode_paged": (i32, [vp, i32, vp, vp, vp, i32, i32, vp, i32, vp, i32, vp, i32, i32, i32, i32, f32,
                                       vp, sz, vp]),
    "nimllm_attn_decode_noalloc_max_bytes": (sz, []),
    "nimllm_attn_decode_noalloc": (i32, [vp, i32, vp, vp, i32, vp, i64, i64, vp, i32, vp, i32, vp, i32, i32, i32,
                                         i32, f32, i32, vp]),
    "nimllm_qkv_rope_append": (i32, [vp, vp, vp, vp, i32, vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, vp, i64, i64, i32, i32,
                                     i32, i32, i32, i32, i32, vp]),
    "nimllm_wo_residual": (i32, [vp, vp, i32, vp, vp, i32, i32, i32, vp]),
    "nimllm_matvec": (i32, [vp, i32, vp, vp, vp, i32, i32, i32, vp]),
    "nimllm_matvec_status": (i32, [i32]),
    "nimllm_attn_combine": (i32, [vp, i32, i32, i32, i32, vp, i32, vp, vp]),
    "nimllm_peer_exchange_create": (vp, [i32, i32, i32, i32]),
    "nimllm_peer_exchange_export": (i32, [vp, vp]),
    "nimllm_peer_exchange_import": (i32, [vp, i32, vp]),
    "nimllm_peer_exchange_import_local": (i32, [vp, i32, vp]),
    "nimllm_peer_exchange_set_wait_limit": (i32, [vp, i32]),
    "nimllm_peer_exchange_ready": (i32, [vp]),
    "nimllm_peer_exchange_destroy": (None, [vp]),
    "nimllm_attn_combine_peers": (i32, [vp, vp, i32, vp, i32, vp, vp]),
    "nimllm_attn_decode_push_workspace_bytes": (sz, [i32, i32, i32, i32, i32]),
    "nimllm_attn_decode_push": (i32, [vp, vp, i32, vp, vp, vp, i64, i64, vp, i32, i32, i32, i32, i32, f32, vp, sz, vp]),
    "nimllm_attn_wait_combine": (i32, [vp, i32, vp, i32, vp, vp]),
    "nimllm_attn_prefill_workspace_bytes": (sz, [i32, i32, i32, i32, i32, i32]),
    "nimllm_attn_prefill_status": (i32, [i32]),
    "nimllm_attn_prefill": (i32, [vp, vp, vp, i32, vp, vp, i32, vp, i32, i32, i32, i32, i32, f32, i32,
                                  vp, vp, i32, vp, i64, i64, i32, vp, vp, sz, vp]),
    "nimllm_attn_prefill_bwd_workspace_bytes": (sz, [i32, i32, i32, i32]),
    "nimllm_attn_prefill_bwd": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, f32,
                                      vp, sz, vp]),
    "gpu_rope_fwd": (None, [vp, vp, vp, i32, i32, i32, i32]),
    "gpu_extract_head": (None, [vp, vp, i32, i32, i32, i32]),
    "gpu_insert_head": (None, [vp, vp, i32, i32, i32, i32]),
    "gpu_extract_kv_head": (None, [vp, vp, i32, i32, i32, i32, i32]),
    "gpu_causal_mask": (None, [vp, f32, i32]),
    "gpu_scale": (None, [vp, f32, vp, i32]),
    "gpu_softmax_fwd": (None, [vp, vp, i32, i32]),
    "gpu_flash_attn_fwd": (None, [vp, vp, vp, vp, i32, i32, f32, i32]),
    "gpu_matvec_q4_0": (None, [vp, vp, vp, i32, i32]),
    "gpu_matvec_q8_0": (None, [vp, vp, vp, i32, i32]),
}

class NimllmAttnError(RuntimeError):
    pass


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise NimllmAttnError(
                f"{LIB_PATH} is missing: build it with `python -m nimllm_b200.build` "
                "(nvcc, sm_100a). There is no fallback path.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise NimllmAttnError(f"status {rc}: {lib().nimllm_attn_last_error().decode()}")
