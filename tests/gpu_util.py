"""Helpers shared by the GPU parity tests (imported only from tests marked gpu)."""
import numpy as np
import torch

from oracle import oracle as O


def dev(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    return t.to(dtype) if dtype is not None else t


def host(t):
    return t.detach().float().cpu().numpy()


def bf16_bits(t):
    """bf16 device tensor -> uint16 numpy bit patterns."""
    return t.detach().cpu().view(torch.int16).numpy().view(np.uint16)


def ragged_cache(seed, lens, Hkv, D, dtype, normal, pad_rows=0):
    """Packed ragged KV: sequence b is a [Hkv, cap_b, D] block, blocks laid end to end.
    Returns numpy fp32 arrays (already rounded to dtype), offsets and head strides."""
    B = len(lens)
    off = np.zeros(B, np.int64); hs = np.zeros(B, np.int64)
    total = 0
    for b in range(B):
        cap = max(int(lens[b]) + pad_rows, 1)
        off[b] = total; hs[b] = cap * D
        total += Hkv * cap * D
    k = normal(seed, 10, (total,)); v = normal(seed, 11, (total,))
    if dtype == torch.bfloat16:
        k = O.from_bf16(O.to_bf16(k)); v = O.from_bf16(O.to_bf16(v))
    return k, v, off, hs


class _Raw:
    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = {"data": (int(ptr), False), "shape": tuple(shape), "typestr": typestr,
                                         "version": 2, "strides": None}


def wrap_ptr(ptr, shape, typestr="<f4"):
    """A torch view of raw device memory owned by the C library (no copy)."""
    return torch.as_tensor(_Raw(ptr, shape, typestr), device="cuda")
