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
    """KV for a ragged batch: sequence b owns a [Hkv, cap, D] block (cap = longest sequence +
    pad_rows, so the head stride is uniform) that starts at an arbitrary 8-element-aligned
    offset kv_off[b]; the gaps between blocks differ so that kv_off is exercised.
    Returns fp32 arrays already rounded to dtype, the offsets and per-sequence head strides."""
    B = len(lens)
    cap = max(int(max(lens)) + pad_rows, 1)
    off = np.zeros(B, np.int64)
    total = 0
    for b in range(B):
        off[b] = total
        total += Hkv * cap * D + 8 * ((b * 5) % 7)
    hs = np.full(B, cap * D, np.int64)
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
