"""The decode entry point that brings its own scratch (nimllm_attn_decode_noalloc).

It serves host code that cannot obtain device memory when the call is made -- nimllm sizes
one scratch arena at start-up and bump-allocates from it, and cudaMalloc would stall the
device -- so the chunk records live in a fixed array inside the library.  The test calls it
through the C ABI, twice in a row (the array is shared and keeps the previous call's
contents), and checks each result against the ordinary entry point on the same inputs and
against float64 ground truth.
This file sorts last on purpose: a run that stops at the first failure has then already
run every other test."""
import numpy as np
import pytest
import torch

from nimllm_b200 import _lib
from nimllm_b200._lib import BF16, F32

pytestmark = pytest.mark.gpu


def _call(noalloc, q, kc, vc, lens, out, Hq, Hkv, D, cap, chunk, ws=None):
    L = _lib.lib()
    B = q.shape[0]
    args = [q.data_ptr(), BF16, kc.data_ptr(), vc.data_ptr(), BF16, None, Hkv * cap * D, cap * D, lens.data_ptr(),
            cap, out.data_ptr(), F32, None, B, Hq, Hkv, D, 1.0 / np.sqrt(D), chunk]
    if noalloc:
        return L.nimllm_attn_decode_noalloc(*args, torch.cuda.current_stream().cuda_stream)
    need = L.nimllm_attn_decode_workspace_bytes(B, Hq, Hkv, D, cap, chunk)
    return L.nimllm_attn_decode(*args, ws.data_ptr(), need, torch.cuda.current_stream().cuda_stream)


def _ground_truth(q, kc, vc, lens, Hq, Hkv, D, cap):
    """float64 attention on the same bf16-rounded inputs (the CPU restatement of the reference's
    per-head decode loop, accumulating in double)."""
    from oracle import oracle as O
    B = q.shape[0]
    bits = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    return O.decode_batch(q.float().cpu().numpy(), bits(kc), bits(vc), np.arange(B, dtype=np.int64) * Hkv * cap * D,
                          np.full(B, cap * D, np.int64), lens.cpu().numpy().astype(np.int32), Hq, Hkv, D,
                          1.0 / np.sqrt(D), acc64=True)


# (B, Hq, Hkv, D, cap, chunk_rows): explicit chunk lengths run the chunk grid; chunk_rows = 0 runs
# the library's own split (its records and prefix array in the built-in array) at D = 64 and at
# 32q/8kv heads of 128, and falls back to the chunk grid at Hq/Hkv = 8 with heads of 128, whose
# records for the library's own split (10 MB) do not fit
CASES = [(7, 9, 3, 64, 700, 128), (3, 32, 8, 128, 1500, 256), (9, 9, 3, 64, 2100, 0), (4, 32, 8, 128, 3000, 0),
         (5, 8, 1, 128, 9000, 0)]


def test_noalloc_decode_matches_workspace_decode_twice():
    L = _lib.lib()
    assert L.nimllm_attn_decode_noalloc_max_bytes() == 8 << 20
    g = torch.Generator(device="cuda").manual_seed(4242)
    for call, (B, Hq, Hkv, D, cap, chunk) in enumerate(CASES + CASES[2:4]):
        kc = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
        vc = torch.randn(B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
        q = torch.randn(B, Hq * D, generator=g, device="cuda").bfloat16()
        lens = torch.randint(1, cap + 1, (B,), generator=g, device="cuda", dtype=torch.int32)
        lens[0] = cap                                    # at least one sequence is split
        need = L.nimllm_attn_decode_workspace_bytes(B, Hq, Hkv, D, cap, chunk)
        assert need > 0
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        ref = torch.zeros(B, Hq * D, device="cuda")
        out = torch.full((B, Hq * D), float("nan"), device="cuda")
        _lib.check(_call(False, q, kc, vc, lens, ref, Hq, Hkv, D, cap, chunk, ws))
        _lib.check(_call(True, q, kc, vc, lens, out, Hq, Hkv, D, cap, chunk))
        torch.cuda.synchronize()
        a, b = out.cpu().numpy(), ref.cpu().numpy()
        assert np.isfinite(a).all(), f"call {call}: non-finite output"
        truth = _ground_truth(q, kc, vc, lens, Hq, Hkv, D, cap)
        # against float64 ground truth: the bf16 bound of the whole suite
        assert np.abs(a - truth).max() <= 2e-2 * np.abs(truth).max(), f"call {call}: differs from the float64 ground truth"
        if (Hq // Hkv, D, chunk) != (8, 128, 0):
            # same kernel, same split: the two entry points must agree to fp32 rounding, whatever
            # the previous call left in the shared array
            assert np.abs(a - b).max() <= 1e-4 * max(np.abs(b).max(), 1e-30), f"call {call} differs"
        else:
            # here the workspace entry point (given 10 MB) runs the library's own split and the
            # built-in array runs the chunk grid: two orders of summation of the same bf16 products
            assert np.abs(a - b).max() <= 2e-2 * max(np.abs(b).max(), 1e-30), f"call {call} differs"


def test_noalloc_refuses_what_does_not_fit():
    L = _lib.lib()
    one = torch.zeros(16, device="cuda")
    # 4096 sequences x 32 heads x 64 chunks of records is far beyond 8 MiB
    assert L.nimllm_attn_decode_workspace_bytes(4096, 32, 8, 128, 8192, 128) > L.nimllm_attn_decode_noalloc_max_bytes()
    rc = L.nimllm_attn_decode_noalloc(one.data_ptr(), F32, one.data_ptr(), one.data_ptr(), BF16, None, 0, 0, None, 8192,
                                      one.data_ptr(), F32, None, 4096, 32, 8, 128, 0.1, 128, None)
    assert rc == 3
    msg = L.nimllm_attn_last_error().decode()
    assert "built-in scratch" in msg and "workspace" in msg
