"""CPU tests of the C-ABI boundary: the library loads, exports every function that
include/nimllm_attn.h declares, the ctypes binding covers them all, and argument
validation answers with a status and a message before anything touches a GPU."""
import ctypes as C
import os
import re

import numpy as np

from nimllm_b200 import _lib
from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "nimllm_attn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:nimllm|gpu)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_symbols_are_exported_and_bound():
    names = _declared()
    assert len(names) >= 25
    L = _lib.lib()
    for n in names:
        assert hasattr(L, n), f"{n} is declared in include/nimllm_attn.h but not exported"
        assert n in _lib.PROTOTYPES, f"{n} has no ctypes prototype"
    assert sorted(_lib.PROTOTYPES) == names


def test_reference_launcher_names_are_kept():
    """The attention-path launchers the Nim side binds today (src/gpu.nim:227-248,274-276,309-311)."""
    for n in ["gpu_rope_fwd", "gpu_extract_head", "gpu_insert_head", "gpu_extract_kv_head", "gpu_causal_mask",
              "gpu_scale", "gpu_softmax_fwd", "gpu_flash_attn_fwd"]:
        assert n in _declared()


def test_validation_errors_have_status_and_message():
    L = _lib.lib()
    rc = L.nimllm_attn_decode(None, 0, None, None, 0, None, 0, 0, None, 16, None, 0, None, 1, 4, 2, 64, 0.125, 0,
                              None, 0, None)
    assert rc == 1 and b"null" in L.nimllm_attn_last_error()
    one = C.c_void_p(16)
    rc = L.nimllm_attn_decode(one, 0, one, one, 0, None, 0, 0, None, 16, one, 0, None, 1, 9, 2, 64, 0.125, 0, None,
                              0, None)
    assert rc == 1 and b"bad shape" in L.nimllm_attn_last_error()       # 9 heads over 2 KV heads
    rc = L.nimllm_attn_decode(one, 0, one, one, 0, None, 0, 0, None, 16, one, 0, None, 1, 4, 2, 96, 0.125, 0, None,
                              0, None)
    assert rc == 2 and b"head_dim" in L.nimllm_attn_last_error()
    rc = L.nimllm_attn_decode(one, 0, one, one, 0, None, 0, 0, None, 4096, one, 0, None, 1, 4, 2, 64, 0.125, 128,
                              None, 0, None)
    assert rc == 3 and b"workspace" in L.nimllm_attn_last_error()
    # a bf16 cache whose KV heads start 6 elements apart: 16-byte loads would be misaligned
    rc = L.nimllm_attn_decode(one, 0, one, one, 1, None, 4096, 6, None, 16, one, 0, None, 1, 4, 2, 64, 0.125, 0, None,
                              0, None)
    assert rc == 1 and b"multiples of 16 bytes" in L.nimllm_attn_last_error()
    rc = L.nimllm_attn_prefill(None, None, None, 0, None, None, 0, None, 1, 8, 4, 2, 64, 0.125, 1, None, None, 0,
                               None, 0, 0, 0, None, None, 0, None)
    assert rc == 1
    rc = L.nimllm_attn_combine(None, 2, 4, 64, 68, None, 0, None, None)
    assert rc == 1
    rc = L.nimllm_rope_append(None, 4, one, one, 0, 1, one, None, None, 0, None, None, 0, None, 0, 0, 0, 0, 1, 1,
                              2, 64, None)
    assert rc == 1 and b"both RoPE tables" in L.nimllm_attn_last_error()
    assert L.nimllm_attn_version() >= 100


def test_workspace_sizing():
    L = _lib.lib()
    assert L.nimllm_attn_decode_workspace_bytes(4, 8, 2, 64, 100, 128) == 0       # one chunk: no scratch
    n = L.nimllm_attn_decode_workspace_bytes(4, 8, 2, 64, 1000, 128)
    assert n == 8 * 4 * 8 * (64 + 4) * 4                                          # ceil(1000/128) chunks
    assert L.nimllm_attn_prefill_workspace_bytes(1, 128, 9, 3, 64, _lib.F32) == 0


def test_host_rope_tables_equal_oracle():
    cos = np.empty((512, 32), np.float32); sin = np.empty_like(cos)
    assert _lib.lib().nimllm_rope_tables_host(cos.ctypes.data, sin.ctypes.data, 512, 64, 10000.0) == 0
    oc, os_ = O.rope_tables(512, 64, 10000.0)
    np.testing.assert_array_equal(cos, oc)
    np.testing.assert_array_equal(sin, os_)
    cos = np.empty((64, 64), np.float32); sin = np.empty_like(cos)
    _lib.lib().nimllm_rope_tables_host(cos.ctypes.data, sin.ctypes.data, 64, 128, 500000.0)
    oc, os_ = O.rope_tables(64, 128, 500000.0)
    np.testing.assert_array_equal(cos, oc)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    try:
        _lib.lib()
        assert False, "expected NimllmAttnError"
    except _lib.NimllmAttnError as e:
        assert "no fallback" in str(e)


def test_balanced_decode_plan_covers_every_unit_once():
    """The balanced decode kernel cuts the flattened batch into equal spans per warp.  Replayed on
    the host (same code as the kernels): every unit of every (sequence, KV head) pair is covered
    exactly once, whole pairs are never also cut, a warp cuts at most two pairs, and the merge
    side finds exactly the records the walk wrote."""
    import ctypes as C
    import numpy as np
    from nimllm_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(11)
    for trial in range(300):
        B = int(rng.integers(1, 40)); Hkv = int(rng.integers(1, 9)); unit = int(rng.choice([16, 32]))
        lens = rng.choice([0, 0, 1, 5, 16, 33, 100, 700, 4096, int(rng.integers(0, 3000))], size=B).astype(np.int32)
        warps = int(rng.choice([8, 37, 1184]))
        segs = np.zeros((20000, 6), np.int32); pairs = np.zeros((B * Hkv, 3), np.int32)
        n = L.nimllm_attn_decode_plan(lens.ctypes.data_as(C.c_void_p), B, Hkv, unit, warps,
                                              segs.ctypes.data_as(C.c_void_p), len(segs), pairs.ctypes.data_as(C.c_void_p))
        assert n >= 0
        segs = segs[:n]
        units = (lens + unit - 1) // unit
        cover = {}
        records = {}
        for w, b, h, i0, i1, slot in segs.tolist():
            assert 0 <= i0 < i1 <= units[b]
            cover.setdefault((b, h), []).append((i0, i1, w, slot))
            if slot >= 0:
                assert (w, slot) not in records and slot in (0, 1)
                records[(w, slot)] = (b, h, i0, i1)
        for b in range(B):
            for h in range(Hkv):
                pieces = sorted(cover.get((b, h), []))
                if units[b] == 0:
                    assert not pieces
                    continue
                assert pieces[0][0] == 0 and pieces[-1][1] == units[b]
                assert all(pieces[i][1] == pieces[i + 1][0] for i in range(len(pieces) - 1))
                wf, cnt, sf = pairs[b * Hkv + h].tolist()
                assert cnt == len(pieces)
                if cnt == 1:
                    assert pieces[0][3] == -1               # a whole pair is written directly
                else:
                    for i, (i0, i1, w, slot) in enumerate(pieces):
                        assert w == wf + i and slot == (sf if i == 0 else 0)
                        assert records[(w, slot)] == (b, h, i0, i1)
        total = int(units.sum()) * Hkv
        if total:
            per_warp = np.bincount(segs[:, 0], weights=(segs[:, 4] - segs[:, 3]))
            assert per_warp.max() - per_warp[per_warp > 0].min() <= 1     # equal spans
