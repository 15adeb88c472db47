"""Host layer over the C ABI, named after the reference's procedures.

  reference (src/model.nim, src/gpu.nim)          here
  ------------------------------------------     ---------------------------------
  initModel's RoPE table loop (:153-163)          rope_tables()
  KvCache / initKvCache / resetKvCache (:70-73,   KvCache (one device allocation per K and V,
    :729-746)                                       [layer][seq][kv head][row][D])
  forward()'s attention block (:494-508)          attn_forward()
  forwardCached()'s attention block (:788-840)    attn_forward_cached()
  (no counterpart: batch 1 only)                  decode_batch(), combine()
  chat loop's reset-when-full cache policy        PagedKvPool (pages shared by many sequences),
    (src/chat.nim:86-91)                            rope_append_paged(), decode_paged()

torch is used for device memory and streams only; every computation goes through
libnimllm_attn.so and raises if that library is missing or reports an error."""
from __future__ import annotations

import math
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import BF16, F32, check, lib

_DT = {torch.float32: F32, torch.bfloat16: BF16}


def _code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise _lib.NimllmAttnError(f"unsupported dtype {t.dtype}: float32 and bfloat16 are built") from None


def _ptr(t: Optional[torch.Tensor]):
    if t is None:
        return None
    if not t.is_cuda:
        raise _lib.NimllmAttnError("device tensor expected (there is no CPU path)")
    if not t.is_contiguous():
        raise _lib.NimllmAttnError("contiguous tensor expected")
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


class _Arena:
    """Caller-owned scratch, the role trackedCreate's arena plays in the reference
    (src/autograd.nim:37-51): grown outside the hot loop, reused by every call."""

    def __init__(self):
        self.buf = {}

    def get(self, nbytes: int, device) -> Optional[torch.Tensor]:
        if nbytes == 0:
            return None
        key = torch.device(device).index or 0
        cur = self.buf.get(key)
        if cur is None or cur.numel() < nbytes:
            cur = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
            self.buf[key] = cur
        return cur


_arena = _Arena()


def rope_tables(max_pos: int, head_dim: int, base: float, device="cuda"):
    """cos/sin tables [max_pos, D/2] fp32, computed on the host as initModel does."""
    cos = np.empty((max_pos, head_dim // 2), np.float32)
    sin = np.empty_like(cos)
    check(lib().nimllm_rope_tables_host(cos.ctypes.data, sin.ctypes.data, max_pos, head_dim, float(base)))
    return torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device)


class KvCache:
    """K and V as [n_layer, n_seq, Hkv, max_seq, D] device tensors plus the host `pos`."""

    def __init__(self, n_layer, n_seq, n_kv_head, max_seq, head_dim, dtype=torch.float32, device="cuda"):
        shape = (n_layer, n_seq, n_kv_head, max_seq, head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.pos = 0
        self.n_layer, self.n_seq, self.n_kv_head, self.max_seq, self.head_dim = shape
        self.seq_stride = n_kv_head * max_seq * head_dim
        self.head_stride = max_seq * head_dim

    def reset(self):
        self.k.zero_()
        self.v.zero_()
        self.pos = 0


class _DeviceView:
    """Device memory owned by the library, shown to torch through __cuda_array_interface__."""

    def __init__(self, ptr, shape, typestr, owner):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}
        self._owner = owner


class PagedKvPool:
    """The library's block manager of the paged cache (nimllm_kvpool_*): pages shared by up to max_seqs
    sequences instead of the reference's one-conversation cache that is reset when full
    (src/chat.nim:86-91).  on_device=False keeps only the host table (no CUDA call)."""

    def __init__(self, n_layer, n_pages, page_rows, n_kv_head, head_dim, max_seqs, max_pages_per_seq,
                 dtype=torch.bfloat16, on_device=True):
        self.shape = (n_pages, n_kv_head, page_rows, head_dim)
        self.n_layer, self.max_seqs, self.max_pages, self.dtype, self.on_device = n_layer, max_seqs, max_pages_per_seq, dtype, on_device
        self._h = lib().nimllm_kvpool_create(n_layer, n_pages, page_rows, n_kv_head, head_dim, _DT[dtype], max_seqs,
                                             max_pages_per_seq, int(on_device))
        if not self._h:
            raise _lib.NimllmAttnError(lib().nimllm_attn_last_error().decode())

    def close(self):
        if self._h:
            lib().nimllm_kvpool_destroy(self._h)
            self._h = None

    __del__ = close

    def reserve(self, seq: int, rows_total: int):
        check(lib().nimllm_kvpool_reserve(self._h, seq, rows_total))

    def release(self, seq: int):
        check(lib().nimllm_kvpool_release(self._h, seq))

    def sync(self):
        check(lib().nimllm_kvpool_sync(self._h, _stream() if self.on_device else None))

    @property
    def free_pages(self) -> int:
        return lib().nimllm_kvpool_free_pages(self._h)

    def seq_pages(self, seq: int) -> int:
        return lib().nimllm_kvpool_seq_pages(self._h, seq)

    def seq_rows(self, seq: int) -> int:
        return lib().nimllm_kvpool_seq_rows(self._h, seq)

    def table_host(self) -> np.ndarray:
        import ctypes
        buf = (ctypes.c_int32 * (self.max_seqs * self.max_pages)).from_address(lib().nimllm_kvpool_table_host(self._h))
        return np.frombuffer(buf, dtype=np.int32).reshape(self.max_seqs, self.max_pages).copy()

    def table(self, first_seq: int = 0) -> torch.Tensor:
        ptr = lib().nimllm_kvpool_table(self._h, first_seq)
        if not ptr:
            raise _lib.NimllmAttnError("the pool has no device table (on_device=False or bad first_seq)")
        return torch.as_tensor(_DeviceView(ptr, (self.max_seqs - first_seq, self.max_pages), "<i4", self), device="cuda")

    def _pages(self, fn, layer):
        ptr = fn(self._h, layer)
        if not ptr:
            raise _lib.NimllmAttnError("the pool has no device pages (on_device=False or bad layer)")
        if self.dtype == torch.float32:
            return torch.as_tensor(_DeviceView(ptr, self.shape, "<f4", self), device="cuda")
        return torch.as_tensor(_DeviceView(ptr, self.shape, "<i2", self), device="cuda").view(torch.bfloat16)

    def k(self, layer: int) -> torch.Tensor:
        return self._pages(lib().nimllm_kvpool_k, layer)

    def v(self, layer: int) -> torch.Tensor:
        return self._pages(lib().nimllm_kvpool_v, layer)


def rope_append(q, k_new, v_new, cos, sin, *, n_head, n_kv_head, head_dim, pos0=0, seq_pos=None,
                k_cache=None, v_cache=None, kv_off=None, seq_stride=0, head_stride=0, cache_row0=0,
                max_seq=0, write_back_k=True):
    """Fused RoPE(q), RoPE(k_new) + cast + scatter of k_new / v_new into the cache."""
    B, n = k_new.shape[0], k_new.shape[1]
    check(lib().nimllm_rope_append(
        _ptr(q), n_head, _ptr(k_new), _ptr(v_new), _code(k_new), int(write_back_k), _ptr(cos), _ptr(sin),
        _ptr(seq_pos), pos0, _ptr(k_cache), _ptr(v_cache), _code(k_cache) if k_cache is not None else F32,
        _ptr(kv_off), seq_stride, head_stride, cache_row0, max_seq, B, n, n_kv_head, head_dim, _stream()))


def decode_batch(q, k_cache, v_cache, *, n_head, n_kv_head, head_dim, max_len, seq_len=None, kv_off=None,
                 seq_stride=0, head_stride=0, scale=None, chunk_rows=0, out=None, out_dtype=torch.float32,
                 partials=False):
    """GQA decode of a batch of independent sequences. Returns out [B, Hq*D] (and the
    (o, m, l) records [B*Hq, D+4] when partials=True)."""
    B = q.shape[0]
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    if out is None:
        out = torch.empty((B, n_head * head_dim), dtype=out_dtype, device=q.device)
    rec = torch.empty((B * n_head, head_dim + 4), dtype=torch.float32, device=q.device) if partials else None
    need = lib().nimllm_attn_decode_workspace_bytes(B, n_head, n_kv_head, head_dim, max_len, chunk_rows)
    ws = _arena.get(need, q.device)
    check(lib().nimllm_attn_decode(
        _ptr(q), _code(q), _ptr(k_cache), _ptr(v_cache), _code(k_cache), _ptr(kv_off), seq_stride, head_stride,
        _ptr(seq_len), max_len, _ptr(out), _code(out), _ptr(rec), B, n_head, n_kv_head, head_dim, scale,
        chunk_rows, _ptr(ws), need, _stream()))
    return (out, rec) if partials else out


def decode_paged(q, k_pages, v_pages, page_table, *, n_head, n_kv_head, head_dim, max_len, seq_len=None, scale=None,
                 out=None, out_dtype=torch.float32, partials=False):
    """GQA decode over a paged bf16 cache: k_pages / v_pages [n_pages, Hkv, page_rows, D], page_table
    int32 [B, max_pages].  Returns out [B, Hq*D] (and the (o, m, l) records when partials=True)."""
    B = q.shape[0]
    page_rows = k_pages.shape[2]
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    if out is None:
        out = torch.empty((B, n_head * head_dim), dtype=out_dtype, device=q.device)
    rec = torch.empty((B * n_head, head_dim + 4), dtype=torch.float32, device=q.device) if partials else None
    need = lib().nimllm_attn_decode_workspace_bytes(B, n_head, n_kv_head, head_dim, max_len, 0)
    ws = _arena.get(need, q.device)
    check(lib().nimllm_attn_decode_paged(
        _ptr(q), _code(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1], page_rows,
        _ptr(seq_len), max_len, _ptr(out), _code(out), _ptr(rec), B, n_head, n_kv_head, head_dim, scale,
        _ptr(ws), need, _stream()))
    return (out, rec) if partials else out


def rope_append_paged(q, k_new, v_new, cos, sin, k_pages, v_pages, page_table, *, n_head, n_kv_head, head_dim,
                      pos0=0, seq_pos=None, write_back_k=True):
    """rope_append into a paged cache: k_pages / v_pages [n_pages, Hkv, page_rows, D], page_table int32
    [B, max_pages]; every new row finds its own page, so n > 1 may cross page boundaries."""
    B, n = k_new.shape[0], k_new.shape[1]
    check(lib().nimllm_rope_append_paged(
        _ptr(q), n_head, _ptr(k_new), _ptr(v_new), _code(k_new), int(write_back_k), _ptr(cos), _ptr(sin),
        _ptr(seq_pos), pos0, _ptr(k_pages), _ptr(v_pages), _code(k_pages), _ptr(page_table), page_table.shape[1],
        k_pages.shape[2], k_pages.shape[0], B, n, n_kv_head, head_dim, _stream()))


def _wtype(w, w_type):
    if w_type is not None:
        return w_type
    return {torch.float32: _lib.W_F32, torch.bfloat16: _lib.W_BF16}[w.dtype]


def qkv_rope_append(x_norm, wq, wk, wv, cos, sin, *, n_head, n_kv_head, head_dim, w_type=None, pos0=0, seq_pos=None,
                    k_cache=None, v_cache=None, kv_off=None, seq_stride=0, head_stride=0, cache_row0=0, max_seq=0,
                    want_kv=False):
    """The q / k / v projections, RoPE and the cache append of one decode step in one launch
    (forwardCached, src/model.nim:775-815).  x_norm [B, n_embd] fp32; weights [out, n_embd] as fp32 or
    bf16 tensors, or uint8 tensors of Q8_0 / Q4_0 blocks with w_type given.  Returns rotated q
    [B, Hq*D] (and rotated k, raw v [B, Hkv*D] with want_kv)."""
    B, n_embd = x_norm.shape
    q = torch.empty((B, n_head * head_dim), dtype=torch.float32, device=x_norm.device)
    k = torch.empty((B, n_kv_head * head_dim), dtype=torch.float32, device=x_norm.device) if want_kv or k_cache is None else None
    v = torch.empty_like(k) if k is not None else None
    check(lib().nimllm_qkv_rope_append(
        _ptr(x_norm), _ptr(wq), _ptr(wk), _ptr(wv), _wtype(wq, w_type), _ptr(q), _ptr(k), _ptr(v), _ptr(cos), _ptr(sin),
        _ptr(seq_pos), pos0, _ptr(k_cache), _ptr(v_cache), _code(k_cache) if k_cache is not None else F32, _ptr(kv_off),
        seq_stride, head_stride, cache_row0, max_seq, B, n_embd, n_head, n_kv_head, head_dim, _stream()))
    return (q, k, v) if k is not None else q


def wo_residual(attn_out, wo, x_resid, *, w_type=None):
    """x_resid + wo attn_out (src/model.nim:843-849) in one launch; attn_out [B, n_in], wo [n_embd, n_in]."""
    B, n_in = attn_out.shape
    n_embd = x_resid.shape[1]
    out = torch.empty_like(x_resid)
    check(lib().nimllm_wo_residual(_ptr(attn_out), _ptr(wo), _wtype(wo, w_type), _ptr(x_resid), _ptr(out), B, n_embd, n_in,
                                   _stream()))
    return out


def matvec(w, x, rows, *, w_type=None, residual=None):
    """y[b] = w x[b] (+ residual[b]); x [B, cols] fp32, w [rows, cols] in any of the weight types."""
    B, cols = x.shape
    y = torch.empty((B, rows), dtype=torch.float32, device=x.device)
    check(lib().nimllm_matvec(_ptr(w), _wtype(w, w_type), _ptr(x), _ptr(residual), _ptr(y), B, rows, cols, _stream()))
    return y


def matvec_status(reset: bool = True) -> int:
    """0 when every staged projection launch since the last reset ran to completion, 1 when a bounded wait
    for weight copies gave up (results of that launch are incomplete).  Synchronises the device."""
    rc = lib().nimllm_matvec_status(int(reset))
    if rc < 0:
        check(-rc)
    return rc


def combine(parts, head_dim, out_dtype=torch.float32, partials=False):
    """Merge (o, m, l) records [n_parts, rows, D+4] -> out [rows, D]."""
    n_parts, rows, W = parts.shape
    out = torch.empty((rows, head_dim), dtype=out_dtype, device=parts.device)
    rec = torch.empty((rows, W), dtype=torch.float32, device=parts.device) if partials else None
    check(lib().nimllm_attn_combine(_ptr(parts), n_parts, rows, head_dim, W, _ptr(out), _code(out), _ptr(rec),
                                    _stream()))
    return (out, rec) if partials else out


def attn_forward(q, k, v, cos, sin, *, n_head, n_kv_head, head_dim, pos0=0, save_cache=True, kv: KvCache = None,
                 layer=0, scale=None, lse=None):
    """forward()'s attention block: RoPE(q, k) then causal GQA attention.
    q [B,S,Hq*D] (or [S,Hq*D]), k, v [B,S,Hkv*D]. q and k are rotated in place like the
    reference's ropeFwd does; with kv given, rows pos0.. of the cache are filled."""
    squeeze = q.dim() == 2
    if squeeze:
        q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
    B, S = q.shape[0], q.shape[1]
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    out = torch.empty_like(q)
    need = lib().nimllm_attn_prefill_workspace_bytes(B, S, n_head, n_kv_head, head_dim, _code(q))
    ws = _arena.get(need, q.device)
    kc = kv.k[layer] if kv is not None else None
    vc = kv.v[layer] if kv is not None else None
    check(lib().nimllm_attn_prefill(
        _ptr(q), _ptr(k), _ptr(v), _code(q), _ptr(cos), _ptr(sin), pos0, _ptr(out), B, S, n_head, n_kv_head,
        head_dim, scale, int(save_cache), _ptr(kc), _ptr(vc), _code(kc) if kc is not None else F32, None,
        kv.seq_stride if kv is not None else 0, kv.head_stride if kv is not None else 0,
        kv.max_seq if kv is not None else 0, _ptr(lse), _ptr(ws), need, _stream()))
    return out[0] if squeeze else out


def prefill_status(reset: bool = True) -> int:
    """0 when every bf16 prefill launch on the current device since the last reset ran to
    completion, 1 when a bounded wait inside one gave up (its outputs are incomplete).  Synchronises."""
    rc = lib().nimllm_attn_prefill_status(int(reset))
    if rc < 0:
        check(-rc)
    return rc


def attn_backward(q_rot, k_rot, v, out, dout, lse, cos, sin, *, n_head, n_kv_head, head_dim, pos0=0, scale=None):
    """Backward of the causal attention block (fp32): returns (dq, dk, dv) in the pre-RoPE space.
    q_rot / k_rot are the rotated activations attn_forward(save_cache=True) left, lse its row
    log-sum-exp [B, Hq, S]."""
    if q_rot.dim() == 2:
        q_rot, k_rot, v, out, dout = (t.unsqueeze(0) for t in (q_rot, k_rot, v, out, dout))
    B, S = q_rot.shape[0], q_rot.shape[1]
    scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
    dq, dk, dv = torch.empty_like(q_rot), torch.empty_like(k_rot), torch.empty_like(v)
    need = lib().nimllm_attn_prefill_bwd_workspace_bytes(B, S, n_head, head_dim)
    ws = _arena.get(need, q_rot.device)
    check(lib().nimllm_attn_prefill_bwd(
        _ptr(q_rot), _ptr(k_rot), _ptr(v), _ptr(out), _ptr(dout), _ptr(lse), _ptr(cos), _ptr(sin), pos0,
        _ptr(dq), _ptr(dk), _ptr(dv), B, S, n_head, n_kv_head, head_dim, scale, _ptr(ws), need, _stream()))
    return dq, dk, dv


def attn_forward_cached(kv: KvCache, layer, q, k_new, v_new, cos, sin, *, n_head, scale=None, chunk_rows=0):
    """forwardCached()'s attention block for one new token per sequence (newTokens == 1):
    RoPE(q, k_new) at row kv.pos, append, attend rows 0..kv.pos.  q [n_seq, Hq*D],
    k_new / v_new [n_seq, Hkv*D].  The caller advances kv.pos after the last layer, as
    the reference does (src/model.nim:890)."""
    B = q.shape[0]
    D, Hkv = kv.head_dim, kv.n_kv_head
    kc, vc = kv.k[layer], kv.v[layer]
    rope_append(q.view(B, 1, -1), k_new.view(B, 1, -1), v_new.view(B, 1, -1), cos, sin, n_head=n_head,
                n_kv_head=Hkv, head_dim=D, pos0=kv.pos, k_cache=kc, v_cache=vc, seq_stride=kv.seq_stride,
                head_stride=kv.head_stride, max_seq=kv.max_seq)
    return decode_batch(q, kc, vc, n_head=n_head, n_kv_head=Hkv, head_dim=D, max_len=kv.pos + 1,
                        seq_stride=kv.seq_stride, head_stride=kv.head_stride, scale=scale,
                        chunk_rows=chunk_rows, out_dtype=torch.float32)
