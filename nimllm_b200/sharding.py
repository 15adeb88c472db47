"""Host-side partitioning of the attention path over the GPUs of one box.

The reference is single-GPU (one process, stream 0, no collective anywhere in src/); these
helpers define how its per-sequence semantics spread over ranks:

  * independent decode sequences  -> partition_sequences(): whole sequences per rank, balanced
    by KV rows (the bytes a rank must stream), no collective;
  * causal prefill                -> head_shard(): KV heads with their query heads per rank, no
    collective (outputs are disjoint column blocks);
  * one long decode sequence      -> kv_shard_rows(): contiguous KV rows per rank; each rank
    produces (o, m, l) records and gather_partials() all-gathers them (the path's only
    exchange step) for nimllm_attn_combine.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import numpy as np


def partition_sequences(lengths: Sequence[int], world: int) -> List[np.ndarray]:
    """Greedy longest-processing-time assignment of sequences to ranks by KV length.
    Returns, per rank, the sorted indices of its sequences. Deterministic."""
    lengths = np.asarray(lengths, np.int64)
    order = np.argsort(-lengths, kind="stable")
    load = np.zeros(world, np.int64)
    bins: List[list] = [[] for _ in range(world)]
    for i in order:
        r = int(np.argmin(load))          # ties -> lowest rank
        bins[r].append(int(i))
        load[r] += lengths[i]
    return [np.array(sorted(b), np.int64) for b in bins]


def kv_shard_rows(total_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous KV rows [row0, row0 + rows) of a sequence held by `rank`; the remainder of
    total_rows / world goes to the lowest ranks."""
    base, rem = divmod(total_rows, world)
    rows = base + (1 if rank < rem else 0)
    row0 = rank * base + min(rank, rem)
    return row0, rows


def head_shard(n_head: int, n_kv_head: int, rank: int, world: int) -> Tuple[range, range]:
    """KV heads and query heads of `rank` for a head-split prefill (KV-head aligned)."""
    if n_kv_head % world:
        raise ValueError(f"{n_kv_head} KV heads do not split over {world} ranks")
    per = n_kv_head // world
    g = n_head // n_kv_head
    kv = range(rank * per, (rank + 1) * per)
    return kv, range(kv.start * g, kv.stop * g)


def gather_partials(rec, group=None):
    """All-gather of per-rank (o, m, l) records [rows, W] -> [world, rows, W] (any backend)."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    out = torch.empty((world,) + tuple(rec.shape), dtype=rec.dtype, device=rec.device)
    dist.all_gather_into_tensor(out.view(-1), rec.contiguous().view(-1), group=group)
    return out


class PeerExchange:
    """Per-rank exchange buffer for KV-sequence-shard partials.  With a process group the ranks of
    the box are wired together through CUDA IPC handles passed over the (host-side) group; with
    `local_peers` (a list of PeerExchange objects of this process, used by single-GPU tests and by
    one process driving several ranks) the peers' buffers are used directly.  combine() and
    decode_combine() are the data path: peer stores + flags + bounded wait + merge, no collective."""

    def __init__(self, rows_max: int, head_dim: int, group=None, rank=None, world=None, wait_limit_ms=None):
        import ctypes as C
        import torch
        from ._lib import check, lib
        self._lib, self._check = lib(), check
        self.head_dim = head_dim
        self._out = None
        solo = rank is not None
        if solo:
            self.rank, self.world = rank, world
        else:
            import torch.distributed as dist
            self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.handle = self._lib.nimllm_peer_exchange_create(self.rank, self.world, rows_max, head_dim)
        if not self.handle:
            raise RuntimeError(self._lib.nimllm_attn_last_error().decode())
        if wait_limit_ms is not None:
            check(self._lib.nimllm_peer_exchange_set_wait_limit(self.handle, int(wait_limit_ms)))
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")
        if solo:
            return                                  # the caller wires the peers with connect_local()
        mine = C.create_string_buffer(64)
        check(self._lib.nimllm_peer_exchange_export(self.handle, mine))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(mine.raw), group=group)
        err = None
        try:
            for r, h in enumerate(handles):
                check(self._lib.nimllm_peer_exchange_import(self.handle, r, C.create_string_buffer(h, 64)))
            check(self._lib.nimllm_peer_exchange_ready(self.handle))
        except Exception as e:                   # e.g. no peer access between two of the GPUs
            err = str(e)
        # every rank learns whether every rank mapped every buffer (this also orders the mapping
        # before first use); on a failure all ranks raise together instead of one leaving the others waiting
        errs = [None] * self.world
        dist.all_gather_object(errs, err, group=group)
        if any(errs):
            self.close()
            raise RuntimeError("peer exchange setup failed: " + "; ".join(f"rank {r}: {e}" for r, e in enumerate(errs) if e))

    @staticmethod
    def connect_local(exchanges):
        """Wire exchange objects that live in this process (one per rank, same device) to each other."""
        for x in exchanges:
            for y in exchanges:
                x._check(x._lib.nimllm_peer_exchange_import_local(x.handle, y.rank, y.handle))
            x._check(x._lib.nimllm_peer_exchange_ready(x.handle))

    def combine(self, rec, out=None):
        """rec [rows, D+4] fp32 (this rank's records) -> merged [rows, D] fp32."""
        import torch
        rows = rec.shape[0]
        if out is None:
            out = torch.empty((rows, self.head_dim), dtype=torch.float32, device=rec.device)
        self._check(self._lib.nimllm_attn_combine_peers(self.handle, rec.data_ptr(), rows, out.data_ptr(), 0,
                                                        self.status.data_ptr(), torch.cuda.current_stream().cuda_stream))
        return out

    def decode_push(self, q, k_cache, v_cache, *, n_head, n_kv_head, head_dim, max_len, seq_len=None, kv_off=None,
                    seq_stride=0, head_stride=0, scale=None, chunk_rows=0):
        """This rank's shard decode; its merge launch stores the records into every peer's buffer."""
        import math
        import torch
        from . import attention as A
        B = q.shape[0]
        scale = 1.0 / math.sqrt(head_dim) if scale is None else scale
        need = self._lib.nimllm_attn_decode_push_workspace_bytes(B, n_head, n_kv_head, head_dim, max_len)
        ws = A._arena.get(max(need, 1), q.device)
        self._check(self._lib.nimllm_attn_decode_push(
            self.handle, q.data_ptr(), A._code(q), k_cache.data_ptr(), v_cache.data_ptr(),
            kv_off.data_ptr() if kv_off is not None else None, seq_stride, head_stride,
            seq_len.data_ptr() if seq_len is not None else None, max_len, B, n_head, n_kv_head, head_dim, scale,
            ws.data_ptr(), need, torch.cuda.current_stream().cuda_stream))
        return B * n_head

    def wait_combine(self, rows, out=None):
        """Bounded wait for every rank's records of this call, then the merge -> [rows, D] fp32."""
        import torch
        if out is None:
            out = torch.empty((rows, self.head_dim), dtype=torch.float32, device="cuda")
        self._check(self._lib.nimllm_attn_wait_combine(self.handle, rows, out.data_ptr(), 0, self.status.data_ptr(),
                                                       torch.cuda.current_stream().cuda_stream))
        return out

    def decode_combine(self, q, k_cache, v_cache, out=None, **geom):
        """The whole sharded step of this rank: decode + merge-and-push, wait + merge.  q [B, Hq*D],
        the rank's rows of the cache; geom as attention.decode_batch takes it.  Returns [B*Hq, D]."""
        return self.wait_combine(self.decode_push(q, k_cache, v_cache, **geom), out)

    def ok(self) -> bool:
        """False if a wait for a peer's records ever ran out (synchronises)."""
        return int(self.status.item()) == 0

    def close(self):
        if self.handle:
            self._lib.nimllm_peer_exchange_destroy(self.handle)
            self.handle = None
