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
