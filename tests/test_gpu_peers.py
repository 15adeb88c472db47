"""KV-sequence shards exchanged over peer memory on 2+ GPUs, one process per GPU: every rank decodes
its rows, its records reach the peers' buffers (stored by the decode's own merge launch,
nimllm_attn_decode_push, or copied by nimllm_attn_combine_peers), and every rank merges --
compared with the unsharded decode and with the NCCL all-gather + nimllm_attn_combine route.
Skipped on a box with a single GPU (tests/test_gpu_peers_local.py covers the kernels there)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from nimllm_b200 import attention as A, sharding
        B, Hq, Hkv, D, L = 2, 32, 8, 128, 4096
        g = torch.Generator(device="cuda").manual_seed(99)          # same data on every rank
        kc = torch.randn(B, Hkv, L, D, generator=g, device="cuda").bfloat16()
        vc = torch.randn(B, Hkv, L, D, generator=g, device="cuda").bfloat16()
        q = torch.randn(B, Hq * D, generator=g, device="cuda").bfloat16()
        base = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
        full = A.decode_batch(q, kc, vc, max_len=L, seq_stride=Hkv * L * D, head_stride=L * D, **base)
        row0, rows = sharding.kv_shard_rows(L, rank, world)
        off = torch.arange(B, device="cuda", dtype=torch.int64) * Hkv * L * D + row0 * D
        xch = sharding.PeerExchange(B * Hq, D)
        errs = []
        for it in range(5):                                          # several calls: slots and counters roll over
            _, rec = A.decode_batch(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, partials=True, **base)
            merged = xch.combine(rec).view(B, Hq * D) if it % 2 else \
                xch.decode_combine(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, **base).view(B, Hq * D)
            gathered = sharding.gather_partials(rec)
            via_nccl = A.combine(gathered, D).view(B, Hq * D)
            torch.cuda.synchronize()
            errs.append((float((merged - full).abs().max() / full.abs().max()),
                         float((merged - via_nccl).abs().max())))
        ok = xch.ok()
        dist.barrier()
        xch.close()
        q_out.put((rank, errs, ok))
    finally:
        dist.destroy_process_group()


def test_peer_exchange_matches_unsharded_and_nccl():
    world = min(torch.cuda.device_count(), 4)
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q_out)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q_out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for rank, errs, ok in res:
        assert ok, f"rank {rank}: a wait for peer records ran out"
        for rel, vs_nccl in errs:
            assert rel < 5e-3 and vs_nccl < 1e-5, (rank, errs)
