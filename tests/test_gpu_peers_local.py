"""The KV-sequence-shard exchange on ONE GPU: the ranks of a box are emulated by exchange buffers
of one process wired to each other directly (no IPC handles), every rank's launches go onto one
stream in an order in which no kernel waits for a later one -- all pushes first, then the waits,
whose flags are then already set.  Covers the push, merge-and-push and wait-and-merge kernels,
the call counters and slots over several steps, and the bounded wait running out."""
import numpy as np
import pytest
import torch

from nimllm_b200 import attention as A, sharding

pytestmark = pytest.mark.gpu


def _shards(B, Hq, Hkv, D, L, world, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    kc = torch.randn(B, Hkv, L, D, generator=g, device="cuda").bfloat16()
    vc = torch.randn(B, Hkv, L, D, generator=g, device="cuda").bfloat16()
    q = torch.randn(B, Hq * D, generator=g, device="cuda").bfloat16()
    return q, kc, vc


@pytest.mark.parametrize("B,Hq,Hkv,D,L,world", [(2, 32, 8, 128, 4096, 2), (3, 9, 3, 64, 3000, 4), (8, 32, 8, 128, 2048, 8)])
def test_fused_push_and_wait_match_unsharded_decode(B, Hq, Hkv, D, L, world):
    q, kc, vc = _shards(B, Hq, Hkv, D, L, world, 31)
    base = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
    full = A.decode_batch(q, kc, vc, max_len=L, seq_stride=Hkv * L * D, head_stride=L * D, **base)
    xs = [sharding.PeerExchange(B * Hq, D, rank=r, world=world) for r in range(world)]
    sharding.PeerExchange.connect_local(xs)
    try:
        for step in range(4):                         # slots and counters roll over
            recs = []
            for r, x in enumerate(xs):
                row0, rows = sharding.kv_shard_rows(L, r, world)
                off = torch.arange(B, device="cuda", dtype=torch.int64) * Hkv * L * D + row0 * D
                x.decode_push(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, **base)
                _, rec = A.decode_batch(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, partials=True, **base)
                recs.append(rec)
            ref = A.combine(torch.stack(recs), D)     # the merge of the same shards without the exchange
            for x in xs:
                merged = x.wait_combine(B * Hq)
                torch.cuda.synchronize()
                assert x.ok()
                assert float((merged - ref).abs().max()) <= 1e-5
                rel = float((merged.view(B, Hq * D) - full).abs().max() / full.abs().max())
                assert rel < 5e-3, rel                # shards round P against their own running maxima
    finally:
        for x in xs:
            x.close()


def test_separate_push_of_records_matches_too():
    """nimllm_attn_combine_peers (push kernel + wait) next to the fused entry: rank 0's second call
    pushes ready-made records while rank 1 uses the fused decode for both of its calls."""
    B, Hq, Hkv, D, L, world = 2, 8, 2, 128, 1024, 2
    q, kc, vc = _shards(B, Hq, Hkv, D, L, world, 32)
    base = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
    xs = [sharding.PeerExchange(B * Hq, D, rank=r, world=world) for r in range(world)]
    sharding.PeerExchange.connect_local(xs)
    try:
        recs = []
        for r in range(world):
            row0, rows = sharding.kv_shard_rows(L, r, world)
            off = torch.arange(B, device="cuda", dtype=torch.int64) * Hkv * L * D + row0 * D
            recs.append(A.decode_batch(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, partials=True, **base)[1])
        ref = A.combine(torch.stack(recs), D)
        for r in (1, 0):
            row0, rows = sharding.kv_shard_rows(L, r, world)
            off = torch.arange(B, device="cuda", dtype=torch.int64) * Hkv * L * D + row0 * D
            xs[r].decode_push(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, **base)
        out0 = xs[0].wait_combine(B * Hq)
        # now rank 0's own combine_peers: its push is call 2, rank 1 catches up with a second decode_push
        row0, rows = sharding.kv_shard_rows(L, 1, world)
        off = torch.arange(B, device="cuda", dtype=torch.int64) * Hkv * L * D + row0 * D
        xs[1].decode_push(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, **base)
        out1 = xs[0].combine(recs[0])                 # push_kernel + wait: rank 1's call 2 is already there
        torch.cuda.synchronize()
        assert xs[0].ok()
        assert float((out0 - ref).abs().max()) <= 1e-5 and float((out1 - ref).abs().max()) <= 1e-5
    finally:
        for x in xs:
            x.close()


def test_bounded_wait_runs_out_and_the_next_call_recovers():
    """Rank 1 skips a step: rank 0's wait gives up after its 50 ms limit, sets the status word and
    returns (no hang, no trap); once rank 1 has caught up, rank 0's next step merges correctly."""
    B, Hq, Hkv, D, L, world = 1, 8, 2, 64, 512, 2
    q, kc, vc = _shards(B, Hq, Hkv, D, L, world, 33)
    base = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
    xs = [sharding.PeerExchange(B * Hq, D, rank=r, world=world, wait_limit_ms=50) for r in range(world)]
    sharding.PeerExchange.connect_local(xs)

    def push(r):
        row0, rows = sharding.kv_shard_rows(L, r, world)
        off = torch.arange(B, device="cuda", dtype=torch.int64) * Hkv * L * D + row0 * D
        xs[r].decode_push(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, **base)
        return A.decode_batch(q, kc, vc, max_len=rows, kv_off=off, head_stride=L * D, partials=True, **base)[1]
    try:
        push(0)                                       # call 1 of rank 0; rank 1 never makes its call 1
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        xs[0].wait_combine(B * Hq)
        t1.record()
        torch.cuda.synchronize()
        assert not xs[0].ok()                         # status word set
        assert 30.0 <= t0.elapsed_time(t1) <= 2000.0  # gave up after about the limit
        xs[0].status.zero_()
        push(1)                                       # rank 1 catches up: its calls 1 and 2
        r1 = push(1)
        r0 = push(0)                                  # call 2 of rank 0
        merged = xs[0].wait_combine(B * Hq)
        torch.cuda.synchronize()
        assert xs[0].ok()
        ref = A.combine(torch.stack([r0, r1]), D)
        assert float((merged - ref).abs().max()) <= 1e-5
    finally:
        for x in xs:
            x.close()
