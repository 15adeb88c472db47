#!/usr/bin/env python
"""Benchmark of the attention hot path on synthetic data of the named shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload all|c3|c5|c4|c3p] [--impl reference]

One JSON line on stdout (rank 0).  A step is one pass of the hot path over one batch:

  c3            batched GQA decode, 256 ragged sequences (L ~ U[512, 4096]), 9 q / 3 kv heads,
                D = 64, bf16 KV cache.  Metric: KV GB/s (HBM roofline).  With N GPUs every rank
                holds its own 256 sequences (weak scaling, no collective on the data path).
  c3p           the same ONE batch of 256 sequences partitioned over the N GPUs by greedy
                longest-first on the KV rows (strong scaling, no collective).
  c5            long-context decode, 8 x 131072 rows, 32 q / 8 kv heads, D = 128, bf16; the KV
                sequence is sharded over the ranks and the (o, m, l) partials are exchanged
                (peer stores or an NCCL all-gather) and merged (strong scaling).
  c4            causal prefill 4 x 8192, 32 q / 8 kv heads, D = 128, bf16 (tensor roofline); KV
                heads are split over the ranks, no collective (strong scaling).
  all (default) the c3 line is the headline; the c4, c5 and c3p measurements of the same run
                are attached to it under "also" (each with its own value, roofline and clocks).

`value` is timed with CUDA events on the launching stream with inputs resident in HBM;
`e2e` is the same metric through the host-facing call: every step copies that step's
activations from pinned host memory, runs RoPE + cache append + attention, and copies the
result back.  `--impl reference` times the CPU restatement of the reference's attention
(the reference has no CPU forward of its own) on the host cores and, when the reference's
kernels were compiled into oracle/_ref, also its own GPU launch sequence on the same batch.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEEDS = {"c3": 20253, "c4": 20254, "c5": 20255}
SHAPE_OVERRIDE = None   # set by --shape (profiling only); the defaults are the named benchmark shapes
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from one ncu
# capture of that kernel on this workload (a constant: re-capture after changing the kernel)
NCU_TRAFFIC_BYTES = {"c3": 462600000 + 900000, "c3p": 462600000 + 900000, "c5": 4295500000 + 1900000,
                     "c4": 1903500000 + 231800000,
                     "proj_q8_0": 32 * (26796252 + 17897384)}
WORKLOAD_TEXT = {
    "c3": "C3 batched GQA decode: 256 ragged sequences per GPU, L~U[512,4096], 9q/3kv heads, D=64, bf16 KV",
    "c3p": "C3 batched GQA decode: one batch of 256 ragged sequences partitioned over the GPUs, L~U[512,4096], 9q/3kv heads, D=64, bf16 KV",
    "c5": "C5 long-context decode: 8 x 131072 rows, 32q/8kv heads, D=128, bf16 KV, KV sequence sharded over the GPUs",
}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm": float(p["hbm_gbs"]), "bf16": float(p["bf16_tflops"]),
                "bf16_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm": 6650.0, "bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self.stop_flag = [], set(), None, False
        self.index, self.thread, self.ok = index, None, False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception as e:  # pragma: no cover
            log(f"clock sampler: NVML unavailable ({e})")

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
                 "hw_thermal_slowdown": 0x40, "hw_power_brake": 0x80}
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self.ok:
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop_flag = True
        if self.thread:
            self.thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


class Dist:
    def __init__(self, n_gpus):
        import torch
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != n_gpus:
            if self.world == 1 and n_gpus > 1:
                raise SystemExit(f"--gpus {n_gpus} needs a launch with torch.distributed.run --nproc-per-node {n_gpus}")
        torch.cuda.set_device(self.local)
        self.torch = torch
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max(self, x):
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum(self, x):
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_steps(torch, step, steps, warmup, flush=None, dist=None):
    """W untimed warm-up steps, then exactly K steps, each bracketed by CUDA events on the
    current stream with an L2 flush outside the bracket.  Returns the per-step ms list."""
    for _ in range(warmup):
        if flush is not None:
            flush.zero_()
        step()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    if dist is not None:
        dist.barrier()
    else:
        torch.cuda.synchronize()
    for a, b in ev:
        if flush is not None:
            flush.zero_()
        a.record()
        step()
        b.record()
    if dist is not None:
        dist.barrier()
    else:
        torch.cuda.synchronize()
    return [a.elapsed_time(b) for a, b in ev]


def timed_bracket(torch, step, steps, warmup, dist=None):
    """W untimed warm-up steps, then exactly K steps between ONE pair of CUDA events on the current
    stream, a barrier + synchronize on both sides.  For steps whose inputs are larger than L2 (no flush
    between them).  Returns the ms of the whole bracket."""
    for _ in range(warmup):
        step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist is not None:
        dist.barrier()
    else:
        torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        step()
    b.record()
    if dist is not None:
        dist.barrier()
    else:
        torch.cuda.synchronize()
    return a.elapsed_time(b)


# ------------------------------------------------------------------------------- c3 / c5
def c3_lengths(rank):
    """The 256 sequence lengths of the c3 batch of `rank` (rank 0's batch is THE batch of c3p)."""
    return np.random.Generator(np.random.Philox(key=SEEDS["c3"] + 1000 * rank)).integers(512, 4097, 256).astype(np.int32)


def decode_workload(name, rank, world, device="cuda"):
    """Shapes and seeded synthetic data of the decode configurations, built on `device`."""
    import torch
    gen = torch.Generator(device=device)
    if name in ("c3", "c3p"):
        Hq, Hkv, D, cap = 9, 3, 64, 4096
        if name == "c3":
            gen.manual_seed(SEEDS[name] + 1000 * rank)
            lens = c3_lengths(rank)
        else:
            # ONE batch of 256 sequences; this rank holds the sequences the greedy longest-first
            # partition by KV rows gives it (nimllm_b200.sharding.partition_sequences)
            from nimllm_b200 import sharding
            all_lens = c3_lengths(0)
            mine = sharding.partition_sequences(all_lens, world)[rank]
            lens = all_lens[mine]
            gen.manual_seed(SEEDS["c3"] + 77 + rank)
        B = len(lens)
        rows = cap
    else:
        B, Hq, Hkv, D, L = 8, 32, 8, 128, 131072
        if SHAPE_OVERRIDE:                              # --shape B,Hq,Hkv,D,L: profiling / experiments
            B, Hq, Hkv, D, L = SHAPE_OVERRIDE
        gen.manual_seed(SEEDS[name] + 1000 * rank)
        rows = L // world           # this rank's contiguous slice of every KV head
        cap = rows
        lens = np.full(B, rows, np.int32)
    kc = torch.empty(B, Hkv, cap, D, dtype=torch.bfloat16, device=device)
    vc = torch.empty_like(kc)
    for t in (kc, vc):              # fill in slices: randn in fp32 then round, without a 2x fp32 copy
        for b in range(B):
            t[b] = torch.randn(Hkv, cap, D, generator=gen, device=device).bfloat16()
    kv_bytes = int(lens.astype(np.int64).sum()) * 2 * Hkv * D * 2
    qo_bytes = B * Hq * D * (2 + 4)
    # c3 moves 453 MB per step, 3.6x the 126 MB L2: the timed loop rotates over `copies` replicas
    # of the cache so that a step never finds lines of its own data left by the step before
    # (>= 1.2 GB are touched between two uses of a replica; a partition of the batch is smaller, so
    # it gets more replicas).  No flush kernel is used: a flush that WRITES leaves L2 full of dirty
    # lines whose write-back is charged to the next step.
    copies = 1
    if name in ("c3", "c3p") and device != "cpu":
        copies = max(3, int(math.ceil(1.2e9 / max(kv_bytes, 1))))
    kcs = [kc] + [kc.clone() for _ in range(copies - 1)]
    vcs = [vc] + [vc.clone() for _ in range(copies - 1)]
    qgen = torch.Generator(device=device).manual_seed(SEEDS[name if name != "c3p" else "c3"] + 7)   # q is the same on every rank of c5
    q = torch.randn(B, Hq * D, generator=qgen if name == "c5" else gen, device=device).bfloat16()
    return dict(B=B, Hq=Hq, Hkv=Hkv, D=D, cap=cap, lens=lens, kc=kc, vc=vc, kcs=kcs, vcs=vcs, q=q, rows=rows,
                bytes=kv_bytes + qo_bytes, scale=1.0 / math.sqrt(D), copies=copies)


def sustained_loop(torch, step, ms_per_step, dist, seconds=2.0, unit_steps=1, capture=True):
    """The same step launched back to back for about `seconds` of device time (captured as a CUDA
    graph of `unit_steps` steps so that the host's launch rate is not what is measured), timed
    with one pair of events; returns (ms per step, steps) as the max over ranks."""
    n_units = max(2, int(math.ceil(seconds * 1e3 / max(ms_per_step, 1e-3) / unit_steps)))
    n_units = min(n_units, 200000)
    try:
        if not capture:
            raise RuntimeError("already a graph")
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(unit_steps):
                step()
        run = g.replay
    except Exception as e:
        if capture:  # pragma: no cover
            log(f"sustained loop: graph capture failed ({e}); launching eagerly")
        def run():
            for _ in range(unit_steps):
                step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dist.barrier()
    a.record()
    for _ in range(n_units):
        run()
    b.record()
    dist.barrier()
    ms = dist.max(a.elapsed_time(b)) / (n_units * unit_steps)
    return ms, n_units * unit_steps


def run_decode(args, dist, name, with_e2e=True, with_cpu=True):
    import torch
    from nimllm_b200 import attention as A
    from nimllm_b200 import _lib
    torch.manual_seed(0)
    w = decode_workload(name, dist.rank, dist.world)
    B, Hq, Hkv, D, cap = w["B"], w["Hq"], w["Hkv"], w["D"], w["cap"]
    seq_len = torch.from_numpy(w["lens"]).cuda()
    max_len = int(w["lens"].max())
    geom = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=max_len, seq_len=seq_len,
                seq_stride=Hkv * cap * D, head_stride=cap * D, scale=w["scale"], chunk_rows=args.chunk_rows)
    out = torch.empty(B, Hq * D, dtype=torch.float32, device="cuda")
    sharded = name == "c5" and dist.world > 1
    xch = None
    if sharded:
        W = D + 4
        gathered = torch.empty(dist.world, B * Hq, W, dtype=torch.float32, device="cuda")
        if args.exchange == "p2p":
            from nimllm_b200 import sharding
            try:
                xch = sharding.PeerExchange(B * Hq, D)
                merged = torch.empty(B * Hq, D, dtype=torch.float32, device="cuda")
            except Exception as e:      # e.g. no peer access between these GPUs: every rank fails alike
                log(f"peer exchange unavailable ({e}); using the NCCL all-gather")
                xch = None

    turn = [0]
    paged = None
    if args.page_rows and not sharded:
        # every replica of the cache re-stored as a pool of pages in random order + one page table
        P = args.page_rows
        n_seq_pages = cap // P
        perm = torch.randperm(B * n_seq_pages, device="cuda")
        table = torch.empty(B * n_seq_pages, dtype=torch.int32, device="cuda")
        table[perm] = torch.arange(B * n_seq_pages, dtype=torch.int32, device="cuda")   # page j of the flat order lives at table[j]
        table = table.view(B, n_seq_pages)

        def to_pages(t):
            flat = t.view(B, Hkv, n_seq_pages, P, D).permute(0, 2, 1, 3, 4).reshape(B * n_seq_pages, Hkv, P, D)
            pool = torch.empty_like(flat)
            pool[table.view(-1).long()] = flat
            return pool
        paged = [(to_pages(k_), to_pages(v_)) for k_, v_ in zip(w["kcs"], w["vcs"])]
        pgeom = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D, max_len=max_len, seq_len=seq_len, scale=w["scale"])

    def step():
        i = turn[0] = (turn[0] + 1) % len(w["kcs"])
        if paged is not None:
            A.decode_paged(w["q"], paged[i][0], paged[i][1], table, out=out, **pgeom)
        elif not sharded:
            A.decode_batch(w["q"], w["kcs"][i], w["vcs"][i], out=out, **geom)
        elif xch is not None:
            # records go straight into every peer's buffer (NVLink stores + flags), then a bounded
            # wait and the merge: no collective library on the data path
            xch.decode_combine(w["q"], w["kc"], w["vc"], merged, **geom)
        else:
            _, rec = A.decode_batch(w["q"], w["kc"], w["vc"], out=out, partials=True, **geom)
            dist.dist.all_gather_into_tensor(gathered.view(-1), rec.view(-1))
            A.combine(gathered, D)

    graphed = False
    eager_step = step
    if sharded:
        # the sharded step is a few dependent launches; replaying them as one CUDA graph takes the
        # host's launch latency off the critical path
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            step = graph.replay
            graphed = True
        except Exception as e:  # pragma: no cover
            log(f"CUDA graph capture of the sharded step failed ({e}); timing eager launches")
    if not sharded and not args.eager:
        # the decode step (decode kernel + its merge launch, a programmatic dependent) replayed as a
        # CUDA graph, one graph per replica of the cache: what a serving loop does with a step whose
        # launches do not depend on host values
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(len(w["kcs"])):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graphs = []
            for _ in range(len(w["kcs"])):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    step()
                graphs.append(g)
            gturn = [0]

            def step():
                gturn[0] = (gturn[0] + 1) % len(graphs)
                graphs[gturn[0]].replay()
            graphed = True
        except Exception as e:  # pragma: no cover
            log(f"CUDA graph capture of the decode step failed ({e}); timing eager launches")
            step = eager_step
    flush = None        # inputs larger than L2 (see decode_workload); no flush kernel
    sampler = ClockSampler(dist.local)
    with sampler:
        # the K steps between one event pair (the headline), then the same K steps with an event pair each
        # (best step; their mean also holds the launch of every step, which back-to-back steps overlap)
        bracket_ms = timed_bracket(torch, step, args.steps, args.warmup, dist)
        ms = timed_steps(torch, step, args.steps, 3, flush, dist)
    # sustained: about two seconds of back-to-back steps (one rotation over the replicas per graph),
    # with its own clock record: a long loop meets the power cap, the short timed region does not
    sus_sampler = ClockSampler(dist.local)
    with sus_sampler:
        sus_ms, sus_steps = sustained_loop(torch, step, sum(ms) / len(ms), dist, seconds=args.sustain,
                                           unit_steps=1 if graphed else len(w["kcs"]), capture=not graphed) \
            if args.sustain > 0 and not sharded else (None, 0)   # (ranks that wait for each other: the timed steps say it all)
    t_local = bracket_ms / 1e3
    t_max = dist.max(t_local)
    total_bytes = dist.sum(float(w["bytes"])) if not sharded else float(w["bytes"]) * dist.world
    value = total_bytes / t_max * args.steps / 1e9
    best_ms = dist.max(min(ms))

    E, Ekv = Hq * D, Hkv * D
    e2e = None
    if with_e2e:
        # ---- end to end through the host-facing call: H2D activations, RoPE + append + decode, D2H
        # the step's activations q | k | v sit back to back in one pinned buffer: one host-to-device copy
        hin = torch.randn(B * (E + 2 * Ekv)).pin_memory()
        hout = torch.empty(B, E).pin_memory()
        din = torch.empty(B * (E + 2 * Ekv), device="cuda")
        dq, dk, dv = din[:B * E].view(B, E), din[B * E:B * (E + Ekv)].view(B, Ekv), din[B * (E + Ekv):].view(B, Ekv)
        # the new token overwrites the last attended row, so the batch keeps its lengths from step to
        # step; in c5 that is global row 131071, which only the last KV-sequence shard stores
        if name == "c5":
            cos, sin = A.rope_tables(w["rows"] * dist.world, D, 500000.0)
            seq_pos = torch.full((B,), w["rows"] * dist.world - 1, dtype=torch.int32, device="cuda")
            row0 = dist.rank * w["rows"]
        else:
            cos, sin = A.rope_tables(max_len + 1, D, 10000.0)
            seq_pos = (seq_len - 1).to(torch.int32)
            row0 = 0

        def e2e_step():
            i = turn[0] = (turn[0] + 1) % len(w["kcs"])
            kci, vci = w["kcs"][i], w["vcs"][i]
            din.copy_(hin, non_blocking=True)
            A.rope_append(dq.view(B, 1, E), dk.view(B, 1, Ekv), dv.view(B, 1, Ekv), cos, sin, n_head=Hq, n_kv_head=Hkv,
                          head_dim=D, seq_pos=seq_pos, k_cache=kci, v_cache=vci, seq_stride=Hkv * cap * D,
                          head_stride=cap * D, cache_row0=row0, max_seq=cap)
            if not sharded:
                A.decode_batch(dq, kci, vci, out=out, **geom)
                hout.copy_(out, non_blocking=True)
            elif xch is not None:
                hout.copy_(xch.decode_combine(dq, w["kc"], w["vc"], merged, **geom).view(B, E), non_blocking=True)
            else:
                _, rec = A.decode_batch(dq, w["kc"], w["vc"], out=out, partials=True, **geom)
                dist.dist.all_gather_into_tensor(gathered.view(-1), rec.view(-1))
                hout.copy_(A.combine(gathered, D).view(B, E), non_blocking=True)

        e2e_ms = timed_steps(torch, e2e_step, args.steps, args.warmup, flush, dist)
        e2e_t = dist.max(sum(e2e_ms) / 1e3)
        e2e = {"value": round(total_bytes / e2e_t * args.steps / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": B * (E + 2 * Ekv) * 4, "d2h_bytes_per_step": B * E * 4,
               "ms_per_step": round(e2e_t / args.steps * 1e3, 5)}
        # restore nothing: the overwritten rows stay valid bf16 data

    pk = peaks()
    needs_merge = lib_needs_combine(_lib, B, Hq, Hkv, D, max_len, args.chunk_rows)
    launches_per_step = 1 + (1 if needs_merge else 0) + (1 if sharded else 0)
    per_rank_ms = bracket_ms / args.steps
    achieved = float(w["bytes"]) / (per_rank_ms / 1e3) / 1e9
    if sharded:
        parallelism = ("kv-sequence shards, (o,m,l) records stored into the peers' buffers over NVLink by the local merge "
                       "kernel + flags + merge" if xch is not None else
                       "kv-sequence shards + NCCL all-gather of (o,m,l) + merge") + \
                      (", step replayed as a CUDA graph" if graphed else "")
    elif name == "c3p":
        parallelism = f"one batch of 256 sequences split over {dist.world} GPU(s) by greedy longest-first on KV rows, no collective"
    else:
        parallelism = f"independent sequences x{dist.world}, no collective"
    if graphed and not sharded:
        parallelism += "; step replayed as a CUDA graph"
    n_tokens = {"c3": B * dist.world, "c3p": 256, "c5": B}[name]
    line = {
        "metric": "decode_attn_kv_gbps", "value": round(value, 2), "unit": "GB/s", "n_gpus": dist.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(t_max / args.steps * 1e3, 5),
        "ms_best_step": round(best_ms, 5), "ms_per_step_own_events": round(dist.max(sum(ms) / len(ms)), 5),
        "timing": "value and ms_per_step: the K steps back to back between one CUDA-event pair on the launching stream "
                  "(barrier + synchronize on both sides, max over ranks); ms_per_step_own_events / ms_best_step: the same K "
                  "steps with an event pair around each",
        "higher_is_better": True, "scaling": "weak" if name == "c3" else "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT[name],
                   "batch_per_gpu": B, "kv_rows_total": int(w["lens"].astype(np.int64).sum()),
                   "parallelism": parallelism,
                   "l2": (f"inputs larger than L2: the timed loop rotates over {w['copies']} replicas of this GPU's batch"
                          if name != "c5" else "inputs larger than L2: 4.3 GB (or its shard) streamed once per step") +
                         "; no flush kernel (a writing flush leaves dirty lines whose write-back lands in the next step)",
                   "tokens_per_s": round(n_tokens / (t_max / args.steps), 1)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": pk["hbm"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm"], 4),
                     "traffic": NCU_TRAFFIC_BYTES[name] if dist.world == 1 else None,
                     "peak_source": pk["source"], "algorithmic_bytes_per_step": int(w["bytes"]),
                     "kernel": "decode_mma_balanced_kernel + its merge launch per step (this GPU's share), CUDA events on "
                               "the launching stream; traffic = dram bytes of the decode kernel from one ncu capture of this workload on one GPU"},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": sampler.summary(),
    }
    if sus_ms is not None:
        line["sustained"] = {"ms_per_step": round(sus_ms, 5), "steps": sus_steps,
                             "value": round(total_bytes / (sus_ms / 1e3) / 1e9, 2), "unit": "GB/s",
                             "frac": round(float(w["bytes"]) / (sus_ms / 1e3) / 1e9 / pk["hbm"], 4),
                             "how": "back-to-back graph-replayed steps for about two seconds, one event pair",
                             "clocks": sus_sampler.summary()}
    if e2e is not None:
        line["e2e"] = e2e
    if paged is not None:
        line["config"]["kv_layout"] = f"pages of {args.page_rows} rows in random order (nimllm_attn_decode_paged); e2e leg uses the contiguous cache"
    if xch is not None:
        line["config"]["peer_exchange_ok"] = xch.ok()
        dist.barrier()
        xch.close()
    if with_cpu and dist.rank == 0 and dist.world == 1:
        line["cpu_baseline"] = cpu_baseline_decode(w, reps=3)
    return line


# ------------------------------------------------------------------------------------ c4
def run_prefill(args, dist, with_e2e=True, with_cpu=True):
    """C4: causal prefill 4 x 8192, 32 q / 8 kv heads, D = 128, bf16, RoPE base 500000.  The
    KV heads (with their query heads) are split over the ranks; no collective."""
    import torch
    from nimllm_b200 import attention as A
    B, S, Hq, Hkv, D = 4, 8192, 32, 8, 128
    if SHAPE_OVERRIDE:                                  # --shape B,S,Hq,Hkv[,D]: small case for ncu captures
        B, S, Hq, Hkv = SHAPE_OVERRIDE[:4]
        if len(SHAPE_OVERRIDE) > 4:
            D = SHAPE_OVERRIDE[4]
    if Hkv % dist.world:
        raise SystemExit("c4 splits 8 KV heads: --gpus must divide 8")
    hq, hkv = Hq // dist.world, Hkv // dist.world
    gen = torch.Generator(device="cuda").manual_seed(SEEDS["c4"] + 1000 * dist.rank)
    q = torch.randn(B, S, hq * D, generator=gen, device="cuda").bfloat16()
    k = torch.randn(B, S, hkv * D, generator=gen, device="cuda").bfloat16()
    v = torch.randn(B, S, hkv * D, generator=gen, device="cuda").bfloat16()
    cos, sin = A.rope_tables(S, D, 500000.0)
    scale = 1.0 / math.sqrt(D)
    flops_rank = 4.0 * B * hq * D * S * (S + 1) / 2
    box = {}

    def step():
        # RoPE(K) pre-pass in place + tensor-core kernel with RoPE(Q) fused into its prologue
        box["out"] = A.attn_forward(q, k, v, cos, sin, n_head=hq, n_kv_head=hkv, head_dim=D, save_cache=False,
                                    scale=scale)

    flush = None        # q, k, v, out are 0.8 GB per step, 6x the L2; no flush kernel
    sampler = ClockSampler(dist.local)
    with sampler:
        ms = timed_steps(torch, step, args.steps, args.warmup, flush, dist)
    sus_sampler = ClockSampler(dist.local)      # the long loop meets the power cap: its own clock record
    with sus_sampler:
        sus_ms, sus_steps = sustained_loop(torch, step, sum(ms) / len(ms), dist, seconds=args.sustain, capture=False) \
            if args.sustain > 0 else (None, 0)
    t_max = dist.max(sum(ms) / 1e3)
    best_ms = dist.max(min(ms))
    value = flops_rank * dist.world * args.steps / t_max / 1e12
    pk = peaks()
    achieved = flops_rank / (sum(ms) / len(ms) / 1e3) / 1e12
    full = (B, S, Hq, Hkv, D) == (4, 8192, 32, 8, 128)
    line = {
        "metric": "prefill_attn_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": dist.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(t_max / args.steps * 1e3, 4),
        "ms_best_step": round(best_ms, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"C4 causal prefill: {B} x {S} tokens, {Hq}q/{Hkv}kv heads, D={D}, bf16, RoPE base 500000",
                   "parallelism": f"KV heads split over {dist.world} GPU(s), no collective",
                   "l2": "inputs larger than L2 (0.8 GB of q, k, v, out per step); no flush kernel",
                   "tokens_per_s": round(B * S / (t_max / args.steps), 1)},
        "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": pk["bf16"], "unit": "TFLOP/s",
                     "frac": round(achieved / pk["bf16"], 4), "frac_of_sustained": round(achieved / pk["bf16_sustained"], 4),
                     "traffic": NCU_TRAFFIC_BYTES["c4"] if (full and dist.world == 1) else None, "peak_source": pk["source"],
                     "algorithmic_flops_per_step": flops_rank,
                     "kernel": "prefill_tc_kernel (+ rope_append_kernel pre-pass on K) per step, CUDA events on the launching "
                               "stream; traffic = dram bytes of the prefill kernel from one ncu launch list of this workload"},
        "gpu_launches": 2 * args.steps,
        "clocks": sampler.summary(),
    }
    if sus_ms is not None:
        line["sustained"] = {"ms_per_step": round(sus_ms, 4), "steps": sus_steps,
                             "value": round(flops_rank * dist.world / (sus_ms / 1e3) / 1e12, 2), "unit": "TFLOP/s",
                             "frac_of_sustained_peak": round(flops_rank / (sus_ms / 1e3) / 1e12 / pk["bf16_sustained"], 4),
                             "how": "back-to-back steps for about two seconds, one event pair", "clocks": sus_sampler.summary()}
    if with_e2e:
        # end to end: pinned host q/k/v -> device, attention, result back to pinned host
        hq_, hk_, hv_ = (torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (q, k, v))
        hq_.copy_(q); hk_.copy_(k); hv_.copy_(v)
        hout = torch.empty(q.shape, dtype=q.dtype).pin_memory()

        def e2e_step():
            q.copy_(hq_, non_blocking=True); k.copy_(hk_, non_blocking=True); v.copy_(hv_, non_blocking=True)
            out = A.attn_forward(q, k, v, cos, sin, n_head=hq, n_kv_head=hkv, head_dim=D, save_cache=False, scale=scale)
            hout.copy_(out, non_blocking=True)

        e_steps = max(3, min(args.steps, 5))
        e2e_ms = timed_steps(torch, e2e_step, e_steps, 3, flush, dist)
        e2e_t = dist.max(sum(e2e_ms) / 1e3)
        line["e2e"] = {"value": round(flops_rank * dist.world * e_steps / e2e_t / 1e12, 2), "unit": "TFLOP/s",
                       "h2d_bytes_per_step": (q.numel() + k.numel() + v.numel()) * 2, "d2h_bytes_per_step": q.numel() * 2,
                       "ms_per_step": round(e2e_t / e_steps * 1e3, 4), "steps": e_steps}
    if with_cpu and dist.rank == 0 and dist.world == 1 and S >= 4096 and hq >= 8 and D == 128:
        line["cpu_baseline"] = cpu_baseline_prefill(q, k, v, hq, hkv, D, scale)
    return line


def run_projections(args, dist):
    """The decode step's projections either side of attention, one new token of one sequence (the
    reference's chat path, src/model.nim:775-815,843-849) through every layer of a model shaped like
    Llama-3-8B's attention (32 layers, 32 q / 8 kv heads, D = 128, n_embd 4096): per layer one fused
    q/k/v projection + RoPE + cache append and one output projection + residual.  The layers' weights
    (1.4 GB as Q8_0) are far larger than L2, so every launch streams its weights from HBM.  Every
    rank runs the same model (replicas)."""
    import torch
    from nimllm_b200 import _lib, attention as A
    layers, Hq, Hkv, D, E, cap = 32, 32, 8, 128, 4096, 64
    kind = args.wtype
    per_weight = {"f32": 4.0, "bf16": 2.0, "q8_0": 34 / 32, "q4_0": 18 / 32}[kind]
    wt = {"f32": _lib.W_F32, "bf16": _lib.W_BF16, "q8_0": _lib.W_Q8_0, "q4_0": _lib.W_Q4_0}[kind]
    gen = torch.Generator(device="cuda").manual_seed(SEEDS["c3"] + 77 + 1000 * dist.rank)

    def weights(rows, cols):
        if kind == "f32":
            return torch.randn(rows, cols, generator=gen, device="cuda") * 0.02
        if kind == "bf16":
            return (torch.randn(rows, cols, generator=gen, device="cuda") * 0.02).bfloat16()
        bs = 34 if kind == "q8_0" else 18
        t = torch.randint(0, 256, (rows * cols // 32, bs), generator=gen, dtype=torch.uint8, device="cuda")
        t[:, 1] = 0x20                 # high byte of the fp16 block scale: small, positive, finite
        return t.reshape(-1)

    W = [(weights(Hq * D, E), weights(Hkv * D, E), weights(Hkv * D, E), weights(E, Hq * D)) for _ in range(layers)]
    x = torch.randn(1, E, generator=gen, device="cuda")
    kc = torch.zeros(layers, 1, Hkv, cap, D, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    cos, sin = A.rope_tables(cap, D, 500000.0)
    box = {}

    def step():
        h = x
        for l, (wq, wk, wv, wo) in enumerate(W):
            q = A.qkv_rope_append(h, wq, wk, wv, cos, sin, n_head=Hq, n_kv_head=Hkv, head_dim=D, w_type=wt, pos0=3,
                                  k_cache=kc[l], v_cache=vc[l], seq_stride=Hkv * cap * D, head_stride=cap * D, max_seq=cap)
            h = A.wo_residual(q, wo, h, w_type=wt)      # (q stands in for the attention output: same shape)
        box["h"] = h

    # replayed as one CUDA graph, the way a whole-token step is replayed
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    sampler = ClockSampler(dist.local)
    with sampler:
        bracket_ms = timed_bracket(torch, graph.replay, args.steps, args.warmup, dist)     # K steps between one event pair
    ms = [bracket_ms / args.steps]
    t_max = dist.max(bracket_ms / 1e3)
    weights_per_layer = (Hq + 2 * Hkv) * D * E + E * Hq * D
    bytes_step = layers * weights_per_layer * per_weight
    pk = peaks()
    achieved = bytes_step / (sum(ms) / len(ms) / 1e3) / 1e9
    return {
        "metric": "decode_projection_weight_gbps", "value": round(bytes_step * dist.world * args.steps / t_max / 1e9, 1),
        "unit": "GB/s", "n_gpus": dist.world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(t_max / args.steps * 1e3, 4), "us_per_layer": round(t_max / args.steps / layers * 1e6, 2),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": kind, "data": "synthetic",
        "config": {"workload": f"decode projections, 1 token of 1 sequence: {layers} layers x (q/k/v projection + RoPE + append, "
                               f"output projection + residual), {Hq}q/{Hkv}kv heads, D={D}, n_embd {E}, {kind} weights",
                   "parallelism": f"{dist.world} replica(s)", "l2": f"{bytes_step / 1e6:.0f} MB of weights per step, larger than L2; no flush kernel",
                   "launch": "one CUDA graph of 64 kernel nodes per step"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm"], 4), "traffic": NCU_TRAFFIC_BYTES.get("proj_" + kind),
                     "peak_source": pk["source"], "algorithmic_bytes_per_step": bytes_step,
                     "kernel": "qkv_rope_append_kernel + matvec_kernel per layer; weight bytes / CUDA-event time of the whole step"},
        "gpu_launches": 2 * layers * args.steps,
        "clocks": sampler.summary(),
    }


def cpu_baseline_prefill(q, k, v, Hq, Hkv, D, scale):
    """The CPU restatement of forward()'s per-head attention loop (oracle_attn_forward: fp32,
    S x S scores per head, OpenMP over heads) on a sample of the workload's (batch, head) pairs."""
    from oracle import oracle as O
    O.lib().oracle_set_threads(os.cpu_count() or 1)
    heads_q, heads_kv, S = 8, 2, 4096          # 8 query heads over 2 KV heads of sequence 0, first 4096 tokens
    qs = q[0, :S, :heads_q * D].float().cpu().numpy().copy()
    ks = k[0, :S, :heads_kv * D].float().cpu().numpy().copy()
    vs = v[0, :S, :heads_kv * D].float().cpu().numpy().copy()
    cos, sin = O.rope_tables(S, D, 500000.0)
    t0 = time.perf_counter()
    O.attn_forward(qs, ks, vs, cos, sin, heads_q, heads_kv, D)
    dt = time.perf_counter() - t0
    flops = 4.0 * heads_q * D * S * (S + 1) / 2
    return {"value": round(flops / dt / 1e12, 5), "unit": "TFLOP/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{heads_q} query heads x first {S} tokens of sequence 0 (fp32 restatement, S x S scores per head); "
                      f"{dt:.2f} s", "host_cpus": os.cpu_count()}


def lib_needs_combine(_lib, B, Hq, Hkv, D, max_len, chunk_rows):
    return _lib.lib().nimllm_attn_decode_workspace_bytes(B, Hq, Hkv, D, max_len, chunk_rows) > 0


def cpu_baseline_decode(w, reps=3, max_seqs=None):
    """The CPU restatement of the reference's per-head decode loop (oracle/attn_oracle.c,
    fp32 arithmetic, OpenMP over sequence x head) on the same batch, all host threads."""
    from oracle import oracle as O
    import torch
    O.lib().oracle_set_threads(os.cpu_count() or 1)
    B, Hq, Hkv, D, cap = w["B"], w["Hq"], w["Hkv"], w["D"], w["cap"]
    n = B if max_seqs is None else min(B, max_seqs)
    kb = w["kc"][:n].cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    vb = w["vc"][:n].cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    q = w["q"][:n].float().cpu().numpy()
    off = np.arange(n, dtype=np.int64) * Hkv * cap * D
    hs = np.full(n, cap * D, np.int64)
    lens = w["lens"][:n]
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        O.decode_batch(q, kb, vb, off, hs, lens, Hq, Hkv, D, w["scale"])
        best = min(best, time.perf_counter() - t0)
    nbytes = int(lens.astype(np.int64).sum()) * 2 * Hkv * D * 2 + n * Hq * D * 6
    return {"value": round(nbytes / best / 1e9, 3), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
            "sample": f"{n} of {B} sequences, 1 step, best of {reps}; {best * 1e3:.1f} ms",
            "host_cpus": os.cpu_count()}


def run_reference_decode(args, dist, name):
    """Reference arm: the CPU restatement on the host cores (and, as extra information, the
    reference's own GPU launch sequence from oracle/_ref on an fp32 copy of a sample)."""
    import torch
    from oracle import oracle as O
    O.lib().oracle_set_threads(os.cpu_count() or 1)      # torchrun exports OMP_NUM_THREADS=1
    if name != "c3":
        return {"impl": "reference", "unavailable": "reference arm is implemented for the c3 workload (the headline)"}
    w = decode_workload(name, 0, 1, "cuda" if torch.cuda.is_available() else "cpu")
    B, Hq, Hkv, D, cap = w["B"], w["Hq"], w["Hkv"], w["D"], w["cap"]
    kb = w["kc"].cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    vb = w["vc"].cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    q = w["q"].float().cpu().numpy()
    off = np.arange(B, dtype=np.int64) * Hkv * cap * D
    hs = np.full(B, cap * D, np.int64)
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        O.decode_batch(q, kb, vb, off, hs, w["lens"], Hq, Hkv, D, w["scale"])
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
    t = sum(times)
    value = w["bytes"] * args.steps / t / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_kv_gbps", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": dist.world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(t / args.steps * 1e3, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT["c3"],
                   "note": "the reference has no CPU forward; this is the C restatement of its attention loop "
                           "(src/model.nim:822-840) with OpenMP over sequence x head; the numerator is the "
                           "workload's algorithmic bytes (bf16 KV), so ratios of values are ratios of speed"},
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": O.num_threads(), "kind": "port",
                         "sample": f"full batch of {B} sequences per step"},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if O.ref_available() and torch.cuda.is_available():
        try:
            n = 32                                 # sample of sequences for the reference's GPU launch loop
            kf = w["kc"][:n].float().contiguous(); vf = w["vc"][:n].float().contiguous()
            qf = w["q"][:n].float().contiguous()
            o = torch.zeros(n, Hq * D, device="cuda"); scr = torch.zeros(2 * cap, device="cuda")
            R = O.ref_lib()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            best = float("inf")
            for _ in range(3):
                torch.cuda.synchronize(); a.record()
                R.ref_decode_batch_dev(qf.data_ptr(), kf.data_ptr(), vf.data_ptr(), off[:n].copy(), hs[:n].copy(),
                                       w["lens"][:n].copy(), o.data_ptr(), scr.data_ptr(), n, Hq, Hkv, D, cap)
                b.record(); torch.cuda.synchronize()
                best = min(best, a.elapsed_time(b))
            nb = int(w["lens"][:n].astype(np.int64).sum()) * 2 * Hkv * D * 2 + n * Hq * D * 6
            line["reference_gpu_path"] = {
                "what": "the reference's compiled kernels + cublasSgemm_v2, 4 launches per query head "
                        "(src/model.nim:822-840), fp32 KV, same B200",
                "sample": f"{n} of {B} sequences", "ms": round(best, 3), "launches": n * Hq * 4,
                "value": round(nb / (best / 1e3) / 1e9, 2), "unit": "GB/s (bf16-equivalent algorithmic bytes)"}
        except Exception as e:  # pragma: no cover
            line["reference_gpu_path"] = {"unavailable": str(e)[:200]}
    return line


def main():
    # Libraries (NCCL's version banner, for one) write to file descriptor 1; the contract is one
    # JSON line on stdout, so everything else is sent to stderr and the line goes to the saved fd.
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    sys.stdout = sys.stderr
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all", "c3", "c3p", "c5", "c4", "proj"])
    ap.add_argument("--wtype", default="q8_0", choices=["f32", "bf16", "q8_0", "q4_0"], help="--workload proj: weight format")
    ap.add_argument("--sustain", type=float, default=2.0, help="seconds of the back-to-back sustained loop per workload (0: skip)")
    ap.add_argument("--chunk-rows", type=int, default=0)
    ap.add_argument("--eager", action="store_true", help="decode workloads: launch the step's kernels eagerly instead of replaying a graph")
    ap.add_argument("--page-rows", type=int, default=0,
                    help="c3 / c5 on one GPU: store the cache in shuffled pages of this many rows and time the paged decode")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="c5 on several GPUs: how the shards' partial records meet (peer stores or NCCL all-gather)")
    ap.add_argument("--shape", default="", help="override: c5 -> B,Hq,Hkv,D,L ; c4 -> B,S,Hq,Hkv[,D] (profiling only)")
    args = ap.parse_args()
    global SHAPE_OVERRIDE
    if args.shape:
        SHAPE_OVERRIDE = [int(x) for x in args.shape.split(",")]
    if args.warmup < 3:
        args.warmup = 3

    import torch
    if args.impl == "reference":
        rank = int(os.environ.get("RANK", "0"))
        if rank != 0:
            return 0
        class _Solo:
            world, rank, local = args.gpus, 0, 0
        if torch.cuda.is_available():
            torch.cuda.set_device(0)
        args.steps = min(args.steps, 20)       # each CPU step is a full batch: bound the run
        args.warmup = min(args.warmup, 10)
        line = run_reference_decode(args, _Solo, "c3" if args.workload == "all" else args.workload)
        print(json.dumps(line), file=real_stdout, flush=True)
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention library has no CPU path")
    from nimllm_b200 import _lib, build
    if not os.path.exists(_lib.LIB_PATH) and int(os.environ.get("WORLD_SIZE", "1")) == 1:
        build.build()
    dist = Dist(args.gpus)
    solo = dist.world == 1
    if args.workload in ("c3", "c3p", "c5"):
        line = run_decode(args, dist, args.workload)
    elif args.workload == "c4":
        line = run_prefill(args, dist)
    elif args.workload == "proj":
        line = run_projections(args, dist)
    else:
        # headline: c3 exactly as `--workload c3` prints it; the other configurations of the same
        # run ride along under "also" (end-to-end legs only on one GPU; the CPU baseline only for
        # the headline)
        also = {}
        # the prefill sub-record times at most 20 steps (40 ms: the burst regime its roofline is quoted against);
        # what two seconds of back-to-back steps run at under the power cap is in its "sustained" object.  It
        # runs first, on a GPU that the other workloads' two-second loops have not heated yet.
        import copy
        c4_args = copy.copy(args)
        c4_args.steps = min(args.steps, 20)

        def sub(key, fn):
            torch.cuda.empty_cache()
            try:
                rec = fn()
            except Exception as e:      # a sub-record must never take the headline down with it
                rec = {"error": f"{type(e).__name__}: {e}"[:300]}
                log(f"also.{key} failed: {rec['error']}")
            if rec is not None:
                also[key] = rec

        sub("c4", lambda: run_prefill(c4_args, dist, with_e2e=solo, with_cpu=False) if 8 % dist.world == 0 else None)
        torch.cuda.empty_cache()
        line = run_decode(args, dist, "c3")
        sub("c5", lambda: run_decode(args, dist, "c5", with_e2e=solo, with_cpu=False))
        sub("c3_partitioned", lambda: run_decode(args, dist, "c3p", with_e2e=False, with_cpu=False))
        sub("projections", lambda: run_projections(args, dist) if solo else None)
        line["also"] = also
    if dist.rank == 0:
        print(json.dumps(line), file=real_stdout, flush=True)
    dist.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
