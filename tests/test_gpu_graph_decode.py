"""A whole decode step -- RoPE + cache append + attention for several layers -- captured once as a
CUDA graph and replayed token after token.  Positions and lengths live in device memory and
the balanced decode kernel partitions the batch on the device, so the captured launches stay
valid while the sequences grow; every replay must match the same step launched eagerly."""
import numpy as np
import pytest
import torch

from gpu_util import host
from nimllm_b200 import attention as A
from oracle import oracle as O
from util import TOL_BF16, assert_close

pytestmark = pytest.mark.gpu


def test_decode_step_graph_replay_matches_eager_and_ground_truth():
    n_layer, B, Hq, Hkv, D, cap, steps = 3, 5, 9, 3, 64, 192, 24
    start = np.array([0, 3, 17, 64, 100], np.int32)          # ragged histories
    g = torch.Generator(device="cuda").manual_seed(4242)
    cos, sin = A.rope_tables(cap, D, 10000.0)
    geom = dict(n_head=Hq, n_kv_head=Hkv, head_dim=D)
    strides = dict(seq_stride=Hkv * cap * D, head_stride=cap * D)

    def fresh():
        kc = [torch.zeros(B, Hkv, cap, D, dtype=torch.bfloat16, device="cuda") for _ in range(n_layer)]
        vc = [torch.zeros(B, Hkv, cap, D, dtype=torch.bfloat16, device="cuda") for _ in range(n_layer)]
        return kc, vc

    # histories: the same pre-filled cache for both runs (K stored rotated, as the append would leave it)
    hist_k = torch.randn(n_layer, B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    hist_v = torch.randn(n_layer, B, Hkv, cap, D, generator=g, device="cuda").bfloat16()
    acts = torch.randn(steps, n_layer, 3, B, Hq * D, generator=g, device="cuda")     # q, k, v inputs per step and layer
    q_in = torch.empty(n_layer, B, 1, Hq * D, device="cuda")
    k_in = torch.empty(n_layer, B, 1, Hkv * D, device="cuda")
    v_in = torch.empty(n_layer, B, 1, Hkv * D, device="cuda")
    outs = torch.empty(n_layer, B, Hq * D, device="cuda")
    pos = torch.empty(B, dtype=torch.int32, device="cuda")
    lens = torch.empty(B, dtype=torch.int32, device="cuda")

    def load_inputs(s):
        q_in.copy_(acts[s, :, 0].unsqueeze(2))
        k_in.copy_(acts[s, :, 1, :, :Hkv * D].unsqueeze(2))
        v_in.copy_(acts[s, :, 2, :, :Hkv * D].unsqueeze(2))

    def step(kc, vc):
        for li in range(n_layer):
            A.rope_append(q_in[li], k_in[li], v_in[li], cos, sin, seq_pos=pos, k_cache=kc[li], v_cache=vc[li],
                          max_seq=cap, **geom, **strides)
            A.decode_batch(q_in[li].view(B, Hq * D), kc[li], vc[li], max_len=cap, seq_len=lens, out=outs[li],
                           **geom, **strides)
        pos.add_(1)
        lens.add_(1)

    def run(graphed):
        kc, vc = fresh()
        for li in range(n_layer):
            kc[li].copy_(hist_k[li]); vc[li].copy_(hist_v[li])
        pos.copy_(torch.from_numpy(start)); lens.copy_(torch.from_numpy(start + 1))
        result = []
        graph = None
        if graphed:
            load_inputs(0)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step(kc, vc)                       # warm-up outside capture (workspace arena, module load)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            for li in range(n_layer):              # undo the warm-up's effects
                kc[li].copy_(hist_k[li]); vc[li].copy_(hist_v[li])
            pos.copy_(torch.from_numpy(start)); lens.copy_(torch.from_numpy(start + 1))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step(kc, vc)
            for li in range(n_layer):              # capture does not execute, but be explicit about the state
                kc[li].copy_(hist_k[li]); vc[li].copy_(hist_v[li])
            pos.copy_(torch.from_numpy(start)); lens.copy_(torch.from_numpy(start + 1))
        for s in range(steps):
            load_inputs(s)
            if graph is not None:
                graph.replay()
            else:
                step(kc, vc)
            result.append(outs.clone())
        torch.cuda.synchronize()
        return torch.stack(result), kc, vc

    eager, kc_e, vc_e = run(False)
    replay, kc_g, vc_g = run(True)
    np.testing.assert_array_equal(host(replay), host(eager))          # same launches, same bits
    for li in range(n_layer):
        np.testing.assert_array_equal(host(kc_g[li]), host(kc_e[li]))
        np.testing.assert_array_equal(host(vc_g[li]), host(vc_e[li]))

    # ground truth of the last step, layer 0, from the final cache (fp64 accumulation on the bf16 cache)
    li, s = 0, steps - 1
    L = start + steps
    qf = host(acts[s, li, 0]).copy()
    ct, st_ = O.rope_tables(cap, D, 10000.0)
    for b in range(B):
        row = qf[b:b + 1].copy()
        O.rope_fwd(row, ct[L[b] - 1:], st_[L[b] - 1:], Hq, D)
        qf[b] = row[0]
    kb = host(kc_e[li]).reshape(-1); vb = host(vc_e[li]).reshape(-1)
    off = np.arange(B, dtype=np.int64) * Hkv * cap * D
    ref = O.decode_batch(qf, kb, vb, off, np.full(B, cap * D, np.int64), L.astype(np.int32), Hq, Hkv, D,
                         1 / np.sqrt(D), acc64=True)
    assert_close(host(eager[s, li]), ref, TOL_BF16, "graph-replayed decode step vs fp64 ground truth")
