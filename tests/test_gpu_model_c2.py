"""Configuration C2: a 30-layer SmolLM2-135M-shaped model with random fp32 weights, prompt of
256 tokens then greedy decoding to a context of 2048, with ONLY the attention block swapped.

Everything except attention runs through the reference's own compiled kernels and cuBLAS
(oracle/_ref: embed, RMSNorm, SwiGLU, residual adds, sgemm in the reference's order).  The
reference side feeds every token through forwardCached one at a time, as its chat loop does
(src/chat.nim:93-98); the library side runs one causal prefill over the prompt (filling its
cache) and then one decode step per token.  Compared: every layer's attention output at every
position, and the argmax token stream."""
import ctypes as C

import numpy as np
import pytest
import torch

from nimllm_b200 import _lib, attention as A
from oracle import oracle as O
from util import SEED_C2, TOL_F32, rng

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built")]

N_LAYER, N_EMBD, N_HEAD, N_KV, HEAD_DIM, FFN, VOCAB = 30, 576, 9, 3, 64, 1536, 49152
PROMPT, CONTEXT = 256, 2048


def _weights():
    """initModel's shapes and scales (src/model.nim:95-135): N(0, 0.02), residual projections
    scaled by 1/sqrt(2*nLayer), norm gains 1."""
    g = torch.Generator(device="cuda").manual_seed(SEED_C2)
    std, res = 0.02, 0.02 / np.sqrt(2 * N_LAYER)
    rnd = lambda *shape, s=std: (torch.randn(*shape, generator=g, device="cuda") * s).contiguous()
    ones = lambda n: torch.ones(n, device="cuda")
    nkv = N_KV * HEAD_DIM
    keep = [rnd(VOCAB, N_EMBD), rnd(VOCAB, N_EMBD), ones(N_EMBD)]
    cos, sin = A.rope_tables(CONTEXT, HEAD_DIM, 10000.0)
    keep += [cos, sin]
    for _ in range(N_LAYER):
        keep += [rnd(N_EMBD, N_EMBD), rnd(nkv, N_EMBD), rnd(nkv, N_EMBD), rnd(N_EMBD, N_EMBD, s=res), rnd(FFN, N_EMBD),
                 rnd(FFN, N_EMBD), rnd(N_EMBD, FFN, s=res), ones(N_EMBD), ones(N_EMBD)]
    return keep


def test_c2_only_attention_swapped():
    R, L = O.ref_lib(), _lib.lib()
    keep = _weights()
    ptrs = np.array([t.data_ptr() for t in keep], np.uint64)
    m = R.ref_model_create(N_LAYER, N_EMBD, N_HEAD, N_KV, HEAD_DIM, FFN, VOCAB, CONTEXT, PROMPT, ptrs)
    assert m
    fn = lambda name: C.cast(getattr(L, name), C.c_void_p)
    R.ref_model_set_attn(m, fn("nimllm_attn_prefill"), fn("nimllm_rope_append"), fn("nimllm_attn_decode_workspace_bytes"),
                         fn("nimllm_attn_decode"))
    try:
        prompt = rng(SEED_C2, 1).integers(0, VOCAB, PROMPT).astype(np.int32)
        logits = np.zeros(VOCAB, np.float32)

        # ---- reference: token by token through forwardCached
        ref_attn = torch.zeros(CONTEXT, N_LAYER, N_EMBD, device="cuda")
        tokens = np.zeros(CONTEXT + 1, np.int32)
        tokens[:PROMPT] = prompt
        margins = np.zeros(CONTEXT)
        for t in range(CONTEXT):
            assert R.ref_model_step(m, int(tokens[t]), 0, ref_attn[t].data_ptr(), logits) == 0
            top2 = np.partition(logits, -2)[-2:]
            margins[t] = top2[1] - top2[0]
            if t + 1 >= PROMPT:
                tokens[t + 1] = int(np.argmax(logits))
        torch.cuda.synchronize()

        # ---- library, teacher-forced on the reference's stream
        pre_attn = torch.zeros(N_LAYER, PROMPT, N_EMBD, device="cuda")
        assert R.ref_model_prefill_lib(m, np.ascontiguousarray(tokens[:PROMPT]), PROMPT, pre_attn.data_ptr(), logits) == 0
        mismatches = []
        if int(np.argmax(logits)) != tokens[PROMPT]:
            mismatches.append((PROMPT - 1, margins[PROMPT - 1]))
        lib_attn = torch.zeros(CONTEXT, N_LAYER, N_EMBD, device="cuda")
        lib_attn[:PROMPT] = pre_attn.permute(1, 0, 2)
        for t in range(PROMPT, CONTEXT):
            assert R.ref_model_step(m, int(tokens[t]), 1, lib_attn[t].data_ptr(), logits) == 0
            if int(np.argmax(logits)) != tokens[t + 1]:
                mismatches.append((t, margins[t]))
        torch.cuda.synchronize()

        # every layer's attention output, prompt rows (prefill kernel) and decoded rows separately
        err = (lib_attn - ref_attn).abs().amax(dim=2) / ref_attn.abs().amax(dim=2).clamp_min(1e-30)   # [pos, layer]
        worst_prefill = float(err[:PROMPT].max()); worst_decode = float(err[PROMPT:].max())
        per_layer = err.amax(dim=0).cpu().numpy()
        print(f"C2 attention rel err: prefill rows {worst_prefill:.2e}, decode rows {worst_decode:.2e}; "
              f"worst layer {int(per_layer.argmax())}; teacher-forced argmax mismatches {len(mismatches)} of {CONTEXT - PROMPT + 1}")
        assert worst_prefill <= TOL_F32 and worst_decode <= TOL_F32
        # identical argmax; a flip is tolerated only on a near-tie of the reference's own logits
        noise = 1e-4 * float(np.abs(logits).max())
        assert all(margin <= noise for _, margin in mismatches), mismatches[:5]

        # ---- library, free running: its own greedy stream equals the reference's
        R.ref_model_reset(m)
        assert R.ref_model_prefill_lib(m, np.ascontiguousarray(tokens[:PROMPT]), PROMPT, None, logits) == 0
        tok = int(np.argmax(logits))
        stream = [tok]
        for t in range(PROMPT, CONTEXT):
            assert R.ref_model_step(m, tok, 1, None, logits) == 0
            tok = int(np.argmax(logits))
            stream.append(tok)
        ref_stream = tokens[PROMPT:CONTEXT + 1].tolist()
        if stream != ref_stream:
            first = next(i for i, (a, b) in enumerate(zip(stream, ref_stream)) if a != b)
            assert margins[PROMPT - 1 + first] <= noise, f"free-running stream diverges at step {first} on a clear margin"
    finally:
        R.ref_model_destroy(m)


def _model(R, L, context, prefill):
    keep = _weights()
    ptrs = np.array([t.data_ptr() for t in keep], np.uint64)
    m = R.ref_model_create(N_LAYER, N_EMBD, N_HEAD, N_KV, HEAD_DIM, FFN, VOCAB, context, prefill, ptrs)
    assert m
    fn = lambda name: C.cast(getattr(L, name), C.c_void_p)
    R.ref_model_set_attn(m, fn("nimllm_attn_prefill"), fn("nimllm_rope_append"), fn("nimllm_attn_decode_workspace_bytes"),
                         fn("nimllm_attn_decode"))
    R.ref_model_set_proj(m, fn("nimllm_qkv_rope_append"), fn("nimllm_wo_residual"))
    return m, keep


def test_c2_attention_and_projections_swapped():
    """The same model with the attention block AND the steps either side of it from the library
    (q/k/v projection + RoPE + append in one launch, decode, output projection + residual in one
    launch; fp32 weights): every layer's attention output within 1e-4 of the reference's token by
    token, the same argmax stream."""
    import time
    R, L = O.ref_lib(), _lib.lib()
    steps = 384
    m, keep = _model(R, L, steps, 8)
    try:
        logits = np.zeros(VOCAB, np.float32)
        tokens = np.zeros(steps + 1, np.int32)
        tokens[:32] = rng(SEED_C2, 2).integers(0, VOCAB, 32)
        ref_attn = torch.zeros(steps, N_LAYER, N_EMBD, device="cuda")
        margins = np.zeros(steps)
        t0 = time.perf_counter()
        for t in range(steps):
            assert R.ref_model_step(m, int(tokens[t]), 0, ref_attn[t].data_ptr(), logits) == 0
            top2 = np.partition(logits, -2)[-2:]
            margins[t] = top2[1] - top2[0]
            if t + 1 >= 32:
                tokens[t + 1] = int(np.argmax(logits))
        t_ref = time.perf_counter() - t0
        noise = 1e-4 * float(np.abs(logits).max())
        lib_attn = torch.zeros(steps, N_LAYER, N_EMBD, device="cuda")
        mism = []
        t0 = time.perf_counter()
        for t in range(steps):
            assert R.ref_model_step(m, int(tokens[t]), 2, lib_attn[t].data_ptr(), logits) == 0
            if t + 1 >= 32 and int(np.argmax(logits)) != tokens[t + 1]:
                mism.append((t, margins[t]))
        t_lib = time.perf_counter() - t0
        torch.cuda.synchronize()
        err = (lib_attn - ref_attn).abs().amax(dim=2) / ref_attn.abs().amax(dim=2).clamp_min(1e-30)
        print(f"attention + projections swapped: worst per-layer attention rel err {float(err.max()):.2e}; argmax mismatches "
              f"{len(mism)} of {steps - 31}; {steps / t_ref:.0f} tokens/s reference sequence, {steps / t_lib:.0f} tokens/s swapped (eager)")
        assert float(err.max()) <= TOL_F32
        assert all(margin <= noise for _, margin in mism), mism[:5]
    finally:
        R.ref_model_destroy(m)


def test_c2_whole_token_step_as_one_cuda_graph():
    """The whole single-token step (embedding to logits, 30 layers) captured once as a CUDA graph
    and replayed per token while the sequence grows: the same argmax stream and logits as the
    eager step, and tokens/s of both.  Uses the build of the reference's kernels whose default
    stream can be captured."""
    import time
    P = O.ref_pts_lib()
    if P is None or not P.ref_model_graph_available():
        pytest.skip("oracle/_ref/libnimllm_ref_pts.so not built")
    L = _lib.lib()
    steps = 256
    m, keep = _model(P, L, steps, 8)
    try:
        logits = np.zeros(VOCAB, np.float32)
        tokens = rng(SEED_C2, 3).integers(0, VOCAB, steps).astype(np.int32)
        eager = np.zeros((steps, VOCAB), np.float32)
        t0 = time.perf_counter()
        for t in range(steps):
            assert P.ref_model_step(m, int(tokens[t]), 2, None, eager[t]) == 0
        t_eager = time.perf_counter() - t0
        P.ref_model_reset(m)
        nodes = C.c_int(0)
        assert P.ref_model_step_graph(m, int(tokens[0]), logits, C.byref(nodes)) == 0       # captures
        worst, flips = float(np.abs(logits - eager[0]).max()), 0
        t0 = time.perf_counter()
        for t in range(1, steps):
            assert P.ref_model_step_graph(m, int(tokens[t]), logits, None) == 0
            worst = max(worst, float(np.abs(logits - eager[t]).max()))
            flips += int(np.argmax(logits) != np.argmax(eager[t]))
        t_graph = time.perf_counter() - t0
        print(f"whole-token graph: {nodes.value} nodes, {(steps - 1) / t_graph:.0f} tokens/s replayed vs {steps / t_eager:.0f} tokens/s eager; "
              f"max |logit difference| {worst:.2e}, argmax flips {flips}")
        assert worst <= 1e-4 * float(np.abs(eager).max()) and flips == 0
        assert _lib.lib().nimllm_attn_prefill_status(0) == 0
    finally:
        P.ref_model_destroy(m)
