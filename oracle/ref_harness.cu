/* ref_harness.cu -- drives the reference's OWN compiled attention kernels.
 *
 * TEST INFRASTRUCTURE ONLY (never linked into or called by the product).
 *
 * The reference's device code (src/kernels.cu) is compiled, unmodified and
 * from where it lies, into the same shared object as this file by
 * oracle/Makefile; nothing of it is copied here.  The reference's host
 * sequencing is Nim (src/model.nim, src/gpu.nim) and no Nim compiler exists on
 * this image, so the host loops are restated below in C++, calling the
 * reference's extern "C" launchers and cublasSgemm_v2 in the order, with the
 * arguments and with the gpuSgemm operand swap the Nim code uses.  Running this
 * on a GPU is therefore "the reference's attention on the same seeded inputs":
 * it pins the CPU restatement (oracle/attn_oracle.c) and is the parity target
 * for the fp32 bound.
 */
#include <cuda_runtime.h>
#include <cublas_v2.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <utility>
#include <vector>

/* the reference's launchers (src/kernels.cu, declared in src/gpu.nim:227-248,274-276) */
extern "C" {
void gpu_scale(const float *x, float s, float *y, int n);
void gpu_causal_mask(float *scores, float scale, int seq_len);
void gpu_softmax_fwd(const float *x, float *y, int rows, int cols);
void gpu_extract_head(const float *src, float *dst, int h, int seq_len, int n_embd, int head_dim);
void gpu_insert_head(const float *src, float *dst, int h, int seq_len, int n_embd, int head_dim);
void gpu_extract_kv_head(const float *src, float *dst, int qHead, int kvRepeat, int seq_len,
                         int n_kv_dim, int head_dim);
void gpu_rope_fwd(float *data, const float *cos_tab, const float *sin_tab, int seq_len,
                  int n_embd, int n_head, int head_dim);
/* backward-path launchers (src/kernels.cu:341-345,390-394,425-431,471-477,159-161) */
void gpu_softmax_bwd(const float *y, const float *dy, float *dx, int rows, int cols);
void gpu_insert_head_acc(const float *src, float *dst, int h, int seq_len, int n_embd, int head_dim);
void gpu_insert_kv_head_acc(const float *src, float *dst, int qHead, int kvRepeat, int seq_len,
                            int n_kv_dim, int head_dim);
void gpu_rope_bwd(float *grad, const float *cos_tab, const float *sin_tab, int seq_len, int n_embd,
                  int n_head, int head_dim);
void gpu_scale(const float *x, float s, float *y, int n);
/* non-attention launchers used by the whole-model harness (src/gpu.nim:219-232,282-290) */
void gpu_embed_fwd(const float *wte, const int *tokens, float *out, int seq_len, int dim);
void gpu_rmsnorm_affine_fwd(const float *x, const float *gamma, float *y, float *rms_out, int rows, int dim);
void gpu_swiglu_fwd(const float *gate, const float *up, float *out, int n);
void gpu_add(const float *a, const float *b, float *y, int n);
}

static cublasHandle_t g_cublas = nullptr;

/* The reference launches everything with <<<grid, block>>> on the default stream.  Built normally
 * that is the legacy stream; built with nvcc --default-stream per-thread (the second library
 * oracle/Makefile makes from the same sources) it is the per-thread stream, which -- unlike the legacy
 * one -- can be captured into a CUDA graph.  The harness follows whichever it was built with. */
#ifdef CUDA_API_PER_THREAD_DEFAULT_STREAM
#define REF_STREAM cudaStreamPerThread
#define REF_CAN_CAPTURE 1
#else
#define REF_STREAM ((cudaStream_t)0)
#define REF_CAN_CAPTURE 0
#endif

#define CK(x)                                                                          \
    do {                                                                               \
        cudaError_t e_ = (x);                                                          \
        if (e_ != cudaSuccess) {                                                       \
            fprintf(stderr, "ref_harness: %s -> %s\n", #x, cudaGetErrorString(e_));    \
            return -1;                                                                 \
        }                                                                              \
    } while (0)

/* src/gpu.nim:185-207 gpuSgemm: row-major GEMM through the column-major swap. */
static void ref_sgemm(int op, int m, int n, int k, const float *a, const float *b, float *c) {
    float alpha = 1.0f, beta = (op & 1) ? 1.0f : 0.0f;
    bool ta = (op & 4) != 0, tb = (op & 2) != 0;
    cublasOperation_t opB = tb ? CUBLAS_OP_T : CUBLAS_OP_N;
    cublasOperation_t opA = ta ? CUBLAS_OP_T : CUBLAS_OP_N;
    int lda = ta ? m : k, ldb = tb ? k : n, ldc = n;
    cublasSgemm_v2(g_cublas, opB, opA, n, m, k, &alpha, b, ldb, a, lda, &beta, c, ldc);
}

extern "C" {

/* src/gpu.nim:173-181 gpuInit */
int ref_init(void) {
    if (g_cublas) return 0;
    if (cublasCreate_v2(&g_cublas) != CUBLAS_STATUS_SUCCESS) return -1;
    cublasSetStream_v2(g_cublas, REF_STREAM);       /* the reference never sets one (src/gpu.nim:166-175): default stream */
    return 0;
}

/* src/model.nim:469-475,494-508 on DEVICE buffers.  q [S,E], k,v [S,Ekv],
 * tables [>=S, D/2], out [S,E]; scratch holds 4*S*D + 2*S*S floats. */
int ref_attn_forward_dev(float *q, float *k, const float *v, const float *cos_tab,
                         const float *sin_tab, float *out, float *scratch, int S, int Hq,
                         int Hkv, int D, int apply_rope) {
    int E = Hq * D, Ekv = Hkv * D, G = Hq / Hkv;
    float scale = 1.0f / sqrtf((float)D);
    float *qH = scratch, *kH = qH + (size_t)S * D, *vH = kH + (size_t)S * D,
          *aH = vH + (size_t)S * D, *scores = aH + (size_t)S * D, *probs = scores + (size_t)S * S;
    if (apply_rope) {
        gpu_rope_fwd(q, cos_tab, sin_tab, S, E, Hq, D);
        gpu_rope_fwd(k, cos_tab, sin_tab, S, Ekv, Hkv, D);
    }
    for (int h = 0; h < Hq; h++) {
        gpu_extract_head(q, qH, h, S, E, D);
        gpu_extract_kv_head(k, kH, h, G, S, Ekv, D);
        gpu_extract_kv_head(v, vH, h, G, S, Ekv, D);
        ref_sgemm(2, S, S, D, qH, kH, scores);
        gpu_causal_mask(scores, scale, S);
        gpu_softmax_fwd(scores, probs, S, S);
        ref_sgemm(0, S, D, S, probs, vH, aH);
        gpu_insert_head(aH, out, h, S, E, D);
    }
    return 0;
}

/* host-buffer wrapper of the above; q and k come back rotated. */
int ref_attn_forward(float *q, float *k, const float *v, const float *cos_tab,
                     const float *sin_tab, float *out, int S, int Hq, int Hkv, int D,
                     int apply_rope) {
    if (ref_init()) return -1;
    size_t E = (size_t)Hq * D, Ekv = (size_t)Hkv * D, half = D / 2;
    float *dq, *dk, *dv, *dc, *ds, *dout, *scr;
    CK(cudaMalloc(&dq, S * E * 4)); CK(cudaMalloc(&dk, S * Ekv * 4)); CK(cudaMalloc(&dv, S * Ekv * 4));
    CK(cudaMalloc(&dc, S * half * 4)); CK(cudaMalloc(&ds, S * half * 4));
    CK(cudaMalloc(&dout, S * E * 4));
    CK(cudaMalloc(&scr, ((size_t)4 * S * D + (size_t)2 * S * S) * 4));
    CK(cudaMemcpy(dq, q, S * E * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dk, k, S * Ekv * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv, v, S * Ekv * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dc, cos_tab, S * half * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(ds, sin_tab, S * half * 4, cudaMemcpyHostToDevice));
    CK(cudaMemset(dout, 0, S * E * 4));
    ref_attn_forward_dev(dq, dk, dv, dc, ds, dout, scr, S, Hq, Hkv, D, apply_rope);
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(q, dq, S * E * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(k, dk, S * Ekv * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(out, dout, S * E * 4, cudaMemcpyDeviceToHost));
    cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(dc); cudaFree(ds); cudaFree(dout); cudaFree(scr);
    return 0;
}

/* src/model.nim:639-685: the attention block of backward(), restated launch by launch with
 * the reference's own kernels and cublasSgemm_v2.  Host buffers: q_rot [S,E], k_rot, v [S,Ekv]
 * (as saveCache left them), d_attn_out [S,E]; dq [S,E], dk, dv [S,Ekv] come back with the
 * rotation undone on dq and dk. */
int ref_attn_backward(const float *q_rot, const float *k_rot, const float *v, const float *d_attn_out,
                      const float *cos_tab, const float *sin_tab, float *dq_h, float *dk_h, float *dv_h,
                      int S, int Hq, int Hkv, int D) {
    if (ref_init()) return -1;
    size_t E = (size_t)Hq * D, Ekv = (size_t)Hkv * D, half = D / 2;
    int G = Hq / Hkv;
    float scale = 1.0f / sqrtf((float)D);
    float *q, *k, *vv, *dout, *dc, *ds, *dq, *dk, *dv, *scr;
    CK(cudaMalloc(&q, S * E * 4)); CK(cudaMalloc(&k, S * Ekv * 4)); CK(cudaMalloc(&vv, S * Ekv * 4));
    CK(cudaMalloc(&dout, S * E * 4));
    CK(cudaMalloc(&dc, S * half * 4)); CK(cudaMalloc(&ds, S * half * 4));
    CK(cudaMalloc(&dq, S * E * 4)); CK(cudaMalloc(&dk, S * Ekv * 4)); CK(cudaMalloc(&dv, S * Ekv * 4));
    CK(cudaMalloc(&scr, ((size_t)7 * S * D + (size_t)4 * S * S) * 4));
    CK(cudaMemcpy(q, q_rot, S * E * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(k, k_rot, S * Ekv * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(vv, v, S * Ekv * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dout, d_attn_out, S * E * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dc, cos_tab, S * half * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(ds, sin_tab, S * half * 4, cudaMemcpyHostToDevice));
    /* trackedCreate hands out zeroed memory (src/autograd.nim:37-51) */
    CK(cudaMemset(dq, 0, S * E * 4)); CK(cudaMemset(dk, 0, S * Ekv * 4)); CK(cudaMemset(dv, 0, S * Ekv * 4));
    float *doutH = scr, *qH = doutH + (size_t)S * D, *kH = qH + (size_t)S * D, *vH = kH + (size_t)S * D,
          *dqH = vH + (size_t)S * D, *dkH = dqH + (size_t)S * D, *dvH = dkH + (size_t)S * D,
          *scores = dvH + (size_t)S * D, *probs = scores + (size_t)S * S, *dW = probs + (size_t)S * S,
          *dScores = dW + (size_t)S * S;
    for (int h = 0; h < Hq; h++) {
        gpu_extract_head(dout, doutH, h, S, (int)E, D);
        gpu_extract_head(q, qH, h, S, (int)E, D);
        gpu_extract_kv_head(k, kH, h, G, S, (int)Ekv, D);
        gpu_extract_kv_head(vv, vH, h, G, S, (int)Ekv, D);
        ref_sgemm(2, S, S, D, qH, kH, scores);
        gpu_causal_mask(scores, scale, S);
        gpu_softmax_fwd(scores, probs, S, S);
        ref_sgemm(2, S, S, D, doutH, vH, dW);
        ref_sgemm(4, S, D, S, probs, doutH, dvH);
        CK(cudaMemset(dScores, 0, (size_t)S * S * 4));
        gpu_softmax_bwd(probs, dW, dScores, S, S);
        gpu_scale(dScores, scale, dScores, S * S);
        ref_sgemm(0, S, D, S, dScores, kH, dqH);
        ref_sgemm(4, S, D, S, dScores, qH, dkH);
        gpu_insert_head_acc(dqH, dq, h, S, (int)E, D);
        gpu_insert_kv_head_acc(dkH, dk, h, G, S, (int)Ekv, D);
        gpu_insert_kv_head_acc(dvH, dv, h, G, S, (int)Ekv, D);
    }
    gpu_rope_bwd(dq, dc, ds, S, (int)E, Hq, D);
    gpu_rope_bwd(dk, dc, ds, S, (int)Ekv, Hkv, D);
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(dq_h, dq, S * E * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dk_h, dk, S * Ekv * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dv_h, dv, S * Ekv * 4, cudaMemcpyDeviceToHost));
    cudaFree(q); cudaFree(k); cudaFree(vv); cudaFree(dout); cudaFree(dc); cudaFree(ds);
    cudaFree(dq); cudaFree(dk); cudaFree(dv); cudaFree(scr);
    return 0;
}

/* src/model.nim:70-73,729-746: one layer's KvCache -- Hkv separately allocated,
 * zero-filled [max_seq, D] fp32 buffers for K and for V, plus the host pos. */
struct RefKv {
    std::vector<float *> k, v;
    int pos, Hkv, D, max_seq;
    float *cos_tab, *sin_tab;   /* device tables [max_seq, D/2] */
    float *scores, *probs, *q, *knew, *vnew, *out;
};

void *ref_kvcache_create(int Hkv, int D, int max_seq, int Hq, const float *cos_tab,
                         const float *sin_tab) {
    if (ref_init()) return nullptr;
    RefKv *kv = new RefKv();
    kv->pos = 0; kv->Hkv = Hkv; kv->D = D; kv->max_seq = max_seq;
    for (int h = 0; h < Hkv; h++) {
        float *a, *b;
        cudaMalloc(&a, (size_t)max_seq * D * 4); cudaMemset(a, 0, (size_t)max_seq * D * 4);
        cudaMalloc(&b, (size_t)max_seq * D * 4); cudaMemset(b, 0, (size_t)max_seq * D * 4);
        kv->k.push_back(a); kv->v.push_back(b);
    }
    size_t tab = (size_t)max_seq * (D / 2) * 4;
    cudaMalloc(&kv->cos_tab, tab); cudaMalloc(&kv->sin_tab, tab);
    cudaMemcpy(kv->cos_tab, cos_tab, tab, cudaMemcpyHostToDevice);
    cudaMemcpy(kv->sin_tab, sin_tab, tab, cudaMemcpyHostToDevice);
    cudaMalloc(&kv->scores, (size_t)max_seq * 4); cudaMalloc(&kv->probs, (size_t)max_seq * 4);
    cudaMalloc(&kv->q, (size_t)Hq * D * 4); cudaMalloc(&kv->out, (size_t)Hq * D * 4);
    cudaMalloc(&kv->knew, (size_t)Hkv * D * 4); cudaMalloc(&kv->vnew, (size_t)Hkv * D * 4);
    return kv;
}

void ref_kvcache_reset(void *h) {
    RefKv *kv = (RefKv *)h;
    for (int i = 0; i < kv->Hkv; i++) {
        cudaMemset(kv->k[i], 0, (size_t)kv->max_seq * kv->D * 4);
        cudaMemset(kv->v[i], 0, (size_t)kv->max_seq * kv->D * 4);
    }
    kv->pos = 0;
}

void ref_kvcache_destroy(void *h) {
    RefKv *kv = (RefKv *)h;
    for (int i = 0; i < kv->Hkv; i++) { cudaFree(kv->k[i]); cudaFree(kv->v[i]); }
    cudaFree(kv->cos_tab); cudaFree(kv->sin_tab); cudaFree(kv->scores); cudaFree(kv->probs);
    cudaFree(kv->q); cudaFree(kv->out); cudaFree(kv->knew); cudaFree(kv->vnew);
    delete kv;
}

int ref_kvcache_pos(void *h) { return ((RefKv *)h)->pos; }

/* fills the cache rows 0..n-1 from already rotated k and raw v [n, Hkv*D]
 * (the multi-token append branch, src/model.nim:810-815) and sets pos = n. */
int ref_kvcache_fill(void *h, const float *k_rot, const float *v, int n) {
    RefKv *kv = (RefKv *)h;
    int Ekv = kv->Hkv * kv->D;
    float *dk, *dv;
    CK(cudaMalloc(&dk, (size_t)n * Ekv * 4)); CK(cudaMalloc(&dv, (size_t)n * Ekv * 4));
    CK(cudaMemcpy(dk, k_rot, (size_t)n * Ekv * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv, v, (size_t)n * Ekv * 4, cudaMemcpyHostToDevice));
    for (int kvh = 0; kvh < kv->Hkv; kvh++) {
        /* kvRepeat = 1 here, so qHead == kvHead selects the column block */
        gpu_extract_kv_head(dk, kv->k[kvh], kvh, 1, n, Ekv, kv->D);
        gpu_extract_kv_head(dv, kv->v[kvh], kvh, 1, n, Ekv, kv->D);
    }
    CK(cudaDeviceSynchronize());
    cudaFree(dk); cudaFree(dv);
    kv->pos = n;
    return 0;
}

/* src/model.nim:788-840 with newTokens == 1.  Host q [Hq*D], k_new, v_new
 * [Hkv*D]; out [Hq*D]; advances pos (src/model.nim:890). */
int ref_attn_forward_cached(void *h, const float *q, const float *k_new, const float *v_new,
                            float *out, int Hq) {
    RefKv *kv = (RefKv *)h;
    int D = kv->D, Hkv = kv->Hkv, E = Hq * D, Ekv = Hkv * D, G = Hq / Hkv, half = D / 2;
    int S = kv->pos + 1;
    if (S > kv->max_seq) return -2;
    float scale = 1.0f / sqrtf((float)D);
    CK(cudaMemcpy(kv->q, q, (size_t)E * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(kv->knew, k_new, (size_t)Ekv * 4, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(kv->vnew, v_new, (size_t)Ekv * 4, cudaMemcpyHostToDevice));
    const float *cosp = kv->cos_tab + (size_t)kv->pos * half;
    const float *sinp = kv->sin_tab + (size_t)kv->pos * half;
    gpu_rope_fwd(kv->q, cosp, sinp, 1, E, Hq, D);
    gpu_rope_fwd(kv->knew, cosp, sinp, 1, Ekv, Hkv, D);
    for (int kvh = 0; kvh < Hkv; kvh++) {
        CK(cudaMemcpy(kv->k[kvh] + (size_t)kv->pos * D, kv->knew + (size_t)kvh * D, (size_t)D * 4,
                      cudaMemcpyDeviceToDevice));
        CK(cudaMemcpy(kv->v[kvh] + (size_t)kv->pos * D, kv->vnew + (size_t)kvh * D, (size_t)D * 4,
                      cudaMemcpyDeviceToDevice));
    }
    for (int hq = 0; hq < Hq; hq++) {
        int kvh = hq / G;
        ref_sgemm(2, 1, S, D, kv->q + (size_t)hq * D, kv->k[kvh], kv->scores);
        gpu_scale(kv->scores, scale, kv->scores, S);
        gpu_softmax_fwd(kv->scores, kv->probs, 1, S);
        ref_sgemm(0, 1, D, S, kv->probs, kv->v[kvh], kv->out + (size_t)hq * D);
    }
    kv->pos += 1;
    CK(cudaMemcpy(out, kv->out, (size_t)E * 4, cudaMemcpyDeviceToHost));
    return 0;
}

/* cache contents as [Hkv, max_seq, D] host arrays */
int ref_kvcache_download(void *h, float *k, float *v) {
    RefKv *kv = (RefKv *)h;
    size_t n = (size_t)kv->max_seq * kv->D;
    for (int i = 0; i < kv->Hkv; i++) {
        CK(cudaMemcpy(k + i * n, kv->k[i], n * 4, cudaMemcpyDeviceToHost));
        CK(cudaMemcpy(v + i * n, kv->v[i], n * 4, cudaMemcpyDeviceToHost));
    }
    return 0;
}

/* The read half of src/model.nim:822-840 over a batch of independent sequences
 * held in DEVICE fp32 buffers, for timing the reference's launch sequence on a
 * batched workload it was never given: per sequence, per query head, the four
 * launches (sgemm, scale, softmax, sgemm).  kv_off / head_stride / seq_len are
 * HOST arrays; scratch holds 2*max_len floats. */
int ref_decode_batch_dev(const float *q, const float *k, const float *v, const int64_t *kv_off,
                         const int64_t *head_stride, const int32_t *seq_len, float *out,
                         float *scratch, int B, int Hq, int Hkv, int D, int max_len) {
    if (ref_init()) return -1;
    int G = Hq / Hkv, E = Hq * D;
    float scale = 1.0f / sqrtf((float)D);
    float *scores = scratch, *probs = scratch + max_len;
    for (int b = 0; b < B; b++)
        for (int h = 0; h < Hq; h++) {
            int S = seq_len[b], kvh = h / G;
            const float *kH = k + kv_off[b] + (int64_t)kvh * head_stride[b];
            const float *vH = v + kv_off[b] + (int64_t)kvh * head_stride[b];
            ref_sgemm(2, 1, S, D, q + (size_t)b * E + (size_t)h * D, kH, scores);
            gpu_scale(scores, scale, scores, S);
            gpu_softmax_fwd(scores, probs, 1, S);
            ref_sgemm(0, 1, D, S, probs, vH, out + (size_t)b * E + (size_t)h * D);
        }
    return 0;
}


/* ===================================================================================
 * Whole-model harness for the "only attention is swapped" configuration: the reference's
 * forward passes (src/model.nim:454-549 forward, :748-895 forwardCached, float32 branch)
 * restated around the reference's own non-attention kernels and cuBLAS, with the attention
 * block either the reference's per-head loop (impl 0) or calls into the library under test
 * through function pointers (impl 1).  Weights and RoPE tables are DEVICE buffers owned by the
 * caller.  Test infrastructure only.
 * =================================================================================== */
typedef int (*PrefillFn)(void *, void *, const void *, int, const float *, const float *, int, void *, int, int, int,
                         int, int, float, int, void *, void *, int, const int64_t *, int64_t, int64_t, int, float *,
                         void *, size_t, void *);
typedef int (*RopeAppendFn)(void *, int, void *, const void *, int, int, const float *, const float *, const int32_t *,
                            int, void *, void *, int, const int64_t *, int64_t, int64_t, int, int, int, int, int, int,
                            void *);
typedef size_t (*DecodeWsFn)(int, int, int, int, int, int);
typedef int (*DecodeFn)(const void *, int, const void *, const void *, int, const int64_t *, int64_t, int64_t,
                        const int32_t *, int, void *, int, float *, int, int, int, int, float, int, void *, size_t,
                        void *);

typedef int (*QkvFn)(const float *, const void *, const void *, const void *, int, float *, float *, float *, const float *,
                     const float *, const int32_t *, int, void *, void *, int, const int64_t *, int64_t, int64_t, int, int,
                     int, int, int, int, int, void *);
typedef int (*WoFn)(const float *, const void *, int, const float *, float *, int, int, int, void *);

struct RefModel {
    int nLayer, nEmbd, nHead, nKvHead, headDim, ffnDim, vocab, maxSeq, maxPrefill;
    const float *wte, *lmHead, *lnFg, *cosTab, *sinTab;
    std::vector<const float *> wq, wk, wv, wo, gate, up, down, ln1, ln2;
    std::vector<std::vector<float *>> kc, vc; /* reference cache: [layer][kv head] -> [maxSeq, D] */
    int pos;
    float *mk, *mv;                           /* library cache: [layer][kv head][maxSeq][D] */
    int mpos;
    int *tokIds;
    float *x, *xn, *rms, *q, *k, *v, *attn, *proj, *x2, *gateo, *upo, *sw, *mlp, *xnew, *scores, *probs, *logits;
    void *ws;
    size_t wsBytes;
    PrefillFn prefill; RopeAppendFn ropeAppend; DecodeWsFn decodeWs; DecodeFn decode;
    QkvFn qkv; WoFn woResid;
    /* whole-token graph: the token id, its position and the attended length live in device memory */
    int32_t *dPos, *dLen;
    cudaGraphExec_t graphExec;
};

static float *dalloc(size_t n) {
    float *p = nullptr;
    cudaMalloc(&p, n * sizeof(float));
    cudaMemset(p, 0, n * sizeof(float));
    return p;
}

/* ptrs: wte, lmHead, lnFg, cosTab, sinTab, then per layer wq wk wv wo gate up down ln1 ln2 */
void *ref_model_create(int nLayer, int nEmbd, int nHead, int nKvHead, int headDim, int ffnDim, int vocab,
                       int maxSeq, int maxPrefill, const uint64_t *ptrs) {
    if (ref_init()) return nullptr;
    RefModel *m = new RefModel();
    m->nLayer = nLayer; m->nEmbd = nEmbd; m->nHead = nHead; m->nKvHead = nKvHead; m->headDim = headDim;
    m->ffnDim = ffnDim; m->vocab = vocab; m->maxSeq = maxSeq; m->maxPrefill = maxPrefill;
    m->wte = (const float *)ptrs[0]; m->lmHead = (const float *)ptrs[1]; m->lnFg = (const float *)ptrs[2];
    m->cosTab = (const float *)ptrs[3]; m->sinTab = (const float *)ptrs[4];
    for (int l = 0; l < nLayer; l++) {
        const uint64_t *p = ptrs + 5 + 9 * l;
        m->wq.push_back((const float *)p[0]); m->wk.push_back((const float *)p[1]); m->wv.push_back((const float *)p[2]);
        m->wo.push_back((const float *)p[3]); m->gate.push_back((const float *)p[4]); m->up.push_back((const float *)p[5]);
        m->down.push_back((const float *)p[6]); m->ln1.push_back((const float *)p[7]); m->ln2.push_back((const float *)p[8]);
        std::vector<float *> kh, vh;
        for (int h = 0; h < nKvHead; h++) {                 /* src/model.nim:729-739 */
            kh.push_back(dalloc((size_t)maxSeq * headDim));
            vh.push_back(dalloc((size_t)maxSeq * headDim));
        }
        m->kc.push_back(kh); m->vc.push_back(vh);
    }
    m->pos = 0; m->mpos = 0;
    size_t cacheN = (size_t)nLayer * nKvHead * maxSeq * headDim;
    m->mk = dalloc(cacheN); m->mv = dalloc(cacheN);
    int S = maxPrefill, n = nEmbd, nKv = nKvHead * headDim;
    cudaMalloc(&m->tokIds, S * sizeof(int));
    m->x = dalloc((size_t)S * n); m->xn = dalloc((size_t)S * n); m->rms = dalloc(S);
    m->q = dalloc((size_t)S * n); m->k = dalloc((size_t)S * nKv); m->v = dalloc((size_t)S * nKv);
    m->attn = dalloc((size_t)S * n); m->proj = dalloc((size_t)S * n); m->x2 = dalloc((size_t)S * n);
    m->gateo = dalloc((size_t)S * ffnDim); m->upo = dalloc((size_t)S * ffnDim); m->sw = dalloc((size_t)S * ffnDim);
    m->mlp = dalloc((size_t)S * n); m->xnew = dalloc((size_t)S * n);
    m->scores = dalloc(maxSeq); m->probs = dalloc(maxSeq);
    m->logits = dalloc((size_t)S * vocab);
    m->wsBytes = 16u << 20;
    cudaMalloc(&m->ws, m->wsBytes);
    m->prefill = nullptr; m->ropeAppend = nullptr; m->decodeWs = nullptr; m->decode = nullptr;
    m->qkv = nullptr; m->woResid = nullptr; m->graphExec = nullptr;
    cudaMalloc(&m->dPos, sizeof(int32_t)); cudaMalloc(&m->dLen, sizeof(int32_t));
    return m;
}

void ref_model_set_attn(void *h, void *prefill, void *ropeAppend, void *decodeWs, void *decode) {
    RefModel *m = (RefModel *)h;
    m->prefill = (PrefillFn)prefill; m->ropeAppend = (RopeAppendFn)ropeAppend;
    m->decodeWs = (DecodeWsFn)decodeWs; m->decode = (DecodeFn)decode;
}

/* the fused projection entry points of the library under test (impl 2 and the graph) */
void ref_model_set_proj(void *h, void *qkv, void *woResid) {
    RefModel *m = (RefModel *)h;
    m->qkv = (QkvFn)qkv; m->woResid = (WoFn)woResid;
}

void ref_model_reset(void *h) {                              /* src/model.nim:741-746 */
    RefModel *m = (RefModel *)h;
    size_t per = (size_t)m->maxSeq * m->headDim * sizeof(float);
    for (auto &l : m->kc) for (float *p : l) cudaMemset(p, 0, per);
    for (auto &l : m->vc) for (float *p : l) cudaMemset(p, 0, per);
    cudaMemset(m->mk, 0, per * m->nLayer * m->nKvHead);
    cudaMemset(m->mv, 0, per * m->nLayer * m->nKvHead);
    m->pos = 0; m->mpos = 0;
}

void ref_model_destroy(void *h) {
    RefModel *m = (RefModel *)h;
    for (auto &l : m->kc) for (float *p : l) cudaFree(p);
    for (auto &l : m->vc) for (float *p : l) cudaFree(p);
    float *bufs[] = {m->mk, m->mv, m->x, m->xn, m->rms, m->q, m->k, m->v, m->attn, m->proj, m->x2, m->gateo, m->upo,
                     m->sw, m->mlp, m->xnew, m->scores, m->probs, m->logits};
    for (float *p : bufs) cudaFree(p);
    cudaFree(m->tokIds); cudaFree(m->ws); cudaFree(m->dPos); cudaFree(m->dLen);
    if (m->graphExec) cudaGraphExecDestroy(m->graphExec);
    delete m;
}

/* the feed-forward half of a layer, from x2 = x + wo(attn): src/model.nim:518-532 / :851-875 */
static float *ref_layer_ffn(RefModel *m, int l, int S) {
    int n = m->nEmbd, f = m->ffnDim;
    gpu_rmsnorm_affine_fwd(m->x2, m->ln2[l], m->xn, m->rms, S, n);
    ref_sgemm(2, S, f, n, m->xn, m->gate[l], m->gateo);
    ref_sgemm(2, S, f, n, m->xn, m->up[l], m->upo);
    gpu_swiglu_fwd(m->gateo, m->upo, m->sw, S * f);
    ref_sgemm(2, S, n, f, m->sw, m->down[l], m->mlp);
    gpu_add(m->x2, m->mlp, m->xnew, S * n);
    return m->xnew;
}

/* everything of a layer after the attention block: src/model.nim:510-532 / :842-875 */
static float *ref_layer_tail(RefModel *m, int l, int S, float *x) {
    int n = m->nEmbd, f = m->ffnDim;
    ref_sgemm(2, S, n, n, m->attn, m->wo[l], m->proj);
    gpu_add(x, m->proj, m->x2, S * n);
    gpu_rmsnorm_affine_fwd(m->x2, m->ln2[l], m->xn, m->rms, S, n);
    ref_sgemm(2, S, f, n, m->xn, m->gate[l], m->gateo);
    ref_sgemm(2, S, f, n, m->xn, m->up[l], m->upo);
    gpu_swiglu_fwd(m->gateo, m->upo, m->sw, S * f);
    ref_sgemm(2, S, n, f, m->sw, m->down[l], m->mlp);
    gpu_add(m->x2, m->mlp, m->xnew, S * n);
    return m->xnew;
}

/* forwardCached with ONE new token (src/model.nim:748-895).  impl 0: the reference's attention
 * (RoPE, cudaMemcpy append, per-head sgemm/scale/softmax/sgemm); impl 1: the library under test.
 * attn_dump: device [nLayer, nEmbd] or NULL; logits_host: [vocab]. */
int ref_model_step(void *h, int token, int impl, float *attn_dump, float *logits_host) {
    RefModel *m = (RefModel *)h;
    int n = m->nEmbd, D = m->headDim, Hq = m->nHead, Hkv = m->nKvHead, nKv = Hkv * D, G = Hq / Hkv, half = D / 2;
    int &pos = impl ? m->mpos : m->pos;
    if (pos + 1 > m->maxSeq) return -2;
    int S = pos + 1;
    float scale = 1.0f / sqrtf((float)D);
    CK(cudaMemcpy(m->tokIds, &token, sizeof(int), cudaMemcpyHostToDevice));
    float *x = m->x;
    gpu_embed_fwd(m->wte, m->tokIds, x, 1, n);
    float *cur = x;
    for (int l = 0; l < m->nLayer; l++) {
        gpu_rmsnorm_affine_fwd(cur, m->ln1[l], m->xn, m->rms, 1, n);
        if (impl == 2) {
            /* attention AND the projections either side of it from the library: q/k/v projection +
             * RoPE + append in one launch, decode, output projection + residual in one launch */
            if (!m->qkv || !m->woResid) return -4;
            int64_t headStride = (int64_t)m->maxSeq * D, seqStride = headStride * Hkv;
            float *kcl = m->mk + (size_t)l * seqStride, *vcl = m->mv + (size_t)l * seqStride;
            int rc = m->qkv(m->xn, m->wq[l], m->wk[l], m->wv[l], 0, m->q, nullptr, nullptr, m->cosTab, m->sinTab, nullptr, pos,
                            kcl, vcl, 0, nullptr, seqStride, headStride, 0, m->maxSeq, 1, n, Hq, Hkv, D, REF_STREAM);
            if (rc) return 400 + rc;
            size_t need = m->decodeWs(1, Hq, Hkv, D, S, 0);
            if (need > m->wsBytes) return -3;
            rc = m->decode(m->q, 0, kcl, vcl, 0, nullptr, seqStride, headStride, nullptr, S, m->attn, 0, nullptr, 1, Hq,
                           Hkv, D, scale, 0, m->ws, need, REF_STREAM);
            if (rc) return 200 + rc;
            if (attn_dump) cudaMemcpyAsync(attn_dump + (size_t)l * n, m->attn, n * sizeof(float), cudaMemcpyDeviceToDevice, REF_STREAM);
            rc = m->woResid(m->attn, m->wo[l], 0, cur, m->x2, 1, n, n, REF_STREAM);
            if (rc) return 500 + rc;
            float *nx = ref_layer_ffn(m, l, 1);
            if (nx == m->xnew) { std::swap(m->x, m->xnew); cur = m->x; }
            continue;
        }
        ref_sgemm(2, 1, n, n, m->xn, m->wq[l], m->q);
        ref_sgemm(2, 1, nKv, n, m->xn, m->wk[l], m->k);
        ref_sgemm(2, 1, nKv, n, m->xn, m->wv[l], m->v);
        if (!impl) {
            const float *cosp = m->cosTab + (size_t)pos * half, *sinp = m->sinTab + (size_t)pos * half;
            gpu_rope_fwd(m->q, cosp, sinp, 1, n, Hq, D);
            gpu_rope_fwd(m->k, cosp, sinp, 1, nKv, Hkv, D);
            for (int kvh = 0; kvh < Hkv; kvh++) {
                cudaMemcpy(m->kc[l][kvh] + (size_t)pos * D, m->k + (size_t)kvh * D, D * sizeof(float), cudaMemcpyDeviceToDevice);
                cudaMemcpy(m->vc[l][kvh] + (size_t)pos * D, m->v + (size_t)kvh * D, D * sizeof(float), cudaMemcpyDeviceToDevice);
            }
            for (int hq = 0; hq < Hq; hq++) {
                int kvh = hq / G;
                ref_sgemm(2, 1, S, D, m->q + (size_t)hq * D, m->kc[l][kvh], m->scores);
                gpu_scale(m->scores, scale, m->scores, S);
                gpu_softmax_fwd(m->scores, m->probs, 1, S);
                ref_sgemm(0, 1, D, S, m->probs, m->vc[l][kvh], m->attn + (size_t)hq * D);
            }
        } else {
            int64_t headStride = (int64_t)m->maxSeq * D, seqStride = headStride * Hkv;
            float *kcl = m->mk + (size_t)l * seqStride, *vcl = m->mv + (size_t)l * seqStride;
            int rc = m->ropeAppend(m->q, Hq, m->k, m->v, 0, 1, m->cosTab, m->sinTab, nullptr, pos, kcl, vcl, 0, nullptr,
                                   seqStride, headStride, 0, m->maxSeq, 1, 1, Hkv, D, nullptr);
            if (rc) return 100 + rc;
            size_t need = m->decodeWs(1, Hq, Hkv, D, S, 0);
            if (need > m->wsBytes) return -3;
            rc = m->decode(m->q, 0, kcl, vcl, 0, nullptr, seqStride, headStride, nullptr, S, m->attn, 0, nullptr, 1, Hq,
                           Hkv, D, scale, 0, m->ws, need, nullptr);
            if (rc) return 200 + rc;
        }
        if (attn_dump) cudaMemcpyAsync(attn_dump + (size_t)l * n, m->attn, n * sizeof(float), cudaMemcpyDeviceToDevice, 0);
        float *nx = ref_layer_tail(m, l, 1, cur);
        /* ping-pong between x and xnew so the next layer's residual input is not overwritten */
        if (nx == m->xnew) { std::swap(m->x, m->xnew); cur = m->x; }
    }
    gpu_rmsnorm_affine_fwd(cur, m->lnFg, m->xn, m->rms, 1, n);
    ref_sgemm(2, 1, m->vocab, n, m->xn, m->lmHead, m->logits);
    pos += 1;
    CK(cudaMemcpy(logits_host, m->logits, (size_t)m->vocab * sizeof(float), cudaMemcpyDeviceToHost));
    return 0;
}

/* ---- the whole single-token step as ONE CUDA graph (the reference's unused graph bindings,
 * src/gpu.nim:80-102, and its TODO "CUDA graphs for the single-token forward") ----------------
 * Same work as ref_model_step with impl 2, but nothing in it depends on host values that change
 * from token to token: the token id, its position and the attended length are read from device
 * memory, the decode is sized for the whole cache.  Captured once, replayed per token.  Needs the
 * build whose default stream can be captured. */
int ref_model_graph_available(void) { return REF_CAN_CAPTURE; }

static int ref_token_body(RefModel *m) {
    int n = m->nEmbd, D = m->headDim, Hq = m->nHead, Hkv = m->nKvHead;
    float scale = 1.0f / sqrtf((float)D);
    int64_t headStride = (int64_t)m->maxSeq * D, seqStride = headStride * Hkv;
    size_t need = m->decodeWs(1, Hq, Hkv, D, m->maxSeq, 0);
    if (need > m->wsBytes) return -3;
    gpu_embed_fwd(m->wte, m->tokIds, m->x, 1, n);
    float *cur = m->x, *other = m->xnew;
    for (int l = 0; l < m->nLayer; l++) {
        gpu_rmsnorm_affine_fwd(cur, m->ln1[l], m->xn, m->rms, 1, n);
        float *kcl = m->mk + (size_t)l * seqStride, *vcl = m->mv + (size_t)l * seqStride;
        int rc = m->qkv(m->xn, m->wq[l], m->wk[l], m->wv[l], 0, m->q, nullptr, nullptr, m->cosTab, m->sinTab, m->dPos, 0, kcl,
                        vcl, 0, nullptr, seqStride, headStride, 0, m->maxSeq, 1, n, Hq, Hkv, D, REF_STREAM);
        if (rc) return 400 + rc;
        rc = m->decode(m->q, 0, kcl, vcl, 0, nullptr, seqStride, headStride, m->dLen, m->maxSeq, m->attn, 0, nullptr, 1, Hq,
                       Hkv, D, scale, 0, m->ws, need, REF_STREAM);
        if (rc) return 200 + rc;
        rc = m->woResid(m->attn, m->wo[l], 0, cur, m->x2, 1, n, n, REF_STREAM);
        if (rc) return 500 + rc;
        /* the feed-forward half with explicit buffers (no pointer swapping inside a captured body) */
        int f = m->ffnDim;
        gpu_rmsnorm_affine_fwd(m->x2, m->ln2[l], m->xn, m->rms, 1, n);
        ref_sgemm(2, 1, f, n, m->xn, m->gate[l], m->gateo);
        ref_sgemm(2, 1, f, n, m->xn, m->up[l], m->upo);
        gpu_swiglu_fwd(m->gateo, m->upo, m->sw, f);
        ref_sgemm(2, 1, n, f, m->sw, m->down[l], m->mlp);
        gpu_add(m->x2, m->mlp, other, n);
        std::swap(cur, other);
    }
    gpu_rmsnorm_affine_fwd(cur, m->lnFg, m->xn, m->rms, 1, n);
    ref_sgemm(2, 1, m->vocab, n, m->xn, m->lmHead, m->logits);
    return 0;
}

/* returns 0, or -5 when this build cannot capture; launches_out (optional): kernel nodes of the graph */
int ref_model_step_graph(void *h, int token, float *logits_host, int *launches_out) {
    RefModel *m = (RefModel *)h;
    if (!REF_CAN_CAPTURE) return -5;
    if (!m->qkv || !m->woResid || !m->decode) return -4;
    if (m->mpos + 1 > m->maxSeq) return -2;
    int32_t pos = m->mpos, len = m->mpos + 1;
    CK(cudaMemcpyAsync(m->tokIds, &token, sizeof(int), cudaMemcpyHostToDevice, REF_STREAM));
    CK(cudaMemcpyAsync(m->dPos, &pos, sizeof(int32_t), cudaMemcpyHostToDevice, REF_STREAM));
    CK(cudaMemcpyAsync(m->dLen, &len, sizeof(int32_t), cudaMemcpyHostToDevice, REF_STREAM));
    CK(cudaStreamSynchronize(REF_STREAM));
    if (!m->graphExec) {
        /* once eagerly (module loading, cuBLAS set-up: none of that may happen inside a capture; the
         * step is idempotent, the replay below recomputes the same token), then the capture */
        int rc = ref_token_body(m);
        if (rc) return rc;
        CK(cudaStreamSynchronize(REF_STREAM));
        cudaGraph_t graph = nullptr;
        CK(cudaStreamBeginCapture(REF_STREAM, cudaStreamCaptureModeThreadLocal));
        rc = ref_token_body(m);
        cudaError_t e = cudaStreamEndCapture(REF_STREAM, &graph);
        if (rc || e != cudaSuccess || !graph) {
            fprintf(stderr, "ref_harness: capture of the token step failed (%d, %s)\n", rc, cudaGetErrorString(e));
            return rc ? rc : -6;
        }
        size_t nodes = 0;
        cudaGraphGetNodes(graph, nullptr, &nodes);
        if (launches_out) *launches_out = (int)nodes;
        CK(cudaGraphInstantiate(&m->graphExec, graph, 0));
        cudaGraphDestroy(graph);
    }
    CK(cudaGraphLaunch(m->graphExec, REF_STREAM));
    CK(cudaMemcpyAsync(logits_host, m->logits, (size_t)m->vocab * sizeof(float), cudaMemcpyDeviceToHost, REF_STREAM));
    CK(cudaStreamSynchronize(REF_STREAM));
    m->mpos += 1;
    return 0;
}

/* forward() over S prompt tokens (src/model.nim:454-549) with the LIBRARY's prefill as the
 * attention block, filling the library-side cache.  attn_dump: device [nLayer, S, nEmbd] or
 * NULL; logits_last_host: [vocab] of the last position. */
int ref_model_prefill_lib(void *h, const int *tokens_host, int S, float *attn_dump, float *logits_last_host) {
    RefModel *m = (RefModel *)h;
    if (S > m->maxPrefill || !m->prefill) return -2;
    int n = m->nEmbd, D = m->headDim, Hq = m->nHead, Hkv = m->nKvHead, nKv = Hkv * D;
    float scale = 1.0f / sqrtf((float)D);
    CK(cudaMemcpy(m->tokIds, tokens_host, S * sizeof(int), cudaMemcpyHostToDevice));
    gpu_embed_fwd(m->wte, m->tokIds, m->x, S, n);
    float *cur = m->x;
    int64_t headStride = (int64_t)m->maxSeq * D, seqStride = headStride * Hkv;
    for (int l = 0; l < m->nLayer; l++) {
        gpu_rmsnorm_affine_fwd(cur, m->ln1[l], m->xn, m->rms, S, n);
        ref_sgemm(2, S, n, n, m->xn, m->wq[l], m->q);
        ref_sgemm(2, S, nKv, n, m->xn, m->wk[l], m->k);
        ref_sgemm(2, S, nKv, n, m->xn, m->wv[l], m->v);
        int rc = m->prefill(m->q, m->k, m->v, 0, m->cosTab, m->sinTab, 0, m->attn, 1, S, Hq, Hkv, D, scale, 0,
                            m->mk + (size_t)l * seqStride, m->mv + (size_t)l * seqStride, 0, nullptr, seqStride,
                            headStride, m->maxSeq, nullptr, nullptr, 0, nullptr);
        if (rc) return 300 + rc;
        if (attn_dump)
            cudaMemcpyAsync(attn_dump + (size_t)l * S * n, m->attn, (size_t)S * n * sizeof(float), cudaMemcpyDeviceToDevice, 0);
        float *nx = ref_layer_tail(m, l, S, cur);
        if (nx == m->xnew) { std::swap(m->x, m->xnew); cur = m->x; }
    }
    gpu_rmsnorm_affine_fwd(cur, m->lnFg, m->xn, m->rms, S, n);
    ref_sgemm(2, S, m->vocab, n, m->xn, m->lmHead, m->logits);
    m->mpos = S;
    CK(cudaMemcpy(logits_last_host, m->logits + (size_t)(S - 1) * m->vocab, (size_t)m->vocab * sizeof(float),
                  cudaMemcpyDeviceToHost));
    return 0;
}

}  /* extern "C" */
