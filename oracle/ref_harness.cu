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
}

static cublasHandle_t g_cublas = nullptr;

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
    return cublasCreate_v2(&g_cublas) == CUBLAS_STATUS_SUCCESS ? 0 : -1;
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

}  /* extern "C" */
