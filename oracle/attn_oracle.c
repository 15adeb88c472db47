/* attn_oracle.c -- CPU restatement of nimllm's GQA attention path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library and
 * the timed CPU baseline of the benchmark; the product never calls it.
 *
 * Every function cites the reference source it restates (paths are relative to
 * the nimllm project root).  The reference has no CPU forward pass: its
 * attention is a Nim host loop (src/model.nim) over cublasSgemm_v2 calls and
 * the scalar fp32 kernels of src/kernels.cu.  What is restated here is the
 * arithmetic of that sequence, in fp32, in the reference's operation order
 * where that order is visible in its sources (the softmax reduction tree is;
 * cuBLAS's accumulation order is not).
 *
 * Pinning: the reference's own tests hold no golden vector for multi-token
 * attention, so the restatement is pinned by running the reference's compiled
 * kernels (oracle/_ref, built from the reference's sources where they lie) on
 * the same seeded inputs on a GPU, and by committed fixtures generated from an
 * independent float64 formulation (tests/golden).
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared -fPIC).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- helpers */

static inline float bf16_to_f32(uint16_t h) {
    uint32_t u = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* round-to-nearest-even fp32 -> bf16 (NaN kept quiet) */
static inline uint16_t f32_to_bf16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

ORACLE_API void oracle_f32_to_bf16(const float *x, uint16_t *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = f32_to_bf16(x[i]);
}

ORACLE_API void oracle_bf16_to_f32(const uint16_t *x, float *y, int64_t n) {
    for (int64_t i = 0; i < n; i++) y[i] = bf16_to_f32(x[i]);
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORACLE_API void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* ------------------------------------------------------------ RoPE tables
 * src/model.nim:153-163 -- tables [max_pos, D/2], fp32 throughout:
 *   theta = float32(pos) / pow(ropeTheta, 2f * f / headDim); cos(theta); sin(theta)
 * Nim's pow/cos/sin on float32 bind the C float functions. */
ORACLE_API void oracle_rope_tables(float *cos_tab, float *sin_tab, int max_pos,
                                   int head_dim, float base) {
    int half = head_dim / 2;
    for (int pos = 0; pos < max_pos; pos++)
        for (int f = 0; f < half; f++) {
            float theta = (float)pos / powf(base, 2.0f * (float)f / (float)head_dim);
            cos_tab[(int64_t)pos * half + f] = cosf(theta);
            sin_tab[(int64_t)pos * half + f] = sinf(theta);
        }
}

/* ------------------------------------------------------------------ RoPE
 * src/kernels.cu:399-423 (k_rope / gpu_rope_fwd), in place on data [S, n_embd],
 * heads are column blocks of width head_dim, pairs (f, f + D/2), table row =
 * row index of data (the decode caller advances the table pointer by pos rows,
 * src/model.nim:790-797). */
ORACLE_API void oracle_rope_fwd(float *data, const float *cos_tab, const float *sin_tab,
                                int seq_len, int n_embd, int n_head, int head_dim) {
    int half = head_dim / 2;
    for (int pos = 0; pos < seq_len; pos++)
        for (int h = 0; h < n_head; h++)
            for (int f = 0; f < half; f++) {
                int64_t base = (int64_t)pos * n_embd + (int64_t)h * head_dim;
                float c = cos_tab[(int64_t)pos * half + f];
                float s = sin_tab[(int64_t)pos * half + f];
                float x0 = data[base + f];
                float x1 = data[base + f + half];
                data[base + f] = x0 * c - x1 * s;
                data[base + f + half] = x0 * s + x1 * c;
            }
}

/* ---------------------------------------------------------------- softmax
 * src/kernels.cu:267-303,330-339 (k_softmax, gpu_softmax_fwd): one block per
 * row, T = min(next_pow2(cols), 256) threads; thread t covers j = t, t+T, ...;
 * max and sum go through a shared-memory halving tree; the row is then
 * multiplied by 1/sum.  The tree order is restated so that the sum's rounding
 * matches the kernel's. */
static int next_pow2_cap256(int n) {
    int p = 1;
    while (p < n) p <<= 1;
    return p < 256 ? p : 256;
}

static void softmax_row(const float *x, float *y, int cols) {
    int T = next_pow2_cap256(cols);
    float part[256];
    float mx = -FLT_MAX;
    for (int j = 0; j < cols; j++) mx = fmaxf(mx, x[j]);
    for (int t = 0; t < T; t++) {
        float s = 0.0f;
        for (int j = t; j < cols; j += T) {
            float e = expf(x[j] - mx);
            y[j] = e;
            s += e;
        }
        part[t] = s;
    }
    for (int s = T / 2; s > 0; s >>= 1)
        for (int t = 0; t < s; t++) part[t] += part[t + s];
    float inv = 1.0f / part[0];
    for (int j = 0; j < cols; j++) y[j] *= inv;
}

ORACLE_API void oracle_softmax_fwd(const float *x, float *y, int rows, int cols) {
    for (int r = 0; r < rows; r++)
        softmax_row(x + (int64_t)r * cols, y + (int64_t)r * cols, cols);
}

/* src/kernels.cu:248-263 (k_causal_mask): col > row -> -1e9f, else *= scale. */
ORACLE_API void oracle_causal_mask(float *scores, float scale, int seq_len) {
    for (int r = 0; r < seq_len; r++)
        for (int c = 0; c < seq_len; c++) {
            int64_t i = (int64_t)r * seq_len + c;
            if (c > r) scores[i] = -1e9f; else scores[i] *= scale;
        }
}

/* src/kernels.cu:145-149,159-161 (k_scale). */
ORACLE_API void oracle_scale(const float *x, float s, float *y, int n) {
    for (int i = 0; i < n; i++) y[i] = x[i] * s;
}

/* src/kernels.cu:349-356 / 358-365 / 439-449: strided head gather / scatter. */
ORACLE_API void oracle_extract_head(const float *src, float *dst, int h, int seq_len,
                                    int n_embd, int head_dim) {
    for (int p = 0; p < seq_len; p++)
        memcpy(dst + (int64_t)p * head_dim, src + (int64_t)p * n_embd + (int64_t)h * head_dim,
               sizeof(float) * head_dim);
}

ORACLE_API void oracle_extract_kv_head(const float *src, float *dst, int q_head, int kv_repeat,
                                       int seq_len, int n_kv_dim, int head_dim) {
    oracle_extract_head(src, dst, q_head / kv_repeat, seq_len, n_kv_dim, head_dim);
}

ORACLE_API void oracle_insert_head(const float *src, float *dst, int h, int seq_len,
                                   int n_embd, int head_dim) {
    for (int p = 0; p < seq_len; p++)
        memcpy(dst + (int64_t)p * n_embd + (int64_t)h * head_dim, src + (int64_t)p * head_dim,
               sizeof(float) * head_dim);
}

/* -------------------------------------------------- row-major fp32 GEMMs
 * src/gpu.nim:185-207 (gpuSgemm): op bit 2 -> B transposed.  Only the two
 * shapes the attention path uses are restated: op 2 (C = A * B^T) and op 0
 * (C = A * B), beta = 0, fp32 multiply and accumulate. */
static void sgemm_nt(int m, int n, int k, const float *a, int lda, const float *b, int ldb,
                     float *c, int ldc) {
    for (int i = 0; i < m; i++)
        for (int j = 0; j < n; j++) {
            const float *ai = a + (int64_t)i * lda, *bj = b + (int64_t)j * ldb;
            float acc = 0.0f;
            for (int d = 0; d < k; d++) acc += ai[d] * bj[d];
            c[(int64_t)i * ldc + j] = acc;
        }
}

static void sgemm_nn(int m, int n, int k, const float *a, int lda, const float *b, int ldb,
                     float *c, int ldc) {
    for (int i = 0; i < m; i++) {
        float *ci = c + (int64_t)i * ldc;
        for (int j = 0; j < n; j++) ci[j] = 0.0f;
        for (int d = 0; d < k; d++) {
            float av = a[(int64_t)i * lda + d];
            const float *bd = b + (int64_t)d * ldb;
            for (int j = 0; j < n; j++) ci[j] += av * bd[j];
        }
    }
}

/* ------------------------------------------------------- prefill attention
 * src/model.nim:469-475,494-508: RoPE(q), RoPE(k) in place, then per QUERY head
 * h: gather q head, gather KV head h / kvRepeat, scores = qH kH^T, causal mask
 * + scale, softmax, attnH = probs vH, scatter into attnOut[:, h*D ..].
 * q [S, Hq*D], k, v [S, Hkv*D], out [S, Hq*D]; q and k are left rotated, as
 * the reference leaves them (the saveCache contract, src/model.nim:534,656-685).
 * cos/sin point at the table row of the first token. */
ORACLE_API void oracle_attn_forward(float *q, float *k, const float *v, const float *cos_tab,
                                    const float *sin_tab, float *out, int S, int Hq, int Hkv,
                                    int D, int apply_rope) {
    int E = Hq * D, Ekv = Hkv * D, G = Hq / Hkv;
    float scale = 1.0f / sqrtf((float)D);
    if (apply_rope) {
        oracle_rope_fwd(q, cos_tab, sin_tab, S, E, Hq, D);
        oracle_rope_fwd(k, cos_tab, sin_tab, S, Ekv, Hkv, D);
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < Hq; h++) {
        float *qH = (float *)malloc(sizeof(float) * S * D);
        float *kH = (float *)malloc(sizeof(float) * S * D);
        float *vH = (float *)malloc(sizeof(float) * S * D);
        float *aH = (float *)malloc(sizeof(float) * S * D);
        float *scores = (float *)malloc(sizeof(float) * (size_t)S * S);
        float *probs = (float *)malloc(sizeof(float) * (size_t)S * S);
        oracle_extract_head(q, qH, h, S, E, D);
        oracle_extract_kv_head(k, kH, h, G, S, Ekv, D);
        oracle_extract_kv_head(v, vH, h, G, S, Ekv, D);
        sgemm_nt(S, S, D, qH, D, kH, D, scores, S);
        oracle_causal_mask(scores, scale, S);
        oracle_softmax_fwd(scores, probs, S, S);
        sgemm_nn(S, D, S, probs, S, vH, D, aH, D);
        oracle_insert_head(aH, out, h, S, E, D);
        free(qH); free(kH); free(vH); free(aH); free(scores); free(probs);
    }
}

/* ------------------------------------------------------- attention backward
 * src/model.nim:639-685: per QUERY head h the probabilities are recomputed (scores = qH kH^T,
 * causal mask + scale, softmax), then dWeights = doutH vH^T, dvH = probs^T doutH,
 * dScores = softmax_bwd(probs, dWeights) (src/kernels.cu:305-328: y * (dy - sum_j dy_j y_j)),
 * dScores *= scale, dqH = dScores kH, dkH = dScores^T qH; dqH goes to columns h*D.. of dq, dkH and
 * dvH are ADDED to the columns of KV head h / kvRepeat (src/kernels.cu:451-461), and finally the
 * rotation is undone on dq and dk (gpu_rope_bwd, src/kernels.cu:425-431: k_rope with sign -1).
 * q_rot, k_rot are the post-RoPE activations the forward saved (saveCache), v raw.
 * dq [S, Hq*D], dk, dv [S, Hkv*D] are overwritten.  acc64 != 0 accumulates every product in
 * float64 (ground truth for tolerance statements). */
static void rope_bwd_rows(float *data, const float *cos_tab, const float *sin_tab, int seq_len,
                          int n_embd, int n_head, int head_dim) {
    int half = head_dim / 2;
    for (int pos = 0; pos < seq_len; pos++)
        for (int h = 0; h < n_head; h++)
            for (int f = 0; f < half; f++) {
                int64_t base = (int64_t)pos * n_embd + (int64_t)h * head_dim;
                float c = cos_tab[(int64_t)pos * half + f];
                float s = -sin_tab[(int64_t)pos * half + f];      /* sign = -1 */
                float x0 = data[base + f];
                float x1 = data[base + f + half];
                data[base + f] = x0 * c - x1 * s;
                data[base + f + half] = x0 * s + x1 * c;
            }
}

ORACLE_API void oracle_rope_bwd(float *data, const float *cos_tab, const float *sin_tab,
                                int seq_len, int n_embd, int n_head, int head_dim) {
    rope_bwd_rows(data, cos_tab, sin_tab, seq_len, n_embd, n_head, head_dim);
}

ORACLE_API void oracle_attn_backward(const float *q_rot, const float *k_rot, const float *v,
                                     const float *dout, const float *cos_tab, const float *sin_tab,
                                     float *dq, float *dk, float *dv, int S, int Hq, int Hkv, int D,
                                     int apply_rope, int acc64) {
    int E = Hq * D, Ekv = Hkv * D, G = Hq / Hkv;
    float scale = 1.0f / sqrtf((float)D);
    memset(dq, 0, sizeof(float) * (size_t)S * E);
    memset(dk, 0, sizeof(float) * (size_t)S * Ekv);
    memset(dv, 0, sizeof(float) * (size_t)S * Ekv);
    /* the query heads of one KV head are walked in order by one thread, like the reference's loop */
#pragma omp parallel for schedule(dynamic, 1)
    for (int kvh = 0; kvh < Hkv; kvh++) {
        float *probs = (float *)malloc(sizeof(float) * (size_t)S * S);
        float *scores = (float *)malloc(sizeof(float) * (size_t)S * S);
        double *dS = (double *)malloc(sizeof(double) * (size_t)S * S);
        for (int h = kvh * G; h < (kvh + 1) * G; h++) {
            const float *qh = q_rot + (int64_t)h * D, *kh = k_rot + (int64_t)kvh * D, *vh = v + (int64_t)kvh * D;
            const float *doh = dout + (int64_t)h * D;
            for (int i = 0; i < S; i++)
                for (int j = 0; j < S; j++) {
                    if (acc64) {
                        double a = 0.0;
                        for (int d = 0; d < D; d++) a += (double)qh[(int64_t)i * E + d] * kh[(int64_t)j * Ekv + d];
                        scores[(int64_t)i * S + j] = (float)a;
                    } else {
                        float a = 0.0f;
                        for (int d = 0; d < D; d++) a += qh[(int64_t)i * E + d] * kh[(int64_t)j * Ekv + d];
                        scores[(int64_t)i * S + j] = a;
                    }
                }
            oracle_causal_mask(scores, scale, S);
            oracle_softmax_fwd(scores, probs, S, S);
            for (int i = 0; i < S; i++) {
                /* dWeights row, then softmax_bwd of the row, then * scale */
                double dot = 0.0;
                float dotf = 0.0f;
                for (int j = 0; j < S; j++) {
                    double a = 0.0;
                    float af = 0.0f;
                    for (int d = 0; d < D; d++) {
                        a += (double)doh[(int64_t)i * E + d] * vh[(int64_t)j * Ekv + d];
                        af += doh[(int64_t)i * E + d] * vh[(int64_t)j * Ekv + d];
                    }
                    dS[(int64_t)i * S + j] = acc64 ? a : (double)af;
                    dot += dS[(int64_t)i * S + j] * probs[(int64_t)i * S + j];
                    dotf += (float)dS[(int64_t)i * S + j] * probs[(int64_t)i * S + j];
                }
                for (int j = 0; j < S; j++) {
                    float pij = probs[(int64_t)i * S + j];
                    if (acc64) dS[(int64_t)i * S + j] = (double)pij * (dS[(int64_t)i * S + j] - dot) * scale;
                    else dS[(int64_t)i * S + j] = (double)((pij * ((float)dS[(int64_t)i * S + j] - dotf)) * scale);
                }
            }
            for (int j = 0; j < S; j++)
                for (int d = 0; d < D; d++) {
                    double av = 0.0, ak = 0.0;
                    float avf = 0.0f, akf = 0.0f;
                    for (int i = j; i < S; i++) {          /* rows above the diagonal have p = dS = 0 */
                        av += (double)probs[(int64_t)i * S + j] * doh[(int64_t)i * E + d];
                        ak += dS[(int64_t)i * S + j] * qh[(int64_t)i * E + d];
                        avf += probs[(int64_t)i * S + j] * doh[(int64_t)i * E + d];
                        akf += (float)dS[(int64_t)i * S + j] * qh[(int64_t)i * E + d];
                    }
                    dv[(int64_t)j * Ekv + (int64_t)kvh * D + d] += acc64 ? (float)av : avf;
                    dk[(int64_t)j * Ekv + (int64_t)kvh * D + d] += acc64 ? (float)ak : akf;
                }
            for (int i = 0; i < S; i++)
                for (int d = 0; d < D; d++) {
                    double a = 0.0;
                    float af = 0.0f;
                    for (int j = 0; j <= i; j++) {
                        a += dS[(int64_t)i * S + j] * kh[(int64_t)j * Ekv + d];
                        af += (float)dS[(int64_t)i * S + j] * kh[(int64_t)j * Ekv + d];
                    }
                    dq[(int64_t)i * E + (int64_t)h * D + d] = acc64 ? (float)a : af;
                }
        }
        free(probs); free(scores); free(dS);
    }
    if (apply_rope) {
        rope_bwd_rows(dq, cos_tab, sin_tab, S, E, Hq, D);
        rope_bwd_rows(dk, cos_tab, sin_tab, S, Ekv, Hkv, D);
    }
}

/* ------------------------------------------------------------- KV append
 * src/model.nim:799-815: row pos (rows pos..pos+n-1) of KV head kvh's buffer
 * [max_seq, D] <- columns kvh*D.. of kNew / vNew [n, Hkv*D].  K arrives
 * already rotated (src/model.nim:797), V raw.  Here the cache of one layer is
 * one array [Hkv, max_seq, D] per K and V (the reference's per-head buffers,
 * src/model.nim:729-739, laid end to end). */
ORACLE_API void oracle_kv_append(const float *k_new, const float *v_new, float *k_cache,
                                 float *v_cache, int pos, int n, int Hkv, int D, int max_seq) {
    int Ekv = Hkv * D;
    for (int h = 0; h < Hkv; h++)
        for (int t = 0; t < n; t++) {
            int64_t dst = ((int64_t)h * max_seq + pos + t) * D;
            int64_t src = (int64_t)t * Ekv + (int64_t)h * D;
            memcpy(k_cache + dst, k_new + src, sizeof(float) * D);
            memcpy(v_cache + dst, v_new + src, sizeof(float) * D);
        }
}

/* --------------------------------------------------------- cached decode
 * src/model.nim:788-840 with newTokens == 1: RoPE(q, kNew) at table row pos,
 * append, then per query head h (kvh = h / kvRepeat): scores[1, L] = qH K^T
 * (L = pos + 1, the appended row included), * scale, softmax, out = probs V.
 * q [Hq*D], k_new / v_new [Hkv*D] (rotated in place, like the reference),
 * caches [Hkv, max_seq, D]; out [Hq*D]. */
ORACLE_API void oracle_attn_forward_cached(float *q, float *k_new, const float *v_new,
                                           const float *cos_tab, const float *sin_tab,
                                           float *k_cache, float *v_cache, int pos, float *out,
                                           int Hq, int Hkv, int D, int max_seq) {
    int E = Hq * D, Ekv = Hkv * D, G = Hq / Hkv, half = D / 2;
    int L = pos + 1;
    float scale = 1.0f / sqrtf((float)D);
    oracle_rope_fwd(q, cos_tab + (int64_t)pos * half, sin_tab + (int64_t)pos * half, 1, E, Hq, D);
    oracle_rope_fwd(k_new, cos_tab + (int64_t)pos * half, sin_tab + (int64_t)pos * half, 1, Ekv,
                    Hkv, D);
    oracle_kv_append(k_new, v_new, k_cache, v_cache, pos, 1, Hkv, D, max_seq);
    float *scores = (float *)malloc(sizeof(float) * L);
    float *probs = (float *)malloc(sizeof(float) * L);
    for (int h = 0; h < Hq; h++) {
        int kvh = h / G;
        const float *kH = k_cache + (int64_t)kvh * max_seq * D;
        const float *vH = v_cache + (int64_t)kvh * max_seq * D;
        sgemm_nt(1, L, D, q + (int64_t)h * D, D, kH, D, scores, L);
        oracle_scale(scores, scale, scores, L);
        oracle_softmax_fwd(scores, probs, 1, L);
        sgemm_nn(1, D, L, probs, L, vH, D, out + (int64_t)h * D, D);
    }
    free(scores);
    free(probs);
}

/* ------------------------------------------- batched ragged decode (read side)
 * The per-sequence read half of src/model.nim:822-840, applied to a batch of
 * independent sequences with their own lengths: for sequence b and query head
 * h, softmax(scale * q_bh . K_b[kvh, 0..L_b)) . V_b[kvh].  No RoPE and no
 * append here (cached K is already rotated; the reference never re-rotates it).
 *
 * q    [B, Hq*D] fp32
 * k, v one array each; sequence b's block starts at element kv_off[b] and is
 *      [Hkv, cap_b, D] with head stride head_stride[b] elements; kv_bf16 != 0
 *      means the arrays hold bf16 bit patterns (uint16), widened exactly.
 * out  [B, Hq*D] fp32.  acc64 != 0 accumulates dot products, the softmax sum
 *      and the output in float64 (the "ground truth" the bf16 tolerance is
 *      stated against); acc64 == 0 is the reference's fp32 arithmetic.
 * If part_m / part_l are non-NULL the routine also returns, per (b, h), the
 * row maximum of the scaled scores and the sum of exp(s - max). */
ORACLE_API void oracle_decode_batch(const float *q, const void *k, const void *v,
                                    const int64_t *kv_off, const int64_t *head_stride,
                                    const int32_t *seq_len, float *out, int B, int Hq, int Hkv,
                                    int D, float scale, int kv_bf16, int acc64, float *part_m,
                                    float *part_l) {
    int G = Hq / Hkv, E = Hq * D;
#pragma omp parallel for collapse(2) schedule(dynamic, 1)
    for (int b = 0; b < B; b++)
        for (int h = 0; h < Hq; h++) {
            int L = seq_len[b];
            int kvh = h / G;
            int64_t base = kv_off[b] + (int64_t)kvh * head_stride[b];
            const float *qh = q + (int64_t)b * E + (int64_t)h * D;
            float *oh = out + (int64_t)b * E + (int64_t)h * D;
            if (L <= 0) {
                for (int d = 0; d < D; d++) oh[d] = 0.0f;
                if (part_m) { part_m[b * Hq + h] = -INFINITY; part_l[b * Hq + h] = 0.0f; }
                continue;
            }
            float *scores = (float *)malloc(sizeof(float) * L);
            double *scores64 = acc64 ? (double *)malloc(sizeof(double) * L) : NULL;
            float krow[512];
            for (int j = 0; j < L; j++) {
                const float *kr;
                if (kv_bf16) {
                    const uint16_t *kp = (const uint16_t *)k + base + (int64_t)j * D;
                    for (int d = 0; d < D; d++) krow[d] = bf16_to_f32(kp[d]);
                    kr = krow;
                } else {
                    kr = (const float *)k + base + (int64_t)j * D;
                }
                if (acc64) {
                    double a = 0.0;
                    for (int d = 0; d < D; d++) a += (double)qh[d] * (double)kr[d];
                    scores64[j] = a * (double)scale;
                } else {
                    float a = 0.0f;
                    for (int d = 0; d < D; d++) a += qh[d] * kr[d];
                    scores[j] = a * scale;
                }
            }
            if (acc64) {
                double mx = -DBL_MAX, sum = 0.0;
                double acc[512];
                for (int j = 0; j < L; j++) if (scores64[j] > mx) mx = scores64[j];
                for (int d = 0; d < D; d++) acc[d] = 0.0;
                for (int j = 0; j < L; j++) {
                    double p = exp(scores64[j] - mx);
                    sum += p;
                    if (kv_bf16) {
                        const uint16_t *vp = (const uint16_t *)v + base + (int64_t)j * D;
                        for (int d = 0; d < D; d++) acc[d] += p * (double)bf16_to_f32(vp[d]);
                    } else {
                        const float *vp = (const float *)v + base + (int64_t)j * D;
                        for (int d = 0; d < D; d++) acc[d] += p * (double)vp[d];
                    }
                }
                for (int d = 0; d < D; d++) oh[d] = (float)(acc[d] / sum);
                if (part_m) { part_m[b * Hq + h] = (float)mx; part_l[b * Hq + h] = (float)sum; }
                free(scores64);
            } else {
                float *probs = (float *)malloc(sizeof(float) * L);
                softmax_row(scores, probs, L);
                for (int d = 0; d < D; d++) oh[d] = 0.0f;
                for (int j = 0; j < L; j++) {
                    float p = probs[j];
                    if (kv_bf16) {
                        const uint16_t *vp = (const uint16_t *)v + base + (int64_t)j * D;
                        for (int d = 0; d < D; d++) oh[d] += p * bf16_to_f32(vp[d]);
                    } else {
                        const float *vp = (const float *)v + base + (int64_t)j * D;
                        for (int d = 0; d < D; d++) oh[d] += p * vp[d];
                    }
                }
                if (part_m) {
                    float mx = -FLT_MAX, sum = 0.0f;
                    for (int j = 0; j < L; j++) mx = fmaxf(mx, scores[j]);
                    for (int j = 0; j < L; j++) sum += expf(scores[j] - mx);
                    part_m[b * Hq + h] = mx;
                    part_l[b * Hq + h] = sum;
                }
                free(probs);
            }
            free(scores);
        }
}

/* ---------------------------------------------- causal prefill, ground truth
 * Same mathematics as oracle_attn_forward (src/model.nim:494-508) on inputs
 * that are already rotated, for a batch and with float64 accumulation, without
 * materialising S x S matrices, restricted to query rows [row0, row1) so that
 * long sequences can be sampled.  q [B, S, Hq*D], k, v [B, S, Hkv*D] fp32
 * (bf16-rounded values widened by the caller), out [B, row1-row0, Hq*D]. */
ORACLE_API void oracle_prefill_f64(const float *q, const float *k, const float *v, float *out,
                                   int B, int S, int Hq, int Hkv, int D, float scale, int row0,
                                   int row1) {
    int G = Hq / Hkv, E = Hq * D, Ekv = Hkv * D, R = row1 - row0;
#pragma omp parallel for collapse(3) schedule(dynamic, 4)
    for (int b = 0; b < B; b++)
        for (int h = 0; h < Hq; h++)
            for (int i = row0; i < row1; i++) {
                int kvh = h / G;
                const float *qi = q + ((int64_t)b * S + i) * E + (int64_t)h * D;
                double *s = (double *)malloc(sizeof(double) * (i + 1));
                double mx = -DBL_MAX, sum = 0.0, acc[512];
                for (int j = 0; j <= i; j++) {
                    const float *kj = k + ((int64_t)b * S + j) * Ekv + (int64_t)kvh * D;
                    double a = 0.0;
                    for (int d = 0; d < D; d++) a += (double)qi[d] * (double)kj[d];
                    s[j] = a * (double)scale;
                    if (s[j] > mx) mx = s[j];
                }
                for (int d = 0; d < D; d++) acc[d] = 0.0;
                for (int j = 0; j <= i; j++) {
                    const float *vj = v + ((int64_t)b * S + j) * Ekv + (int64_t)kvh * D;
                    double p = exp(s[j] - mx);
                    sum += p;
                    for (int d = 0; d < D; d++) acc[d] += p * (double)vj[d];
                }
                float *o = out + ((int64_t)b * R + (i - row0)) * E + (int64_t)h * D;
                for (int d = 0; d < D; d++) o[d] = (float)(acc[d] / sum);
                free(s);
            }
}

/* ------------------------------------------------ split-KV partial combine
 * Not in the reference (it never splits the KV sequence); this is the algebra
 * that makes a split softmax equal the unsplit one of src/kernels.cu:267-303:
 * with partials (m_r, l_r, o_r), o_r normalised by l_r,
 *   m = max m_r;  w_r = l_r exp(m_r - m);  out = sum w_r o_r / sum w_r.
 * parts [n_parts, rows, W] with W >= D + 2 floats per record: o[D], m, l, padding. */
ORACLE_API void oracle_combine(const float *parts, int n_parts, int rows, int D, int W,
                               float *out, float *out_m, float *out_l) {
    for (int r = 0; r < rows; r++) {
        double m = -INFINITY, wsum = 0.0, acc[512];
        for (int p = 0; p < n_parts; p++) {
            const float *pp = parts + ((int64_t)p * rows + r) * W;
            if (pp[D + 1] > 0.0f && pp[D] > m) m = pp[D];
        }
        for (int d = 0; d < D; d++) acc[d] = 0.0;
        for (int p = 0; p < n_parts; p++) {
            const float *pp = parts + ((int64_t)p * rows + r) * W;
            if (!(pp[D + 1] > 0.0f)) continue;
            double w = (double)pp[D + 1] * exp((double)pp[D] - m);
            wsum += w;
            for (int d = 0; d < D; d++) acc[d] += w * (double)pp[d];
        }
        for (int d = 0; d < D; d++) out[(int64_t)r * D + d] = wsum > 0.0 ? (float)(acc[d] / wsum) : 0.0f;
        if (out_m) { out_m[r] = (float)m; out_l[r] = (float)wsum; }
    }
}

/* ------------------------------------------------ quantised weights (decode projections)
 * Block formats of src/kernels.cu:898-901 (Q4_0: half scale + 16 bytes of nibbles) and
 * :1013-1016 (Q8_0: half scale + 32 int8).  Blocks are packed without padding: 18 and 34 bytes. */
static inline uint16_t f32_to_f16_bits(float f) { _Float16 h = (_Float16)f; uint16_t u; memcpy(&u, &h, 2); return u; }
static inline float f16_bits_to_f32(uint16_t u) { _Float16 h; memcpy(&h, &u, 2); return (float)h; }

/* k_quantize_q4_0, src/kernels.cu:904-932: d = amax / 7, q = min(15, (int)(x / d + 8.5)) */
ORACLE_API void oracle_quantize_q4_0(const float *x, uint8_t *y, int64_t n) {
    for (int64_t blk = 0; blk < n / 32; blk++) {
        const float *src = x + blk * 32;
        uint8_t *dst = y + blk * 18;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) { float a = fabsf(src[i]); if (a > amax) amax = a; }
        float d = amax / 7.0f;
        float id = d ? 1.0f / d : 0.0f;
        uint16_t hb = f32_to_f16_bits(d);
        memcpy(dst, &hb, 2);
        for (int i = 0; i < 16; i++) {
            int v0 = (int)(src[i * 2 + 0] * id + 8.5f); if (v0 > 15) v0 = 15;
            int v1 = (int)(src[i * 2 + 1] * id + 8.5f); if (v1 > 15) v1 = 15;
            dst[2 + i] = (uint8_t)(v0 | (v1 << 4));
        }
    }
}

/* The reference has no Q8_0 quantiser (its Q8_0 weights come out of GGUF files,
 * src/model.nim:405-407); this is the usual one for the format: d = amax / 127, q = round(x / d). */
ORACLE_API void oracle_quantize_q8_0(const float *x, uint8_t *y, int64_t n) {
    for (int64_t blk = 0; blk < n / 32; blk++) {
        const float *src = x + blk * 32;
        uint8_t *dst = y + blk * 34;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) { float a = fabsf(src[i]); if (a > amax) amax = a; }
        float d = amax / 127.0f;
        float id = d ? 1.0f / d : 0.0f;
        uint16_t hb = f32_to_f16_bits(d);
        memcpy(dst, &hb, 2);
        for (int i = 0; i < 32; i++) dst[2 + i] = (uint8_t)(int8_t)lrintf(src[i] * id);
    }
}

/* value of weight j of a row: d * (nibble - 8) (src/kernels.cu:966-970) or d * q (:1033-1036) */
ORACLE_API void oracle_dequantize(const uint8_t *A, int q4, float *out, int64_t n) {
    const int bs = q4 ? 18 : 34;
    for (int64_t blk = 0; blk < n / 32; blk++) {
        const uint8_t *b = A + blk * bs;
        uint16_t hb; memcpy(&hb, b, 2);
        const float d = f16_bits_to_f32(hb);
        for (int i = 0; i < 32; i++) {
            int q = q4 ? ((i & 1) ? (b[2 + i / 2] >> 4) : (b[2 + i / 2] & 0x0F)) - 8 : (int)(int8_t)b[2 + i];
            out[blk * 32 + i] = d * (float)q;
        }
    }
}

/* k_matvec_q4_0 / k_matvec_q8_0: y[row] = sum over blocks of d * (sum over the block of q * x), the
 * block sums in float as the kernels form them; the sum over blocks in float (acc64 = 0, any order
 * is within the 1e-4 bound) or in double (acc64 = 1: ground truth). */
ORACLE_API void oracle_matvec_q(const uint8_t *A, int q4, const float *x, float *y, int rows, int cols, int acc64) {
    const int bs = q4 ? 18 : 34, bpr = cols / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const uint8_t *rp = A + (int64_t)r * bpr * bs;
        double sum64 = 0.0; float sum32 = 0.0f;
        for (int blk = 0; blk < bpr; blk++) {
            const uint8_t *b = rp + blk * bs;
            uint16_t hb; memcpy(&hb, b, 2);
            const float d = f16_bits_to_f32(hb);
            if (acc64) {
                double local = 0.0;
                for (int i = 0; i < 32; i++) {
                    int q = q4 ? ((i & 1) ? (b[2 + i / 2] >> 4) : (b[2 + i / 2] & 0x0F)) - 8 : (int)(int8_t)b[2 + i];
                    local += (double)q * (double)x[blk * 32 + i];
                }
                sum64 += (double)d * local;
            } else {
                float local = 0.0f;
                for (int i = 0; i < 32; i++) {
                    int q = q4 ? ((i & 1) ? (b[2 + i / 2] >> 4) : (b[2 + i / 2] & 0x0F)) - 8 : (int)(int8_t)b[2 + i];
                    local += (float)q * x[blk * 32 + i];
                }
                sum32 += d * local;
            }
        }
        y[r] = acc64 ? (float)sum64 : sum32;
    }
}
