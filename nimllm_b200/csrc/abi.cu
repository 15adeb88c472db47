// abi.cu -- C entry points that are not tied to one kernel file: error reporting, RoPE
// tables, the contiguous KV cache, the RoPE/append entry and the prefill dispatcher.
#include <math.h>
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace nimllm {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace nimllm

using namespace nimllm;

struct nimllm_kvcache {
    void *k, *v;
    int n_layer, n_seq, n_kv_head, max_seq, head_dim, dtype, pos, device;
    size_t bytes;  // per K or V array
};

extern "C" {

const char *nimllm_attn_last_error(void) { return g_err; }
int nimllm_attn_version(void) { return 100; }

// src/model.nim:153-163
int nimllm_rope_tables_host(float *cos_tab, float *sin_tab, int max_pos, int head_dim, float base) {
    if (!cos_tab || !sin_tab || max_pos < 0 || head_dim <= 0 || (head_dim & 1))
        return fail(NIMLLM_ERR_ARG, "rope_tables_host: bad arguments");
    const int half = head_dim / 2;
    for (int pos = 0; pos < max_pos; pos++)
        for (int f = 0; f < half; f++) {
            float theta = (float)pos / powf(base, 2.0f * (float)f / (float)head_dim);
            cos_tab[(size_t)pos * half + f] = cosf(theta);
            sin_tab[(size_t)pos * half + f] = sinf(theta);
        }
    return NIMLLM_OK;
}

// src/model.nim:729-739 (initKvCache), one allocation per K and V instead of one per
// (layer, KV head)
nimllm_kvcache *nimllm_kvcache_create(int n_layer, int n_seq, int n_kv_head, int max_seq,
                                      int head_dim, int dtype) {
    if (n_layer <= 0 || n_seq <= 0 || n_kv_head <= 0 || max_seq <= 0 || head_dim <= 0 ||
        head_dim % 8 != 0 || !dtype_ok(dtype)) {
        set_error("kvcache_create: bad arguments");
        return nullptr;
    }
    nimllm_kvcache *kv = new nimllm_kvcache();
    kv->n_layer = n_layer; kv->n_seq = n_seq; kv->n_kv_head = n_kv_head; kv->max_seq = max_seq;
    kv->head_dim = head_dim; kv->dtype = dtype; kv->pos = 0;
    cudaGetDevice(&kv->device);
    kv->bytes = (size_t)n_layer * n_seq * n_kv_head * max_seq * head_dim * dtype_size(dtype);
    if (cudaMalloc(&kv->k, kv->bytes) != cudaSuccess) { set_error("kvcache_create: cudaMalloc(K) failed"); delete kv; return nullptr; }
    if (cudaMalloc(&kv->v, kv->bytes) != cudaSuccess) { set_error("kvcache_create: cudaMalloc(V) failed"); cudaFree(kv->k); delete kv; return nullptr; }
    cudaMemset(kv->k, 0, kv->bytes);
    cudaMemset(kv->v, 0, kv->bytes);
    return kv;
}

void nimllm_kvcache_destroy(nimllm_kvcache *kv) {
    if (!kv) return;
    cudaFree(kv->k);
    cudaFree(kv->v);
    delete kv;
}

// src/model.nim:741-746 (resetKvCache)
int nimllm_kvcache_reset(nimllm_kvcache *kv, void *stream) {
    if (!kv) return fail(NIMLLM_ERR_ARG, "kvcache_reset: null handle");
    cudaError_t e = cudaMemsetAsync(kv->k, 0, kv->bytes, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(kv->v, 0, kv->bytes, (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "kvcache_reset: %s", cudaGetErrorString(e));
    kv->pos = 0;
    return NIMLLM_OK;
}

static void *layer_ptr(const nimllm_kvcache *kv, void *base, int layer) {
    if (!kv || layer < 0 || layer >= kv->n_layer) return nullptr;
    size_t per_layer = kv->bytes / kv->n_layer;
    return (char *)base + per_layer * layer;
}
void *nimllm_kvcache_k(const nimllm_kvcache *kv, int layer) { return kv ? layer_ptr(kv, kv->k, layer) : nullptr; }
void *nimllm_kvcache_v(const nimllm_kvcache *kv, int layer) { return kv ? layer_ptr(kv, kv->v, layer) : nullptr; }
int nimllm_kvcache_pos(const nimllm_kvcache *kv) { return kv ? kv->pos : -1; }
void nimllm_kvcache_set_pos(nimllm_kvcache *kv, int pos) { if (kv) kv->pos = pos; }
int64_t nimllm_kvcache_seq_stride(const nimllm_kvcache *kv) {
    return kv ? (int64_t)kv->n_kv_head * kv->max_seq * kv->head_dim : 0;
}
int64_t nimllm_kvcache_head_stride(const nimllm_kvcache *kv) {
    return kv ? (int64_t)kv->max_seq * kv->head_dim : 0;
}

int nimllm_rope_append(void *q, int n_head, void *k_new, const void *v_new, int act_dtype,
                       int write_back_k, const float *rope_cos, const float *rope_sin,
                       const int32_t *seq_pos, int pos0, void *k_cache, void *v_cache,
                       int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                       int64_t head_stride, int cache_row0, int max_seq, int batch, int n,
                       int n_kv_head, int head_dim, void *stream) {
    if (batch < 0 || n < 0 || n_kv_head < 0 || n_head < 0 || head_dim <= 0 || head_dim % 8 != 0)
        return fail(NIMLLM_ERR_ARG, "rope_append: bad shape B=%d n=%d Hq=%d Hkv=%d D=%d", batch, n, n_head,
                    n_kv_head, head_dim);
    if (!dtype_ok(act_dtype) || !dtype_ok(cache_dtype)) return fail(NIMLLM_ERR_ARG, "rope_append: unknown dtype");
    if ((rope_cos == nullptr) != (rope_sin == nullptr))
        return fail(NIMLLM_ERR_ARG, "rope_append: give both RoPE tables or neither");
    if ((k_cache == nullptr) != (v_cache == nullptr))
        return fail(NIMLLM_ERR_ARG, "rope_append: give both cache pointers or neither");
    if (n_kv_head > 0 && (!k_new || !v_new)) return fail(NIMLLM_ERR_ARG, "rope_append: null k_new / v_new");
    if (k_cache && (head_stride % 8 != 0 || seq_stride % 8 != 0 || max_seq <= 0))
        return fail(NIMLLM_ERR_ARG, "rope_append: cache strides must be multiples of 8 elements and max_seq > 0");
    if (((uintptr_t)q | (uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)k_cache | (uintptr_t)v_cache |
         (uintptr_t)rope_cos | (uintptr_t)rope_sin) & 15)
        return fail(NIMLLM_ERR_ARG, "rope_append: q, k_new, v_new, the caches and the tables must be 16-byte aligned");
    if (batch == 0 || n == 0) return NIMLLM_OK;
    return launch_rope_append(q, q ? n_head : 0, k_new, v_new, act_dtype, write_back_k, rope_cos, rope_sin,
                              seq_pos, pos0, k_cache, v_cache, cache_dtype, kv_off, seq_stride, head_stride,
                              cache_row0, max_seq, batch, n, n_kv_head, head_dim, (cudaStream_t)stream);
}

// Same launch with the page of every new row resolved inside the kernel.
int nimllm_rope_append_paged(void *q, int n_head, void *k_new, const void *v_new, int act_dtype,
                             int write_back_k, const float *rope_cos, const float *rope_sin,
                             const int32_t *seq_pos, int pos0, void *k_pages, void *v_pages, int cache_dtype,
                             const int32_t *page_table, int max_pages, int page_rows, int n_pages, int batch,
                             int n, int n_kv_head, int head_dim, void *stream) {
    if (batch < 0 || n < 0 || n_kv_head <= 0 || n_head < 0 || head_dim <= 0 || head_dim % 8 != 0)
        return fail(NIMLLM_ERR_ARG, "rope_append_paged: bad shape B=%d n=%d Hq=%d Hkv=%d D=%d", batch, n, n_head,
                    n_kv_head, head_dim);
    if (!dtype_ok(act_dtype) || !dtype_ok(cache_dtype)) return fail(NIMLLM_ERR_ARG, "rope_append_paged: unknown dtype");
    if ((rope_cos == nullptr) != (rope_sin == nullptr))
        return fail(NIMLLM_ERR_ARG, "rope_append_paged: give both RoPE tables or neither");
    if (!k_new || !v_new || !k_pages || !v_pages || !page_table)
        return fail(NIMLLM_ERR_ARG, "rope_append_paged: null k_new / v_new / pages / page table");
    int shift = 0;
    while ((1 << shift) < page_rows) shift++;
    if (page_rows < 1 || (1 << shift) != page_rows || max_pages <= 0 || n_pages <= 0)
        return fail(NIMLLM_ERR_ARG, "rope_append_paged: page_rows %d must be a power of two, max_pages and n_pages > 0",
                    page_rows);
    if (((uintptr_t)k_pages | (uintptr_t)v_pages | (uintptr_t)k_new | (uintptr_t)v_new | (uintptr_t)q) & 15)
        return fail(NIMLLM_ERR_ARG, "rope_append_paged: q, k_new, v_new and the pages must be 16-byte aligned");
    if (batch == 0 || n == 0) return NIMLLM_OK;
    return launch_rope_append(q, q ? n_head : 0, k_new, v_new, act_dtype, write_back_k, rope_cos, rope_sin, seq_pos,
                              pos0, k_pages, v_pages, cache_dtype, nullptr, 0, 0, 0, 0, batch, n, n_kv_head, head_dim,
                              (cudaStream_t)stream, page_table, max_pages, shift, n_pages);
}

size_t nimllm_attn_prefill_workspace_bytes(int batch, int seq_len, int n_head, int n_kv_head,
                                           int head_dim, int dtype) {
    // neither path needs scratch memory (kept in the interface so that a future kernel may ask for some)
    (void)batch; (void)seq_len; (void)n_head; (void)n_kv_head; (void)head_dim; (void)dtype;
    return 0;
}

int nimllm_attn_prefill(void *q, void *k, const void *v, int dtype, const float *rope_cos,
                        const float *rope_sin, int pos0, void *out, int batch, int seq_len,
                        int n_head, int n_kv_head, int head_dim, float scale, int save_cache,
                        void *k_cache, void *v_cache, int cache_dtype, const int64_t *kv_off,
                        int64_t seq_stride, int64_t head_stride, int max_seq, float *lse,
                        void *workspace, size_t workspace_bytes, void *stream) {
    if (!q || !k || !v || !out) return fail(NIMLLM_ERR_ARG, "attn_prefill: null q / k / v / out");
    if (batch < 0 || seq_len < 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head != 0)
        return fail(NIMLLM_ERR_ARG, "attn_prefill: bad shape B=%d S=%d Hq=%d Hkv=%d", batch, seq_len, n_head,
                    n_kv_head);
    if (!dtype_ok(dtype)) return fail(NIMLLM_ERR_ARG, "attn_prefill: unknown dtype");
    if ((rope_cos == nullptr) != (rope_sin == nullptr))
        return fail(NIMLLM_ERR_ARG, "attn_prefill: give both RoPE tables or neither");
    if (batch == 0 || seq_len == 0) return NIMLLM_OK;
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        return fail(NIMLLM_ERR_ARG, "attn_prefill: q, k, v, out must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;

    if (dtype == NIMLLM_F32) {
        // pre-pass: RoPE on q and k in place (the reference's ropeFwd pair) + optional cache fill
        if (rope_cos || k_cache) {
            int rc = nimllm_rope_append(rope_cos ? q : nullptr, n_head, k, v, dtype, 1, rope_cos, rope_sin, nullptr,
                                        pos0, k_cache, v_cache, cache_dtype, kv_off, seq_stride, head_stride, 0,
                                        max_seq, batch, seq_len, n_kv_head, head_dim, stream);
            if (rc) return rc;
        }
        return launch_prefill_f32((const float *)q, (const float *)k, (const float *)v, (float *)out, lse, batch,
                                  seq_len, n_head, n_kv_head, head_dim, scale, 1, st);
    }
    // bf16: K is rotated (and the cache filled) by the pre-pass; q is rotated inside the
    // tensor-core kernel's prologue and written back only when save_cache asks for it.
    if (rope_cos || k_cache) {
        int rc = nimllm_rope_append(nullptr, n_head, k, v, dtype, 1, rope_cos, rope_sin, nullptr, pos0, k_cache,
                                    v_cache, cache_dtype, kv_off, seq_stride, head_stride, 0, max_seq, batch,
                                    seq_len, n_kv_head, head_dim, stream);
        if (rc) return rc;
    }
    (void)workspace; (void)workspace_bytes;
    return launch_prefill_tc(q, k, v, out, lse, rope_cos, rope_sin, pos0, save_cache ? 1 : 0, batch, seq_len,
                             n_head, n_kv_head, head_dim, scale, st);
}

int nimllm_attn_prefill_status(int reset) {
    int st = 0;
    const int rc = prefill_tc_status(reset, &st);
    return rc ? -rc : st;
}

}  // extern "C"
