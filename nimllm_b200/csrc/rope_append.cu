// rope_append.cu -- one launch for everything the reference does between the QKV
// projections and the attention loop: RoPE on q and on the new K rows
// (src/model.nim:494-495 / 790-797 via src/kernels.cu:399-423) and the copy of the new
// K/V rows into the cache (src/model.nim:799-815: 2*Hkv cudaMemcpy D2D per token, or
// gpu_extract_kv_head for several), with the cast to the cache's element type folded in.
//
// HBM-bound elementwise work: one thread moves 4 + 4 elements (the rotation pair
// f..f+3 and f+D/2..f+D/2+3) with 16-byte (fp32) or 8-byte (bf16) accesses.
#include "common.cuh"

namespace nimllm {

namespace {

struct RopeAppendParams {
    void *q;
    void *k_new;
    const void *v_new;
    const float *cos_tab, *sin_tab;
    const int32_t *seq_pos;
    void *k_cache, *v_cache;
    const int64_t *kv_off;
    int64_t seq_stride, head_stride;
    int pos0, cache_row0, max_seq;
    int B, n, Hq, Hkv, D;
    int write_back_k;
    // paged cache (page_table != null): page_table [B, max_pages] -> page of page_rows rows,
    // pages [n_pages][Hkv][page_rows][D]; kv_off / strides / cache_row0 are not used then
    const int32_t *page_table;
    int max_pages, page_shift, n_pages;
};

template <typename T> __device__ __forceinline__ void load4(const T *p, float *f);
template <> __device__ __forceinline__ void load4<float>(const float *p, float *f) {
    float4 v = *reinterpret_cast<const float4 *>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16 *p, float *f) {
    uint2 v = *reinterpret_cast<const uint2 *>(p);
    f[0] = bf16lo(v.x); f[1] = bf16hi(v.x); f[2] = bf16lo(v.y); f[3] = bf16hi(v.y);
}
template <typename T> __device__ __forceinline__ void store4(T *p, const float *f);
template <> __device__ __forceinline__ void store4<float>(float *p, const float *f) {
    *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *p, const float *f) {
    uint2 v;
    v.x = pack_bf16(f[0], f[1]);
    v.y = pack_bf16(f[2], f[3]);
    *reinterpret_cast<uint2 *>(p) = v;
}

// Work item = (sequence b, token t, slot, group of 4 frequencies).  Slots 0..Hq-1 are
// the query heads, Hq..Hq+Hkv-1 the K heads, the last Hkv the V heads.
template <typename ActT, typename CacheT>
__global__ void __launch_bounds__(256) rope_append_kernel(RopeAppendParams p) {
    const int half = p.D / 2;
    const int f4_per_head = half / 4;
    const int n_q = p.q ? p.Hq : 0;
    const int slots = n_q + p.Hkv + (p.k_cache ? p.Hkv : 0);    // V rows only move when there is a cache
    const int64_t total = (int64_t)p.B * p.n * slots * f4_per_head;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        int f = (int)(idx % f4_per_head) * 4;
        int64_t r = idx / f4_per_head;
        int slot = (int)(r % slots);
        r /= slots;
        int t = (int)(r % p.n);
        int b = (int)(r / p.n);
        int pos = (p.seq_pos ? p.seq_pos[b] : p.pos0) + t;

        const bool is_q = slot < n_q;
        const bool is_k = !is_q && slot < n_q + p.Hkv;
        const int head = is_q ? slot : (is_k ? slot - n_q : slot - n_q - p.Hkv);
        const int row_w = is_q ? p.Hq * p.D : p.Hkv * p.D;
        ActT *src = reinterpret_cast<ActT *>(is_q ? p.q : (is_k ? p.k_new : const_cast<void *>(p.v_new)));
        ActT *x = src + ((int64_t)b * p.n + t) * row_w + (int64_t)head * p.D + f;

        float x0[4], x1[4];
        load4<ActT>(x, x0);
        load4<ActT>(x + half, x1);
        if ((is_q || is_k) && p.cos_tab) {
            float c[4], s[4];
            load4<float>(p.cos_tab + (int64_t)pos * half + f, c);
            load4<float>(p.sin_tab + (int64_t)pos * half + f, s);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                // the expression of src/kernels.cu:412-413 with sign = +1
                float a = x0[i] * c[i] - x1[i] * s[i];
                float d = x0[i] * s[i] + x1[i] * c[i];
                x0[i] = a;
                x1[i] = d;
            }
            if (is_q || p.write_back_k) {
                store4<ActT>(x, x0);
                store4<ActT>(x + half, x1);
            }
        }
        if (!is_q && p.k_cache && p.page_table) {
            // every row finds its own page: an append may cross page boundaries; rows past the
            // table, unassigned entries (< 0) and pages outside the pool are not stored
            const int pr = pos >> p.page_shift;
            if (pos >= 0 && pr < p.max_pages) {
                const int pg = p.page_table[(int64_t)b * p.max_pages + pr];
                if (pg >= 0 && pg < p.n_pages) {
                    const int64_t base = (((int64_t)pg * p.Hkv + head) << p.page_shift) * p.D +
                                         (int64_t)(pos & ((1 << p.page_shift) - 1)) * p.D + f;
                    CacheT *dst = reinterpret_cast<CacheT *>(is_k ? p.k_cache : p.v_cache) + base;
                    store4<CacheT>(dst, x0);
                    store4<CacheT>(dst + half, x1);
                }
            }
        } else if (!is_q && p.k_cache) {
            int row = pos - p.cache_row0;
            if (row >= 0 && row < p.max_seq) {
                int64_t base = (p.kv_off ? p.kv_off[b] : (int64_t)b * p.seq_stride) +
                               (int64_t)head * p.head_stride + (int64_t)row * p.D + f;
                CacheT *dst = reinterpret_cast<CacheT *>(is_k ? p.k_cache : p.v_cache) + base;
                store4<CacheT>(dst, x0);
                store4<CacheT>(dst + half, x1);
            }
        }
    }
}

}  // namespace

int launch_rope_append(void *q, int Hq, void *k_new, const void *v_new, int act_dtype,
                       int write_back_k, const float *cos_tab, const float *sin_tab,
                       const int32_t *seq_pos, int pos0, void *k_cache, void *v_cache,
                       int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                       int64_t head_stride, int cache_row0, int max_seq, int B, int n, int Hkv,
                       int D, cudaStream_t st, const int32_t *page_table, int max_pages, int page_shift,
                       int n_pages) {
    RopeAppendParams p;
    p.page_table = page_table; p.max_pages = max_pages; p.page_shift = page_shift; p.n_pages = n_pages;
    p.q = q; p.k_new = k_new; p.v_new = v_new;
    p.cos_tab = cos_tab; p.sin_tab = sin_tab; p.seq_pos = seq_pos;
    p.k_cache = k_cache; p.v_cache = v_cache; p.kv_off = kv_off;
    p.seq_stride = seq_stride; p.head_stride = head_stride;
    p.pos0 = pos0; p.cache_row0 = cache_row0; p.max_seq = max_seq;
    p.B = B; p.n = n; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.write_back_k = write_back_k;

    int64_t total = (int64_t)B * n * ((q ? Hq : 0) + Hkv + (k_cache ? Hkv : 0)) * (D / 8);
    if (total == 0) return NIMLLM_OK;
    int64_t blocks = (total + 255) / 256;
    int64_t cap = (int64_t)sm_count() * 16;
    int grid = (int)(blocks < cap ? blocks : cap);
    if (act_dtype == NIMLLM_F32 && cache_dtype == NIMLLM_F32)
        rope_append_kernel<float, float><<<grid, 256, 0, st>>>(p);
    else if (act_dtype == NIMLLM_F32)
        rope_append_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>(p);
    else if (cache_dtype == NIMLLM_F32)
        rope_append_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(p);
    else
        rope_append_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(p);
    NIMLLM_CHECK_LAUNCH("rope_append");
    return NIMLLM_OK;
}

}  // namespace nimllm
