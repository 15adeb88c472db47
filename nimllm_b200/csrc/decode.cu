// decode.cu -- GQA decode attention over a KV cache (HBM-bound).
//
// Replaces the per-query-head loop of src/model.nim:822-840 (per head: cublasSgemm_v2
// [1,D]x[L,D]^T, gpu_scale, gpu_softmax_fwd, cublasSgemm_v2 [1,L]x[L,D]).  One CTA owns
// one (sequence, KV head, chunk of KV rows) and serves ALL query heads of that KV head,
// so every cached K and V row is fetched from HBM once (the reference re-reads it once
// per query head).  Chunks produce (max, sum, output) partials that are merged by
// log-sum-exp -- in this file for the chunks of one GPU, and through the same combine
// kernel for KV-sequence shards gathered from other GPUs.
//
// Two kernels:
//   decode_mma_kernel      bf16 cache.  The G (<= 8) query heads are the rows of a 16-row
//                          A operand of mma.sync.m16n8k16; K rows are the B operand of
//                          Q K^T and V rows the B operand of P V.  Each lane fetches its
//                          fragments straight from global memory with 16-byte loads: the
//                          contraction index of Q K^T and the output column of P V may be
//                          permuted freely, and the permutations below are chosen so that
//                          a lane's 16 contiguous bytes are exactly what its fragments
//                          need (K) or need after one byte-permute (V).
//   decode_generic_kernel  fp32 or bf16 cache, fp32 FMA on the CUDA cores: the <= 1e-4
//                          parity path for the reference's fp32 cache, and the fallback
//                          for group sizes the mma kernel does not take.
#include <atomic>

#include "common.cuh"

namespace nimllm {

namespace {

constexpr int kWarps = 4;

struct DecodeParams {
    const void *q;
    const void *k, *v;
    const int64_t *kv_off;
    int64_t seq_stride, head_stride;
    const int32_t *seq_len;
    void *out;
    float *partials_out;
    float *ws;               // partial records of split sequences
    int q_dtype, out_dtype;
    int max_len, chunk_rows;
    int B, Hq, Hkv, G;
    float scale_log2e;
    // paged cache (balanced kernel only): page_table [B, max_pages] -> page index; a page is
    // [Hkv][page_rows][D] elements of K (and of V), page_rows = 1 << page_shift
    const int32_t *page_table;
    int max_pages, page_shift;
    int64_t page_stride;
};

__device__ __forceinline__ int seq_rows(const DecodeParams &p, int b) {
    int L = p.seq_len ? p.seq_len[b] : p.max_len;
    return L < 0 ? 0 : (L > p.max_len ? p.max_len : L);
}

// Final write of one (sequence, query head, column): either the finished output (single
// chunk) or a partial record for the combine kernel.
__device__ __forceinline__ void emit(const DecodeParams &p, int D, int b, int hq, int chunk,
                                     int n_chunks, int d, float o, float l, float m2) {
    const int W = rec_stride(D);
    const float val = l > 0.f ? o / l : 0.f;
    const int64_t row = (int64_t)b * p.Hq + hq;
    if (n_chunks <= 1) {
        if (p.out) store_from_f32(p.out, p.out_dtype, row * D + d, val);
        if (p.partials_out) {
            float *rec = p.partials_out + row * W;
            rec[d] = val;
            if (d == 0) { rec[D] = m2 * kLn2; rec[D + 1] = l; rec[D + 2] = 0.f; rec[D + 3] = 0.f; }
        }
    } else {
        float *rec = p.ws + ((int64_t)chunk * p.B * p.Hq + row) * W;
        rec[d] = val;
        if (d == 0) { rec[D] = m2 * kLn2; rec[D + 1] = l; rec[D + 2] = 0.f; rec[D + 3] = 0.f; }
    }
}

// Merge of the per-warp states left in shared memory (NH heads, D columns).  (Letting the
// last-arriving CTA of a split sequence merge the chunks in-kernel was measured slower than
// the separate combine launch: its serial tail costs more than the launch it saves.)
template <int D, int NW = kWarps>
__device__ __forceinline__ void merge_warps_and_emit(const DecodeParams &p, const float *sm_m,
                                                     const float *sm_l, const float *sm_o,
                                                     int nh_stride, int nh, int b, int hq0,
                                                     int chunk, int n_chunks) {
    for (int idx = threadIdx.x; idx < nh * D; idx += NW * 32) {
        int g = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, sm_m[w * nh_stride + g]);
        float safe = (M == -INFINITY) ? 0.f : M;
        float l = 0.f, o = 0.f;
#pragma unroll
        for (int w = 0; w < NW; w++) {
            float c = ex2(sm_m[w * nh_stride + g] - safe);
            l += sm_l[w * nh_stride + g] * c;
            o += sm_o[((size_t)w * nh_stride + g) * D + d] * c;
        }
        emit(p, D, b, hq0 + g, chunk, n_chunks, d, o, l, M);
    }
}

// ------------------------------------------------------------------ generic kernel
// Lane groups of LPR lanes own one KV row at a time (16 bytes per lane); every group
// keeps its own online-softmax state for the GT query heads and the states are merged
// at the end (lane groups by shuffles, warps through shared memory).
template <typename T, int D, int GT>
__global__ void __launch_bounds__(kWarps * 32) decode_generic_kernel(DecodeParams p) {
    constexpr int VEC = Elem<T>::kVec;
    constexpr int LPR = D / VEC;        // lanes per row
    constexpr int RPW = 32 / LPR;       // rows per warp step
    constexpr int NWK = kWarps * RPW;   // row workers per CTA
    constexpr int U = 4;                // rows in flight per worker
    static_assert(LPR <= 32 && LPR >= 1, "head_dim too large for one warp");

    __shared__ float sm_m[kWarps * GT], sm_l[kWarps * GT];
    __shared__ float sm_o[kWarps * GT * D];

    const int b = blockIdx.z, chunk = blockIdx.x;
    const int groups = (p.G + GT - 1) / GT;
    const int kvh = blockIdx.y / groups, grp = blockIdx.y % groups;
    const int L = seq_rows(p, b);
    const int n_chunks = L <= p.chunk_rows ? 1 : (L + p.chunk_rows - 1) / p.chunk_rows;
    if (chunk >= n_chunks) return;
    const int r0 = chunk * p.chunk_rows;
    const int r1 = min(L, r0 + p.chunk_rows);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lir = lane % LPR, rw = lane / LPR;
    const int g0 = grp * GT;
    const int ng = min(GT, p.G - g0);
    const int hq0 = kvh * p.G + g0;
    const int E = p.Hq * D;

    float qr[GT][VEC];
#pragma unroll
    for (int g = 0; g < GT; g++)
#pragma unroll
        for (int i = 0; i < VEC; i++)
            qr[g][i] = g < ng ? load_as_f32(p.q, p.q_dtype, (int64_t)b * E + (int64_t)(hq0 + g) * D + lir * VEC + i) *
                                    p.scale_log2e
                              : 0.f;

    float m[GT], l[GT], acc[GT][VEC];
#pragma unroll
    for (int g = 0; g < GT; g++) {
        m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; i++) acc[g][i] = 0.f;
    }

    const int64_t base = (p.kv_off ? p.kv_off[b] : (int64_t)b * p.seq_stride) + (int64_t)kvh * p.head_stride + lir * VEC;
    const T *kb = reinterpret_cast<const T *>(p.k) + base;
    const T *vb = reinterpret_cast<const T *>(p.v) + base;

    // rb is warp-uniform (the shuffles below need the whole warp in the loop); lane group rw
    // of warp w owns rows rb + rw + u*NWK
    for (int rb = r0 + warp * RPW; rb < r1; rb += NWK * U) {
        uint4 kx[U], vx[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            int row = min(rb + rw + u * NWK, r1 - 1);
            kx[u] = ldg_stream(kb + (int64_t)row * D);
            vx[u] = ldg_stream(vb + (int64_t)row * D);
        }
        float s[U][GT];
#pragma unroll
        for (int u = 0; u < U; u++) {
            float kf[VEC];
            Elem<T>::unpack(kx[u], kf);
#pragma unroll
            for (int g = 0; g < GT; g++) {
                float a = 0.f;
#pragma unroll
                for (int i = 0; i < VEC; i++) a = fmaf(qr[g][i], kf[i], a);
                s[u][g] = a;
            }
        }
#pragma unroll
        for (int off = LPR / 2; off > 0; off >>= 1)
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int g = 0; g < GT; g++) s[u][g] += __shfl_xor_sync(0xffffffffu, s[u][g], off);
        float pr[U][GT];
#pragma unroll
        for (int g = 0; g < GT; g++) {
            float mx = -INFINITY;
#pragma unroll
            for (int u = 0; u < U; u++) {
                if (rb + rw + u * NWK >= r1) s[u][g] = -INFINITY;
                mx = fmaxf(mx, s[u][g]);
            }
            float m_new = fmaxf(m[g], mx);
            float safe = (m_new == -INFINITY) ? 0.f : m_new;
            float corr = ex2(m[g] - safe);
            float sum = 0.f;
#pragma unroll
            for (int u = 0; u < U; u++) { pr[u][g] = ex2(s[u][g] - safe); sum += pr[u][g]; }
            l[g] = l[g] * corr + sum;
            m[g] = m_new;
#pragma unroll
            for (int i = 0; i < VEC; i++) acc[g][i] *= corr;
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            float vf[VEC];
            Elem<T>::unpack(vx[u], vf);
#pragma unroll
            for (int g = 0; g < GT; g++)
#pragma unroll
                for (int i = 0; i < VEC; i++) acc[g][i] = fmaf(pr[u][g], vf[i], acc[g][i]);
        }
    }

    // merge the RPW lane groups of this warp
#pragma unroll
    for (int off = LPR; off < 32; off <<= 1) {
#pragma unroll
        for (int g = 0; g < GT; g++) {
            float mo = __shfl_xor_sync(0xffffffffu, m[g], off);
            float lo = __shfl_xor_sync(0xffffffffu, l[g], off);
            float m_new = fmaxf(m[g], mo);
            float safe = (m_new == -INFINITY) ? 0.f : m_new;
            float ca = ex2(m[g] - safe), cb = ex2(mo - safe);
            l[g] = l[g] * ca + lo * cb;
            m[g] = m_new;
#pragma unroll
            for (int i = 0; i < VEC; i++) {
                float ao = __shfl_xor_sync(0xffffffffu, acc[g][i], off);
                acc[g][i] = acc[g][i] * ca + ao * cb;
            }
        }
    }
    if (rw == 0) {
#pragma unroll
        for (int g = 0; g < GT; g++) {
            if (lir == 0) { sm_m[warp * GT + g] = m[g]; sm_l[warp * GT + g] = l[g]; }
#pragma unroll
            for (int i = 0; i < VEC; i++) sm_o[(warp * GT + g) * D + lir * VEC + i] = acc[g][i];
        }
    }
    __syncthreads();
    merge_warps_and_emit<D>(p, sm_m, sm_l, sm_o, GT, ng, b, hq0, chunk, n_chunks);
}

// ---------------------------------------------------------------------- mma kernel
__device__ __forceinline__ void mma_bf16_16816(float &d0, float &d1, uint32_t a0, uint32_t a2,
                                               uint32_t b0, uint32_t b1) {
    // rows 8..15 of A are zero padding (a1 = a3 = 0); their outputs are discarded
    float d2, d3;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%10,%10};"
        : "+f"(d0), "+f"(d1), "=f"(d2), "=f"(d3)
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

template <int D> struct KvFrag {
    uint32_t k[2][D / 32][4];  // [row tile][32-column chunk][16 bytes]
    uint32_t v[4][D / 64][4];  // [row 2t, 2t+1, 2t+8, 2t+9][64-column half][16 bytes]
};

// Lane (g = lane/4, t = lane%4) of a warp working on the 16 rows starting at rb.
//  K: rows rb+g and rb+8+g, columns c*32 + t*8 .. +7     (B operand of Q K^T, n = g)
//  V: rows rb+2t, +2t+1, +2t+8, +2t+9, columns h*64 + g*8 .. +7  (B operand of P V)
// Rows past the end of the chunk are clamped (their probabilities are forced to 0).
template <int D>
__device__ __forceinline__ void load_frag(KvFrag<D> &f, const __nv_bfloat16 *kb,
                                          const __nv_bfloat16 *vb, int rb, int r_last, int g, int t) {
#pragma unroll
    for (int nt = 0; nt < 2; nt++) {
        int row = min(rb + nt * 8 + g, r_last);
#pragma unroll
        for (int c = 0; c < D / 32; c++) {
            uint4 x = ldg_stream(kb + (int64_t)row * D + c * 32 + t * 8);
            f.k[nt][c][0] = x.x; f.k[nt][c][1] = x.y; f.k[nt][c][2] = x.z; f.k[nt][c][3] = x.w;
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        int row = min(rb + 2 * t + (i & 1) + (i >> 1) * 8, r_last);
#pragma unroll
        for (int h = 0; h < D / 64; h++) {
            uint4 x = ldg_stream(vb + (int64_t)row * D + h * 64 + g * 8);
            f.v[i][h][0] = x.x; f.v[i][h][1] = x.y; f.v[i][h][2] = x.z; f.v[i][h][3] = x.w;
        }
    }
}

template <int D>
__device__ __forceinline__ void consume_frag(const KvFrag<D> &f, const uint32_t (*qreg)[4],
                                             float (*o)[2], float &m, float &l, int rb, int r1,
                                             int t, float scale_log2e) {
    // scores: head g (row of A), KV rows rb + nt*8 + 2t + {0,1}
    float s[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int c = 0; c < D / 32; c++)
#pragma unroll
            for (int j = 0; j < 2; j++)
                mma_bf16_16816(s[nt][0], s[nt][1], qreg[c][2 * j], qreg[c][2 * j + 1],
                               f.k[nt][c][2 * j], f.k[nt][c][2 * j + 1]);
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
            int row = rb + nt * 8 + 2 * t + e;
            s[nt][e] = row < r1 ? s[nt][e] * scale_log2e : -INFINITY;
            mx = fmaxf(mx, s[nt][e]);
        }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    float m_new = fmaxf(m, mx);
    float safe = (m_new == -INFINITY) ? 0.f : m_new;
    float corr = ex2(m - safe);
    float p00 = ex2(s[0][0] - safe), p01 = ex2(s[0][1] - safe);
    float p10 = ex2(s[1][0] - safe), p11 = ex2(s[1][1] - safe);
    l = l * corr + (p00 + p01) + (p10 + p11);
    m = m_new;
    const uint32_t pa0 = pack_bf16(p00, p01);  // k slots 2t, 2t+1   <-> rows rb+2t, rb+2t+1
    const uint32_t pa2 = pack_bf16(p10, p11);  // k slots 2t+8, 2t+9 <-> rows rb+8+2t, rb+9+2t
#pragma unroll
    for (int h = 0; h < D / 64; h++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
            uint32_t b0 = prmt(f.v[0][h][j >> 1], f.v[1][h][j >> 1], sel);
            uint32_t b1 = prmt(f.v[2][h][j >> 1], f.v[3][h][j >> 1], sel);
            float *acc = o[h * 8 + j];
            acc[0] *= corr;
            acc[1] *= corr;
            mma_bf16_16816(acc[0], acc[1], pa0, pa2, b0, b1);
        }
}

// MINB = resident CTAs per SM the register budget is held to.
// BLK = 16-row blocks per prefetched fragment set: what a lane keeps in flight is BLK * D/8
// 16-byte loads; 8 KiB per warp (BLK = 2 at D = 64, 1 at D = 128) is what it takes to approach
// the HBM rate with 8 warps per SM.
template <int D, int MINB, int BLK, int NW>
__global__ void __launch_bounds__(NW * 32, MINB) decode_mma_kernel(DecodeParams p) {
    constexpr int NH = 8;  // head rows kept (G <= 8)
    __shared__ float sm_m[NW * NH], sm_l[NW * NH];
    __shared__ float sm_o[NW * NH * D];

    const int b = blockIdx.z, chunk = blockIdx.x, kvh = blockIdx.y;
    const int L = seq_rows(p, b);
    const int n_chunks = L <= p.chunk_rows ? 1 : (L + p.chunk_rows - 1) / p.chunk_rows;
    if (chunk >= n_chunks) return;
    const int r0 = chunk * p.chunk_rows;
    const int r1 = min(L, r0 + p.chunk_rows);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int E = p.Hq * D;
    const int hq0 = kvh * p.G;

    float o[D / 8][2];
#pragma unroll
    for (int i = 0; i < D / 8; i++) { o[i][0] = 0.f; o[i][1] = 0.f; }
    float m = -INFINITY, l = 0.f;

    const int64_t base = (p.kv_off ? p.kv_off[b] : (int64_t)b * p.seq_stride) + (int64_t)kvh * p.head_stride;
    const __nv_bfloat16 *kb = reinterpret_cast<const __nv_bfloat16 *>(p.k) + base;
    const __nv_bfloat16 *vb = reinterpret_cast<const __nv_bfloat16 *>(p.v) + base;

    constexpr int STEP = NW * 16 * BLK;
    int rb = r0 + warp * 16 * BLK;
    KvFrag<D> fa[BLK], fb[BLK];
    uint32_t qreg[D / 32][4];
    auto load = [&](KvFrag<D> *f, int row) {
#pragma unroll
        for (int u = 0; u < BLK; u++) load_frag<D>(f[u], kb, vb, row + u * 16, r1 - 1, g, t);
    };
    auto consume = [&](const KvFrag<D> *f, int row) {
#pragma unroll
        for (int u = 0; u < BLK; u++) consume_frag<D>(f[u], qreg, o, m, l, row + u * 16, r1, t, p.scale_log2e);
    };
    // A operand: Q[head g][c*32 + t*8 .. +7] as bf16 pairs (zero for padding heads)
#pragma unroll
    for (int c = 0; c < D / 32; c++) {
        float x[8];
#pragma unroll
        for (int i = 0; i < 8; i++)
            x[i] = g < p.G ? load_as_f32(p.q, p.q_dtype, (int64_t)b * E + (int64_t)(hq0 + g) * D + c * 32 + t * 8 + i)
                           : 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) qreg[c][i] = pack_bf16(x[2 * i], x[2 * i + 1]);
    }
    if (rb < r1) load(fa, rb);
    while (rb < r1) {
        if (rb + STEP < r1) load(fb, rb + STEP);
        consume(fa, rb);
        rb += STEP;
        if (rb >= r1) break;
        if (rb + STEP < r1) load(fa, rb + STEP);
        consume(fb, rb);
        rb += STEP;
    }

    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (t == 0) { sm_m[warp * NH + g] = m; sm_l[warp * NH + g] = l; }
    // accumulator tile h*8+j, element e  <->  column h*64 + (2t+e)*8 + j
#pragma unroll
    for (int h = 0; h < D / 64; h++)
#pragma unroll
        for (int j = 0; j < 8; j++)
#pragma unroll
            for (int e = 0; e < 2; e++)
                sm_o[(warp * NH + g) * D + h * 64 + (2 * t + e) * 8 + j] = o[h * 8 + j][e];
    __syncthreads();
    merge_warps_and_emit<D, NW>(p, sm_m, sm_l, sm_o, NH, p.G, b, hq0, chunk, n_chunks);
}

// ------------------------------------------------------- balanced mma kernel (no chunk grid)
// The grid above gives every (sequence, KV head, chunk) its own CTA: a batch is a few rounds of
// CTAs, and every round pays the start-up of a CTA again (sequence length -> offsets -> q ->
// first rows: about 3.3 us per round measured on B200) plus the ragged tail of unequal lengths.
// Here the whole batch is ONE flattened list of row units (U = 16 * BLK rows), ordered by
// sequence, KV head, row; it is cut into as many equal spans as there are warps in a grid that
// fills the GPU exactly once, and every warp streams its own span on its own:
//   * one start-up per launch instead of one per round, no tail, no block-level barrier after
//     the prefix sum;
//   * a span may cover the end of one (sequence, KV head) pair, any number of whole pairs and
//     the start of another.  Whole pairs are written out directly; the at most two cut pairs of
//     a warp go to the warp's two record slots, and combine_balanced_kernel merges the pieces of
//     every cut pair (the warps holding them are consecutive, so it finds them by arithmetic).
constexpr int kBalMaxB = 4096;      // sequences whose unit counts fit the shared-memory prefix
constexpr int kBalMinUnits = 4;     // a warp gets at least this many units (small batches use fewer warps)

// warp w of wa owns units [w*T/wa, (w+1)*T/wa); the warp owning unit u:
__host__ __device__ __forceinline__ int64_t bal_first_unit(int w, int64_t T, int wa) { return (int64_t)w * T / wa; }
__host__ __device__ __forceinline__ int bal_owner(int64_t u, int64_t T, int wa) { return (int)(((u + 1) * wa - 1) / T); }
__host__ __device__ __forceinline__ int bal_active_warps(int64_t T, int wk) {
    int64_t a = T / kBalMinUnits;
    return (int)(a < 1 ? 1 : (a > wk ? wk : a));
}

// Walk of one warp's span, segment by segment.  `cum(b)` = units of one KV head of the sequences
// before b.  The position is kept as (sequence, KV head, unit) so the loop carries no 64-bit state.
// Shared by the kernel and by the host-side plan used in the CPU tests.
struct BalWalk {
    int b, kvh, i0, remaining;
    bool first;
};
struct BalSeg {
    int b, kvh, i0, i1, nb, slot;      // units [i0, i1) of the pair's nb; record slot when the pair is cut
    bool whole;
};
template <typename CumFn>
__host__ __device__ __forceinline__ void bal_walk_init(BalWalk &wk, int64_t u0, int64_t u1, int B, int Hkv, CumFn cum) {
    int lo = 0, hi = B - 1;            // largest b whose first unit is at or before u0 (it is not empty)
    while (lo < hi) {
        int mid = (lo + hi + 1) >> 1;
        if ((int64_t)Hkv * cum(mid) <= u0) lo = mid; else hi = mid - 1;
    }
    wk.b = lo;
    wk.remaining = (int)(u1 - u0);
    wk.first = true;
    wk.kvh = 0; wk.i0 = 0;
    if (wk.remaining > 0) {
        const int nb0 = cum(lo + 1) - cum(lo);
        const int64_t within = u0 - (int64_t)Hkv * cum(lo);
        wk.kvh = (int)(within / nb0);
        wk.i0 = (int)(within % nb0);
    }
}
template <typename CumFn>
__host__ __device__ __forceinline__ bool bal_walk_next(BalWalk &wk, int Hkv, CumFn cum, BalSeg &sg) {
    while (wk.remaining > 0) {
        const int nb = cum(wk.b + 1) - cum(wk.b);
        if (wk.kvh >= Hkv || nb == 0) { wk.b++; wk.kvh = 0; wk.i0 = 0; continue; }
        sg.b = wk.b; sg.kvh = wk.kvh; sg.i0 = wk.i0; sg.nb = nb;
        sg.i1 = nb < wk.i0 + wk.remaining ? nb : wk.i0 + wk.remaining;
        sg.whole = sg.i0 == 0 && sg.i1 == nb;
        sg.slot = wk.first ? 0 : 1;
        wk.remaining -= sg.i1 - sg.i0;
        wk.first = false;
        wk.i0 = sg.i1;
        if (wk.i0 == nb) { wk.i0 = 0; wk.kvh++; }
        return true;
    }
    return false;
}
// merge side: the consecutive warps holding the pieces of the pair that starts at unit s
__host__ __device__ __forceinline__ void bal_pair_pieces(int64_t s, int nb, int64_t T, int wa, int &w_first, int &n, int &slot_first) {
    w_first = bal_owner(s, T, wa);
    n = bal_owner(s + nb - 1, T, wa) - w_first + 1;
    slot_first = bal_first_unit(w_first, T, wa) < s ? 1 : 0;
}

template <int D, int MINB, int BLK, int NW, bool PAGED>
__global__ void __launch_bounds__(NW * 32, MINB) decode_mma_balanced_kernel(DecodeParams p, int *cum_out) {
    constexpr int U = 16 * BLK;
    constexpr int W = D + 4;
    __shared__ int s_cum[kBalMaxB + 1];
    __shared__ int s_warp[NW];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int n_uniform = (p.max_len + U - 1) / U;
    // Launched as a programmatic dependent of whatever precedes it in the stream: when that kernel
    // lets its dependents go early (this library's merge kernels do), the CTAs of this grid are
    // already in place when it ends.  Nothing is read or written before this wait.
    grid_dependency_wait();
    // the merge kernel that follows is a programmatic dependent in turn: its CTAs may take their
    // places now and wait there for this grid to finish, instead of being launched after it
    launch_dependents();

    if (p.seq_len) {
        // exclusive prefix of the unit counts of the sequences (one KV head's worth)
        const int per = (p.B + NW * 32 - 1) / (NW * 32);
        const int i_beg = min(p.B, (int)threadIdx.x * per), i_end = min(p.B, i_beg + per);
        int sum = 0;
        for (int i = i_beg; i < i_end; i++) sum += (seq_rows(p, i) + U - 1) / U;
        int incl = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int v = __shfl_up_sync(0xffffffffu, incl, off);
            if (lane >= off) incl += v;
        }
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        int excl = incl - sum;
        for (int w2 = 0; w2 < warp; w2++) excl += s_warp[w2];
        for (int i = i_beg; i < i_end; i++) {
            s_cum[i] = excl;
            excl += (seq_rows(p, i) + U - 1) / U;
        }
        if (threadIdx.x == NW * 32 - 1) s_cum[p.B] = excl;
        __syncthreads();
        if (blockIdx.x == 0)
            for (int i = threadIdx.x; i <= p.B; i += NW * 32) cum_out[i] = s_cum[i];
    }
    auto cum = [&](int b) -> int { return p.seq_len ? s_cum[b] : b * n_uniform; };

    const int64_t T = (int64_t)p.Hkv * cum(p.B);
    if (T == 0) return;                                   // every row is written (as zeros) by the combine kernel
    const int wa = bal_active_warps(T, gridDim.x * NW);
    const int w = warp * gridDim.x + blockIdx.x;          // active warps spread over all CTAs
    if (w >= wa) return;
    const int64_t u0 = bal_first_unit(w, T, wa), u1 = bal_first_unit(w + 1, T, wa);

    const int E = p.Hq * D;
    BalWalk walk;
    bal_walk_init(walk, u0, u1, p.B, p.Hkv, cum);
    BalSeg sg;
    while (bal_walk_next(walk, p.Hkv, cum, sg)) {
        const int b = sg.b, kvh = sg.kvh, i0 = sg.i0, i1 = sg.i1;
        const int r0 = i0 * U, r1 = min(seq_rows(p, b), i1 * U);
        const int hq0 = kvh * p.G;
        const int64_t base = (p.kv_off ? p.kv_off[b] : (int64_t)b * p.seq_stride) + (int64_t)kvh * p.head_stride;
        const __nv_bfloat16 *kb = reinterpret_cast<const __nv_bfloat16 *>(p.k) + base;
        const __nv_bfloat16 *vb = reinterpret_cast<const __nv_bfloat16 *>(p.v) + base;

        KvFrag<D> fa[BLK], fb[BLK];
        uint32_t qreg[D / 32][4];
        float o[D / 8][2];
#pragma unroll
        for (int i = 0; i < D / 8; i++) { o[i][0] = 0.f; o[i][1] = 0.f; }
        float m = -INFINITY, l = 0.f;
        // Paged cache: the lanes hold a window of 32 page-table entries of this sequence, so a
        // 16-row block finds its page with a shuffle instead of a dependent global load; the
        // window only moves forward (rows are walked in order).
        int win_first = 0, pt_reg = 0;
        auto load_window = [&](int first) {
            win_first = first;
            const int e = min(first + lane, p.max_pages - 1);
            pt_reg = p.page_table[(int64_t)b * p.max_pages + e];
        };
        if (PAGED) load_window(r0 >> p.page_shift);
        auto load = [&](KvFrag<D> *f, int row) {
#pragma unroll
            for (int x = 0; x < BLK; x++) {
                const int rr = row + x * 16;
                if (PAGED) {
                    const int pg = min(rr, r1 - 1) >> p.page_shift;      // a block past the end reads (clamped) rows of the last page
                    if (pg >= win_first + 32) load_window(pg);
                    const int entry = __shfl_sync(0xffffffffu, pt_reg, pg - win_first);
                    const int64_t off = (int64_t)entry * p.page_stride + ((int64_t)kvh << p.page_shift) * D;
                    const __nv_bfloat16 *kp = reinterpret_cast<const __nv_bfloat16 *>(p.k) + off;
                    const __nv_bfloat16 *vp = reinterpret_cast<const __nv_bfloat16 *>(p.v) + off;
                    load_frag<D>(f[x], kp, vp, rr - (pg << p.page_shift), (r1 - 1) - (pg << p.page_shift), g, t);
                } else {
                    load_frag<D>(f[x], kb, vb, rr, r1 - 1, g, t);
                }
            }
        };
        auto consume = [&](const KvFrag<D> *f, int row) {
#pragma unroll
            for (int x = 0; x < BLK; x++) consume_frag<D>(f[x], qreg, o, m, l, row + x * 16, r1, t, p.scale_log2e);
        };
        int rb = r0;
        load(fa, rb);                                     // in flight together with the q loads below
#pragma unroll
        for (int c = 0; c < D / 32; c++) {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; i++)
                x[i] = g < p.G ? load_as_f32(p.q, p.q_dtype, (int64_t)b * E + (int64_t)(hq0 + g) * D + c * 32 + t * 8 + i)
                               : 0.f;
#pragma unroll
            for (int i = 0; i < 4; i++) qreg[c][i] = pack_bf16(x[2 * i], x[2 * i + 1]);
        }
        while (rb < r1) {
            if (rb + U < r1) load(fb, rb + U);
            consume(fa, rb);
            rb += U;
            if (rb >= r1) break;
            if (rb + U < r1) load(fa, rb + U);
            consume(fb, rb);
            rb += U;
        }

        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const float inv = l > 0.f ? 1.f / l : 0.f;
        if (g < p.G) {
            if (sg.whole) {                               // the whole pair: final result
                const int64_t row = (int64_t)b * p.Hq + hq0 + g;
                // accumulator tile h*8+j, element e  <->  column h*64 + (2t+e)*8 + j
#pragma unroll
                for (int h = 0; h < D / 64; h++)
#pragma unroll
                    for (int e = 0; e < 2; e++)
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int col = h * 64 + (2 * t + e) * 8 + j;
                            const float val = o[h * 8 + j][e] * inv;
                            if (p.out) store_from_f32(p.out, p.out_dtype, row * D + col, val);
                            if (p.partials_out) p.partials_out[row * W + col] = val;
                        }
                if (p.partials_out && t == 0) {
                    float *rec = p.partials_out + row * W;
                    rec[D] = m * kLn2; rec[D + 1] = l; rec[D + 2] = 0.f; rec[D + 3] = 0.f;
                }
            } else {                                      // a piece: slot 0 if it opens the span, else 1
                float *rec = p.ws + (((int64_t)w * 2 + sg.slot) * p.G + g) * W;
#pragma unroll
                for (int h = 0; h < D / 64; h++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        float4 lo4 = make_float4(o[h * 8 + 0][e] * inv, o[h * 8 + 1][e] * inv, o[h * 8 + 2][e] * inv, o[h * 8 + 3][e] * inv);
                        float4 hi4 = make_float4(o[h * 8 + 4][e] * inv, o[h * 8 + 5][e] * inv, o[h * 8 + 6][e] * inv, o[h * 8 + 7][e] * inv);
                        float4 *dst = reinterpret_cast<float4 *>(rec + h * 64 + (2 * t + e) * 8);
                        dst[0] = lo4;
                        dst[1] = hi4;
                    }
                if (t == 0) *reinterpret_cast<float4 *>(rec + D) = make_float4(m * kLn2, l, 0.f, 0.f);
            }
        }
    }
}

struct BalCombineParams {
    const float *recs;
    const int *cum;
    const int32_t *seq_len;
    void *out;
    float *partials_out;
    int out_dtype;
    int B, Hq, Hkv, G, D, W, U, max_len, wk;
    // KV-sequence shards: every finished record also goes to this rank's slot in every peer's
    // exchange buffer (plain stores over NVLink), and the last CTA raises the rank's flag there
    int do_push;
    PeerPush push;
};

// one finished record row -> the local outputs and, when pushing, every peer
struct RowSink {
    const BalCombineParams &c;
    int row;
    unsigned int epoch;
    __device__ __forceinline__ void value(int d, float val) const {
        if (c.out) store_from_f32(c.out, c.out_dtype, (int64_t)row * c.D + d, val);
        if (c.partials_out) c.partials_out[(int64_t)row * c.W + d] = val;
        if (c.do_push)
            for (int r = 0; r < c.push.world; r++) peer_push_slot(c.push, r, epoch)[(int64_t)row * c.W + d] = val;
    }
    __device__ __forceinline__ void stats(float m, float l) const {
        const float4 t = make_float4(m, l, 0.f, 0.f);
        if (c.partials_out) *reinterpret_cast<float4 *>(c.partials_out + (int64_t)row * c.W + c.D) = t;
        if (c.do_push)
            for (int r = 0; r < c.push.world; r++)
                *reinterpret_cast<float4 *>(peer_push_slot(c.push, r, epoch) + (int64_t)row * c.W + c.D) = t;
    }
    // a row the decode kernel finished by itself: only the peers still need it
    __device__ __forceinline__ void forward(int tid, int nthreads) const {
        if (!c.do_push) return;
        const float4 *src = reinterpret_cast<const float4 *>(c.partials_out + (int64_t)row * c.W);
        for (int i = tid; i < c.W / 4; i += nthreads) {
            const float4 t = __ldcg(src + i);
            for (int r = 0; r < c.push.world; r++)
                reinterpret_cast<float4 *>(peer_push_slot(c.push, r, epoch) + (int64_t)row * c.W)[i] = t;
        }
    }
};

// What a merge thread needs to know about its output row (sequence, query head): which records
// hold the pieces of the row's (sequence, KV head) pair.  n = 0: empty sequence, n = 1: one warp
// covered the pair and wrote the row itself.
struct BalRow {
    int g, n, w_first, slot_first;
};
__device__ __forceinline__ BalRow bal_row(const BalCombineParams &c, int row) {
    BalRow r;
    const int b = row / c.Hq, hq = row % c.Hq, kvh = hq / c.G;
    r.g = hq % c.G;
    const int n_uniform = (c.max_len + c.U - 1) / c.U;
    const int cb = c.seq_len ? c.cum[b] : b * n_uniform;
    const int nb = (c.seq_len ? c.cum[b + 1] : (b + 1) * n_uniform) - cb;
    const int64_t T = (int64_t)c.Hkv * (c.seq_len ? c.cum[c.B] : c.B * n_uniform);
    r.n = 0; r.w_first = 0; r.slot_first = 0;
    if (nb > 0)
        bal_pair_pieces((int64_t)c.Hkv * cb + (int64_t)kvh * nb, nb, T, bal_active_warps(T, c.wk), r.w_first, r.n, r.slot_first);
    return r;
}
__device__ __forceinline__ const float *bal_rec(const BalCombineParams &c, const BalRow &r, int i) {
    return c.recs + (((int64_t)(r.w_first + i) * 2 + (i == 0 ? r.slot_first : 0)) * c.G + r.g) * c.W;
}
// zeros (and an empty record) for a row of an empty sequence, written by `nthreads` threads
__device__ __forceinline__ void bal_write_empty(const RowSink &sink, int tid, int nthreads) {
    for (int d = tid; d < sink.c.D; d += nthreads) sink.value(d, 0.f);
    if (tid == 0) sink.stats(-INFINITY, 0.f);
}

// Variant for batches of many pairs cut into few pieces (measured faster there than the
// four-warp CTA per row below): one warp per output row; rows of empty sequences become zeros, rows
// whose pair one warp covered are already final, the others merge the records of the
// consecutive warps that hold their pieces.
__device__ __forceinline__ void combine_row_warp(const BalCombineParams &c, int row, int lane, unsigned int epoch) {
    const RowSink sink{c, row, epoch};
    const BalRow br = bal_row(c, row);
    if (br.n == 0) { bal_write_empty(sink, lane, 32); return; }
    if (br.n == 1) { sink.forward(lane, 32); return; }
    const int n = br.n;
    auto rec_of = [&](int i) -> const float * { return bal_rec(c, br, i); };
    float M = -INFINITY, wsum = 0.f;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.f;
    if (n <= 4) {
        // the usual case (a pair cut once or twice): every load of the merge is issued before
        // anything is computed, so the warp waits for memory once
        float mi[4], li[4], v[4][8];
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const float *r = rec_of(x < n ? x : 0);
            mi[x] = r[c.D];
            li[x] = x < n ? r[c.D + 1] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int d = lane + 32 * j;
                v[x][j] = d < c.D ? r[d] : 0.f;
            }
        }
#pragma unroll
        for (int x = 0; x < 4; x++)
            if (li[x] > 0.f) M = fmaxf(M, mi[x]);
        const float safe = (M == -INFINITY) ? 0.f : M;
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const float wt = li[x] > 0.f ? li[x] * ex2((mi[x] - safe) * kLog2e) : 0.f;
            wsum += wt;
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = fmaf(wt, v[x][j], acc[j]);
        }
    } else {
        for (int i = lane; i < n; i += 32) {
            const float *r = rec_of(i);
            if (r[c.D + 1] > 0.f) M = fmaxf(M, r[c.D]);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        const float safe = (M == -INFINITY) ? 0.f : M;
        for (int i0 = 0; i0 < n; i0 += 32) {
            float w_mine = 0.f;
            if (i0 + lane < n) {
                const float *r = rec_of(i0 + lane);
                const float li = r[c.D + 1];
                w_mine = li > 0.f ? li * ex2((r[c.D] - safe) * kLog2e) : 0.f;
            }
            const int cnt = min(32, n - i0);
            for (int ii = 0; ii < cnt; ii += 4) {
                float v[4][8], wt[4];
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    const bool ok = ii + x < cnt;
                    const float *r = rec_of(i0 + ii + (ok ? x : 0));
                    wt[x] = ok ? __shfl_sync(0xffffffffu, w_mine, (ii + x) & 31) : 0.f;
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int d = lane + 32 * j;
                        v[x][j] = d < c.D ? r[d] : 0.f;
                    }
                }
#pragma unroll
                for (int x = 0; x < 4; x++) {
                    wsum += wt[x];
#pragma unroll
                    for (int j = 0; j < 8; j++) acc[j] = fmaf(wt[x], v[x][j], acc[j]);
                }
            }
        }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int d = lane + 32 * j;
        if (d < c.D) sink.value(d, acc[j] * inv);
    }
    if (lane == 0) sink.stats(M, wsum);
}
__global__ void __launch_bounds__(128) combine_balanced_warp_kernel(BalCombineParams c) {
    launch_dependents();                 // the next kernel of the stream may place its CTAs (it waits for this grid)
    grid_dependency_wait();              // the decode kernel's records and prefix array are complete
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const unsigned int epoch = c.do_push ? peer_push_epoch(c.push) : 0u;
    if (row < c.B * c.Hq) combine_row_warp(c, row, threadIdx.x & 31, epoch);
    if (c.do_push) peer_push_publish(c.push, epoch);
}

// One CTA of four warps per output row (sequence, query head): rows of empty sequences become
// zeros, rows whose pair one warp covered are already final, the others merge the records of the
// consecutive warps that hold their pieces.  Warp k takes pieces k, k+4, ... and loads them
// before the row maximum is known, so the usual row (up to 16 pieces) waits for memory once for
// its indices and once for its records; the four partial sums meet in shared memory.
__device__ __forceinline__ void combine_row_cta(const BalCombineParams &c, int row, unsigned int epoch,
                                                float (*s_acc)[256], float *s_w) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const RowSink sink{c, row, epoch};
    const BalRow br = bal_row(c, row);                    // the same for every thread of the CTA
    if (br.n == 0) { bal_write_empty(sink, threadIdx.x, 128); return; }
    if (br.n == 1) { sink.forward(threadIdx.x, 128); return; }
    const int n = br.n;
    auto rec_of = [&](int i) -> const float * { return bal_rec(c, br, i); };
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.f;
    float wsum = 0.f;
    float mi[4], li[4], v[4][8];
    auto load_batch = [&](int i_base) {
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const int i = i_base + 4 * x;
            const float *r = rec_of(i < n ? i : 0);
            mi[x] = r[c.D];
            li[x] = i < n ? r[c.D + 1] : 0.f;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int d = lane + 32 * j;
                v[x][j] = d < c.D ? r[d] : 0.f;
            }
        }
    };
    load_batch(warp);
    float M = -INFINITY;
    for (int i = lane; i < n; i += 32) {
        const float *r = rec_of(i);
        if (r[c.D + 1] > 0.f) M = fmaxf(M, r[c.D]);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float safe = (M == -INFINITY) ? 0.f : M;
    for (int i_base = warp; i_base < n; i_base += 16) {
        if (i_base != warp) load_batch(i_base);
#pragma unroll
        for (int x = 0; x < 4; x++) {
            const float wt = li[x] > 0.f ? li[x] * ex2((mi[x] - safe) * kLog2e) : 0.f;
            wsum += wt;
#pragma unroll
            for (int j = 0; j < 8; j++) acc[j] = fmaf(wt, v[x][j], acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < 8; j++) s_acc[warp][lane + 32 * j] = acc[j];
    if (lane == 0) s_w[warp] = wsum;
    __syncthreads();
    wsum = (s_w[0] + s_w[1]) + (s_w[2] + s_w[3]);
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    for (int d = threadIdx.x; d < c.D; d += 128)
        sink.value(d, ((s_acc[0][d] + s_acc[1][d]) + (s_acc[2][d] + s_acc[3][d])) * inv);
    if (threadIdx.x == 0) sink.stats(M, wsum);
}
__global__ void __launch_bounds__(128) combine_balanced_kernel(BalCombineParams c) {
    __shared__ float s_acc[4][256];
    __shared__ float s_w[4];
    launch_dependents();                 // the next kernel of the stream may place its CTAs (it waits for this grid)
    grid_dependency_wait();              // the decode kernel's records and prefix array are complete
    const unsigned int epoch = c.do_push ? peer_push_epoch(c.push) : 0u;
    combine_row_cta(c, blockIdx.x, epoch, s_acc, s_w);
    if (c.do_push) peer_push_publish(c.push, epoch);
}

// ------------------------------------------------------------------ combine kernel
// One warp per output row (sequence, query head).  parts[(part * rows + row) * W].
// With seq_len given, the number of parts of a row is the number of chunks of its
// sequence and rows with a single chunk are skipped (the decode kernel already wrote
// them); without it every row merges n_parts records.
struct CombineParams {
    const float *parts;
    const int32_t *seq_len;
    void *out;
    float *partials_out;
    int out_dtype;
    int n_parts, rows, D, W, Hq, chunk_rows, max_len;
};

__global__ void __launch_bounds__(128) combine_kernel(CombineParams p) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= p.rows) return;
    int n = p.n_parts;
    if (p.seq_len) {
        int L = p.seq_len[row / p.Hq];
        L = L < 0 ? 0 : (L > p.max_len ? p.max_len : L);
        n = (L + p.chunk_rows - 1) / p.chunk_rows;
        if (n <= 1) return;
    }
    const int64_t pstride = (int64_t)p.rows * p.W;
    const float *rec = p.parts + (int64_t)row * p.W;
    // lane i holds (m, l) of parts i, i + 32, ...: one latency for all of them instead of a
    // serial walk (the records of a long sequence sit in L2, ~1 us apart when read one by one)
    float M = -INFINITY;
    for (int i = lane; i < n; i += 32) {
        float li = rec[i * pstride + p.D + 1];
        float mi = rec[i * pstride + p.D];
        if (li > 0.f) M = fmaxf(M, mi);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float safe = (M == -INFINITY) ? 0.f : M;
    float acc[8];  // D <= 256
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.f;
    float wsum = 0.f;
    for (int i0 = 0; i0 < n; i0 += 32) {
        float w_mine = 0.f;
        if (i0 + lane < n) {
            const float *r = rec + (int64_t)(i0 + lane) * pstride;
            float li = r[p.D + 1];
            w_mine = li > 0.f ? li * ex2((r[p.D] - safe) * kLog2e) : 0.f;
        }
        const int cnt = min(32, n - i0);
        for (int ii = 0; ii < cnt; ii += 4) {
            // four parts per step: their loads are independent of the weights and of each other
            float v[4][8], w[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const bool ok = ii + u < cnt;
                const float *r = rec + (int64_t)(i0 + ii + (ok ? u : 0)) * pstride;
                w[u] = ok ? __shfl_sync(0xffffffffu, w_mine, (ii + u) & 31) : 0.f;
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    int d = lane + 32 * j;
                    v[u][j] = d < p.D ? r[d] : 0.f;
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                wsum += w[u];
#pragma unroll
                for (int j = 0; j < 8; j++) acc[j] = fmaf(w[u], v[u][j], acc[j]);
            }
        }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        int d = lane + 32 * j;
        if (d < p.D) {
            float val = acc[j] * inv;
            if (p.out) store_from_f32(p.out, p.out_dtype, (int64_t)row * p.D + d, val);
            if (p.partials_out) p.partials_out[(int64_t)row * p.W + d] = val;
        }
    }
    if (p.partials_out && lane == 0) {
        float *o = p.partials_out + (int64_t)row * p.W;
        o[p.D] = M; o[p.D + 1] = wsum; o[p.D + 2] = 0.f; o[p.D + 3] = 0.f;
    }
}

int auto_chunk_rows(int B, int Hkv, int max_len);

// launch shape of the balanced kernel: a grid that fills the GPU exactly once
struct BalShape { int minb, nw, unit, grid; };
BalShape bal_shape(int head_dim) {
    BalShape s;
    s.minb = 1;                          // one CTA of eight warps per SM at both head sizes (two CTAs of four warps were
    s.nw = 8;                            // measured at 128: a 537 MB batch 92.4 -> 90.5 us with eight)
    s.unit = head_dim == 64 ? 32 : 16;
    s.grid = sm_count() * s.minb;
    return s;
}
size_t bal_record_bytes(int n_head, int n_kv_head, int head_dim) {
    BalShape s = bal_shape(head_dim);
    size_t b = (size_t)s.grid * s.nw * 2 * (n_head / n_kv_head) * rec_stride(head_dim) * sizeof(float);
    return (b + 15) / 16 * 16;
}
// 0 when the shape is outside what the balanced kernel takes
size_t bal_workspace_bytes(int batch, int n_head, int n_kv_head, int head_dim, int max_len, bool ragged) {
    if (head_dim != 64 && head_dim != 128) return 0;
    if (n_head % n_kv_head != 0 || n_head / n_kv_head > 8) return 0;
    if (ragged && batch > kBalMaxB) return 0;
    BalShape s = bal_shape(head_dim);
    if ((int64_t)batch * ((max_len + s.unit - 1) / s.unit) >= (1ll << 30)) return 0;
    return bal_record_bytes(n_head, n_kv_head, head_dim) + ((size_t)batch + 1) * sizeof(int);
}
size_t split_workspace_bytes(int batch, int n_head, int n_kv_head, int head_dim, int max_len, int chunk_rows) {
    if (chunk_rows <= 0) chunk_rows = auto_chunk_rows(batch, n_kv_head, max_len);
    int max_chunks = (max_len + chunk_rows - 1) / chunk_rows;
    if (max_chunks <= 1) return 0;
    return (size_t)max_chunks * batch * n_head * rec_stride(head_dim) * sizeof(float);
}


int auto_chunk_rows(int B, int Hkv, int max_len) {
    // enough (sequence, KV head) pairs for a few waves of the ~2 resident CTAs per SM: do not
    // split at all (no partial records, no combine launch; measured best on the ragged batch.
    // Dispatching the CTAs longest-sequence-first was also measured: the in-kernel ranking costs
    // more than the shorter tail saves)
    if ((int64_t)B * Hkv >= (int64_t)sm_count() * 4 && max_len <= 8192) return (max_len + 63) / 64 * 64;
    int64_t total = (int64_t)B * Hkv * max_len;
    // measured on B200: long chunks win (fewer CTA start-ups and partial records) until the
    // grid drops below a few waves of the ~3 resident CTAs per SM
    int64_t target = (int64_t)sm_count() * 8;
    int64_t c = (total + target - 1) / target;
    c = (c + 63) / 64 * 64;
    if (c < 256) c = 256;
    if (c > 4096) c = 4096;
    return (int)c;
}

template <typename T, int D>
void launch_generic(const DecodeParams &p, dim3 grid_base, cudaStream_t st) {
    // GT query heads per CTA; groups > 1 only for G > 4
    int G = p.G;
    if (G == 1) { decode_generic_kernel<T, D, 1><<<grid_base, kWarps * 32, 0, st>>>(p); }
    else if (G == 2) { decode_generic_kernel<T, D, 2><<<grid_base, kWarps * 32, 0, st>>>(p); }
    else if (G == 3) { decode_generic_kernel<T, D, 3><<<grid_base, kWarps * 32, 0, st>>>(p); }
    else {
        dim3 grid = grid_base;
        grid.y *= (G + 3) / 4;
        decode_generic_kernel<T, D, 4><<<grid, kWarps * 32, 0, st>>>(p);
    }
}

// the balanced kernel and its merge launch; p.ws and the prefix array live in `workspace`
int launch_balanced(DecodeParams &p, const int32_t *seq_len, void *out, int out_dtype, float *partials_out, int batch,
                    int n_head, int n_kv_head, int head_dim, int max_len, void *workspace, cudaStream_t st,
                    const PeerPush *push = nullptr) {
    const BalShape bs = bal_shape(head_dim);
    int *cum = reinterpret_cast<int *>(reinterpret_cast<unsigned char *>(workspace) +
                                       bal_record_bytes(n_head, n_kv_head, head_dim));
    const bool paged = p.page_table != nullptr;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(bs.grid); cfg.blockDim = dim3(bs.nw * 32); cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e;
    if (head_dim == 64) {
        if (paged) e = cudaLaunchKernelEx(&cfg, decode_mma_balanced_kernel<64, 1, 2, 8, true>, p, cum);
        else e = cudaLaunchKernelEx(&cfg, decode_mma_balanced_kernel<64, 1, 2, 8, false>, p, cum);
    } else {
        if (paged) e = cudaLaunchKernelEx(&cfg, decode_mma_balanced_kernel<128, 1, 1, 8, true>, p, cum);
        else e = cudaLaunchKernelEx(&cfg, decode_mma_balanced_kernel<128, 1, 1, 8, false>, p, cum);
    }
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_decode balanced: %s", cudaGetErrorString(e));
    BalCombineParams c;
    c.recs = p.ws; c.cum = cum; c.seq_len = seq_len; c.out = out; c.partials_out = partials_out;
    c.out_dtype = out_dtype; c.B = batch; c.Hq = n_head; c.Hkv = n_kv_head; c.G = p.G; c.D = head_dim;
    c.W = rec_stride(head_dim); c.U = bs.unit; c.max_len = max_len; c.wk = bs.grid * bs.nw;
    c.do_push = push ? 1 : 0;
    if (push) c.push = *push; else c.push = PeerPush{nullptr, 0, 0, 0, 0, 0};
    // The merge launch is a programmatic dependent of the decode kernel (its CTAs are placed while
    // the decode still runs and wait for it on the device).  Few pieces per pair (a large batch):
    // one warp per row; many pieces: a CTA per row.
    cfg.blockDim = dim3(128);
    if ((int64_t)c.wk < 4ll * batch * n_kv_head) {
        cfg.gridDim = dim3((batch * n_head + 3) / 4);
        e = cudaLaunchKernelEx(&cfg, combine_balanced_warp_kernel, c);
    } else {
        cfg.gridDim = dim3(batch * n_head);
        e = cudaLaunchKernelEx(&cfg, combine_balanced_kernel, c);
    }
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_decode balanced combine: %s", cudaGetErrorString(e));
    return NIMLLM_OK;
}

}  // namespace

}  // namespace nimllm

using namespace nimllm;

extern "C" {

// Host-side replay of the balanced kernel's work split (no GPU needed): the same
// walk and merge arithmetic the kernels run, for `warps` workers over sequences of `lens` rows.
// segs_out receives (warp, sequence, kv head, first unit, end unit, slot or -1 for a whole pair)
// per segment, pairs_out (first warp, pieces, slot of the first piece) per (sequence, KV head);
// returns the number of segments, or -1 when max_segs is too small.
int nimllm_attn_decode_plan(const int32_t *lens, int batch, int n_kv_head, int unit, int warps,
                                    int32_t *segs_out, int max_segs, int32_t *pairs_out) {
    if (!lens || batch <= 0 || n_kv_head <= 0 || unit <= 0 || warps <= 0) return -1;
    int *cum_v = new int[batch + 1];
    cum_v[0] = 0;
    for (int b = 0; b < batch; b++) cum_v[b + 1] = cum_v[b] + ((lens[b] < 0 ? 0 : lens[b]) + unit - 1) / unit;
    auto cum = [&](int b) -> int { return cum_v[b]; };
    const int64_t T = (int64_t)n_kv_head * cum_v[batch];
    int n_segs = 0;
    if (T > 0) {
        const int wa = bal_active_warps(T, warps);
        for (int w = 0; w < wa && n_segs >= 0; w++) {
            BalWalk walk;
            bal_walk_init(walk, bal_first_unit(w, T, wa), bal_first_unit(w + 1, T, wa), batch, n_kv_head, cum);
            BalSeg sg;
            while (bal_walk_next(walk, n_kv_head, cum, sg)) {
                if (n_segs >= max_segs) { n_segs = -1; break; }
                int32_t *o = segs_out + 6 * n_segs++;
                o[0] = w; o[1] = sg.b; o[2] = sg.kvh; o[3] = sg.i0; o[4] = sg.i1; o[5] = sg.whole ? -1 : sg.slot;
            }
        }
        if (pairs_out)
            for (int b = 0; b < batch; b++)
                for (int h = 0; h < n_kv_head; h++) {
                    int32_t *o = pairs_out + 3 * (b * n_kv_head + h);
                    const int nb = cum_v[b + 1] - cum_v[b];
                    o[0] = o[1] = o[2] = 0;
                    if (nb > 0) {
                        int wf, n, sf;
                        bal_pair_pieces((int64_t)n_kv_head * cum_v[b] + (int64_t)h * nb, nb, T, wa, wf, n, sf);
                        o[0] = wf; o[1] = n; o[2] = sf;
                    }
                }
    }
    delete[] cum_v;
    return n_segs;
}

size_t nimllm_attn_decode_workspace_bytes(int batch, int n_head, int n_kv_head, int head_dim,
                                          int max_len, int chunk_rows) {
    if (batch <= 0 || n_head <= 0 || n_kv_head <= 0 || max_len <= 0) return 0;
    // with chunk_rows = 0 the library picks the kernel: enough for either choice (the balanced
    // kernel keeps two records per warp and the prefix of the sequences' unit counts)
    const size_t split = split_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, chunk_rows);
    if (chunk_rows > 0 || n_head % n_kv_head != 0) return split;
    const size_t bal = bal_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, true);
    return split > bal ? split : bal;
}

int nimllm_attn_decode(const void *q, int q_dtype, const void *k_cache, const void *v_cache,
                       int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                       int64_t head_stride, const int32_t *seq_len, int max_len, void *out,
                       int out_dtype, float *partials_out, int batch, int n_head,
                       int n_kv_head, int head_dim, float scale, int chunk_rows,
                       void *workspace, size_t workspace_bytes, void *stream) {
    if (!q || !k_cache || !v_cache || (!out && !partials_out))
        return fail(NIMLLM_ERR_ARG, "attn_decode: null q / cache / output pointer");
    if (batch <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head != 0 || max_len <= 0)
        return fail(NIMLLM_ERR_ARG, "attn_decode: bad shape B=%d Hq=%d Hkv=%d max_len=%d", batch,
                    n_head, n_kv_head, max_len);
    if (!dtype_ok(q_dtype) || !dtype_ok(cache_dtype) || !dtype_ok(out_dtype))
        return fail(NIMLLM_ERR_ARG, "attn_decode: unknown dtype");
    if (head_dim != 64 && head_dim != 128)
        return fail(NIMLLM_ERR_UNSUPPORTED, "attn_decode: head_dim %d (64 and 128 are built)", head_dim);
    if (chunk_rows < 0 || (chunk_rows > 0 && chunk_rows % 64 != 0))
        return fail(NIMLLM_ERR_ARG, "attn_decode: chunk_rows must be a multiple of 64");
    if (batch > 65535) return fail(NIMLLM_ERR_UNSUPPORTED, "attn_decode: batch %d > 65535", batch);
    if (((uintptr_t)k_cache | (uintptr_t)v_cache) & 15)
        return fail(NIMLLM_ERR_ARG, "attn_decode: cache pointers must be 16-byte aligned");
    {   // rows are read 16 bytes at a time: every (sequence, KV head) block must start on such a boundary
        const int64_t per16 = cache_dtype == NIMLLM_BF16 ? 8 : 4;
        if (head_stride % per16 != 0 || (!kv_off && seq_stride % per16 != 0))
            return fail(NIMLLM_ERR_ARG, "attn_decode: seq_stride and head_stride must be multiples of 16 bytes");
    }
    const bool mma_ok = cache_dtype == NIMLLM_BF16 && n_head / n_kv_head <= 8;
    // The balanced kernel is the default for a bf16 cache when the caller leaves the chunking to
    // the library and the workspace holds its records; an explicit chunk_rows keeps the chunk grid.
    const size_t bal_need = (mma_ok && chunk_rows == 0)
                                ? bal_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, seq_len != nullptr)
                                : 0;
    const bool balanced = bal_need > 0 && workspace && workspace_bytes >= bal_need && !((uintptr_t)workspace & 15);
    if (chunk_rows == 0) chunk_rows = auto_chunk_rows(batch, n_kv_head, max_len);
    const int max_chunks = (max_len + chunk_rows - 1) / chunk_rows;
    const size_t need = balanced ? bal_need : split_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, chunk_rows);
    if (need > 0 && (!workspace || workspace_bytes < need))
        return fail(NIMLLM_ERR_WORKSPACE, "attn_decode: workspace %zu bytes, need %zu", workspace_bytes, need);
    if (need > 0 && ((uintptr_t)workspace & 15))
        return fail(NIMLLM_ERR_ARG, "attn_decode: workspace must be 16-byte aligned");

    DecodeParams p;
    p.q = q; p.k = k_cache; p.v = v_cache; p.kv_off = kv_off;
    p.seq_stride = seq_stride; p.head_stride = head_stride; p.seq_len = seq_len;
    p.out = out; p.partials_out = partials_out;
    p.ws = (float *)workspace;
    p.q_dtype = q_dtype; p.out_dtype = out_dtype; p.max_len = max_len; p.chunk_rows = chunk_rows;
    p.B = batch; p.Hq = n_head; p.Hkv = n_kv_head; p.G = n_head / n_kv_head;
    p.scale_log2e = scale * kLog2e;
    p.page_table = nullptr; p.max_pages = 0; p.page_shift = 0; p.page_stride = 0;
    cudaStream_t st = (cudaStream_t)stream;

    if (balanced) return launch_balanced(p, seq_len, out, out_dtype, partials_out, batch, n_head, n_kv_head, head_dim,
                                         max_len, workspace, st);

    dim3 grid(max_chunks, n_kv_head, batch);
    if (mma_ok) {
        // D = 64: one 8-warp CTA per SM (8 KiB in flight per warp, finer tail than two 4-warp
        // CTAs: measured 0.790 vs 0.783 of the HBM peak on the ragged batch); D = 128: two
        // 4-warp CTAs per SM
        if (head_dim == 64) decode_mma_kernel<64, 1, 2, 8><<<grid, 256, 0, st>>>(p);
        else decode_mma_kernel<128, 2, 1, 4><<<grid, 128, 0, st>>>(p);
    } else if (cache_dtype == NIMLLM_BF16) {
        if (head_dim == 64) launch_generic<__nv_bfloat16, 64>(p, grid, st);
        else launch_generic<__nv_bfloat16, 128>(p, grid, st);
    } else {
        if (head_dim == 64) launch_generic<float, 64>(p, grid, st);
        else launch_generic<float, 128>(p, grid, st);
    }
    NIMLLM_CHECK_LAUNCH("attn_decode");

    if (max_chunks > 1) {
        CombineParams c;
        c.parts = p.ws; c.seq_len = seq_len; c.out = out;
        c.partials_out = partials_out; c.out_dtype = out_dtype;
        c.n_parts = max_chunks; c.rows = batch * n_head; c.D = head_dim;
        c.W = rec_stride(head_dim); c.Hq = n_head; c.chunk_rows = chunk_rows; c.max_len = max_len;
        combine_kernel<<<(c.rows + 3) / 4, 128, 0, st>>>(c);
        NIMLLM_CHECK_LAUNCH("attn_decode combine");
    }
    return NIMLLM_OK;
}

// ---- decode over a paged cache --------------------------------------------------------------
// K and V live in fixed-size pages [Hkv][page_rows][D] handed out by the caller's block manager
// (the multi-turn KV reuse the reference's chat loop wants, src/chat.nim:57,86-91); sequence b's
// rows r*page_rows .. are in page page_table[b][r].  Same balanced kernel, same records and merge.
int nimllm_attn_decode_paged(const void *q, int q_dtype, const void *k_pages, const void *v_pages,
                             const int32_t *page_table, int max_pages, int page_rows, const int32_t *seq_len,
                             int max_len, void *out, int out_dtype, float *partials_out, int batch, int n_head,
                             int n_kv_head, int head_dim, float scale, void *workspace, size_t workspace_bytes,
                             void *stream) {
    if (!q || !k_pages || !v_pages || !page_table || (!out && !partials_out))
        return fail(NIMLLM_ERR_ARG, "attn_decode_paged: null q / pages / page table / output pointer");
    if (batch <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head != 0 || max_len <= 0 || max_pages <= 0)
        return fail(NIMLLM_ERR_ARG, "attn_decode_paged: bad shape B=%d Hq=%d Hkv=%d max_len=%d max_pages=%d", batch,
                    n_head, n_kv_head, max_len, max_pages);
    if (!dtype_ok(q_dtype) || !dtype_ok(out_dtype)) return fail(NIMLLM_ERR_ARG, "attn_decode_paged: unknown dtype");
    if (head_dim != 64 && head_dim != 128)
        return fail(NIMLLM_ERR_UNSUPPORTED, "attn_decode_paged: head_dim %d (64 and 128 are built)", head_dim);
    if (n_head / n_kv_head > 8) return fail(NIMLLM_ERR_UNSUPPORTED, "attn_decode_paged: Hq/Hkv > 8");
    int shift = 0;
    while ((1 << shift) < page_rows) shift++;
    if (page_rows < 32 || (1 << shift) != page_rows)
        return fail(NIMLLM_ERR_ARG, "attn_decode_paged: page_rows %d must be a power of two >= 32", page_rows);
    if ((int64_t)max_pages * page_rows < max_len)
        return fail(NIMLLM_ERR_ARG, "attn_decode_paged: %d pages of %d rows cannot hold max_len %d", max_pages, page_rows, max_len);
    const size_t need = bal_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, seq_len != nullptr);
    if (need == 0) return fail(NIMLLM_ERR_UNSUPPORTED, "attn_decode_paged: batch %d is outside what the balanced kernel takes", batch);
    if (!workspace || workspace_bytes < need)
        return fail(NIMLLM_ERR_WORKSPACE, "attn_decode_paged: workspace %zu bytes, need %zu", workspace_bytes, need);
    if ((((uintptr_t)k_pages | (uintptr_t)v_pages) & 15) || ((uintptr_t)workspace & 15))
        return fail(NIMLLM_ERR_ARG, "attn_decode_paged: pages and workspace must be 16-byte aligned");
    DecodeParams p;
    p.q = q; p.k = k_pages; p.v = v_pages; p.kv_off = nullptr; p.seq_stride = 0; p.head_stride = 0;
    p.seq_len = seq_len; p.out = out; p.partials_out = partials_out; p.ws = (float *)workspace;
    p.q_dtype = q_dtype; p.out_dtype = out_dtype; p.max_len = max_len; p.chunk_rows = 0;
    p.B = batch; p.Hq = n_head; p.Hkv = n_kv_head; p.G = n_head / n_kv_head;
    p.scale_log2e = scale * kLog2e;
    p.page_table = page_table; p.max_pages = max_pages; p.page_shift = shift;
    p.page_stride = (int64_t)n_kv_head * page_rows * head_dim;
    return launch_balanced(p, seq_len, out, out_dtype, partials_out, batch, n_head, n_kv_head, head_dim, max_len,
                           workspace, (cudaStream_t)stream);
}

// ---- this rank's part of a KV-sequence-sharded decode ---------------------------------------
// The shard decode with the exchange fused into its merge launch: the merge kernel holds every
// finished (o, m, l) record in registers and stores it straight into every peer's exchange
// buffer; its last CTA raises the rank's flag.  nimllm_attn_wait_combine finishes the step.
size_t nimllm_attn_decode_push_workspace_bytes(int batch, int n_head, int n_kv_head, int head_dim, int max_len) {
    if (batch <= 0 || n_head <= 0 || n_kv_head <= 0 || max_len <= 0 || n_head % n_kv_head != 0) return 0;
    const size_t bal = bal_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, true);
    if (bal == 0) return 0;
    // + the rows the decode kernel finishes by itself, kept where the merge kernel forwards them from
    return (bal + 255) / 256 * 256 + (size_t)batch * n_head * rec_stride(head_dim) * sizeof(float);
}

int nimllm_attn_decode_push(nimllm_peer_exchange *x, const void *q, int q_dtype, const void *k_cache,
                            const void *v_cache, const int64_t *kv_off, int64_t seq_stride, int64_t head_stride,
                            const int32_t *seq_len, int max_len, int batch, int n_head, int n_kv_head, int head_dim,
                            float scale, void *workspace, size_t workspace_bytes, void *stream) {
    if (!x || !q || !k_cache || !v_cache) return fail(NIMLLM_ERR_ARG, "attn_decode_push: null exchange / q / cache");
    if (batch <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head != 0 || max_len <= 0)
        return fail(NIMLLM_ERR_ARG, "attn_decode_push: bad shape B=%d Hq=%d Hkv=%d max_len=%d", batch, n_head, n_kv_head, max_len);
    if (!dtype_ok(q_dtype)) return fail(NIMLLM_ERR_ARG, "attn_decode_push: unknown dtype");
    if (head_dim != peer_head_dim(x) || batch * n_head > peer_rows_max(x))
        return fail(NIMLLM_ERR_ARG, "attn_decode_push: the exchange was created for head_dim %d and %d rows", peer_head_dim(x),
                    peer_rows_max(x));
    const size_t need = nimllm_attn_decode_push_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len);
    if (need == 0)
        return fail(NIMLLM_ERR_UNSUPPORTED, "attn_decode_push: needs head_dim 64 or 128 and Hq/Hkv <= 8 (use nimllm_attn_decode "
                                            "with partials_out and nimllm_attn_combine_peers otherwise)");
    if (!workspace || workspace_bytes < need)
        return fail(NIMLLM_ERR_WORKSPACE, "attn_decode_push: workspace %zu bytes, need %zu", workspace_bytes, need);
    if ((((uintptr_t)k_cache | (uintptr_t)v_cache) & 15) || ((uintptr_t)workspace & 255))
        return fail(NIMLLM_ERR_ARG, "attn_decode_push: caches 16-byte, workspace 256-byte aligned");
    if (head_stride % 8 != 0 || (!kv_off && seq_stride % 8 != 0))
        return fail(NIMLLM_ERR_ARG, "attn_decode_push: seq_stride and head_stride must be multiples of 16 bytes");
    const size_t bal = bal_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, true);
    float *rows_done = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + (bal + 255) / 256 * 256);
    DecodeParams p;
    p.q = q; p.k = k_cache; p.v = v_cache; p.kv_off = kv_off; p.seq_stride = seq_stride; p.head_stride = head_stride;
    p.seq_len = seq_len; p.out = nullptr; p.partials_out = rows_done; p.ws = (float *)workspace;
    p.q_dtype = q_dtype; p.out_dtype = NIMLLM_F32; p.max_len = max_len; p.chunk_rows = 0;
    p.B = batch; p.Hq = n_head; p.Hkv = n_kv_head; p.G = n_head / n_kv_head;
    p.scale_log2e = scale * kLog2e;
    p.page_table = nullptr; p.max_pages = 0; p.page_shift = 0; p.page_stride = 0;
    const PeerPush px = peer_push_of(x);
    return launch_balanced(p, seq_len, nullptr, NIMLLM_F32, rows_done, batch, n_head, n_kv_head, head_dim, max_len, workspace,
                           (cudaStream_t)stream, &px);
}

// ---- decode without a caller-provided workspace ------------------------------------------
// The chunk records of a split decode normally live in the caller's workspace.  This variant
// keeps them in a fixed array inside the library instead, for callers that have nowhere to
// get device memory from at the moment of the call (see include/nimllm_attn.h).
constexpr size_t kBuiltinScratchBytes = 8u << 20;   // 8 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

size_t nimllm_attn_decode_noalloc_max_bytes(void) { return kBuiltinScratchBytes; }

int nimllm_attn_decode_noalloc(const void *q, int q_dtype, const void *k_cache, const void *v_cache,
                               int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                               int64_t head_stride, const int32_t *seq_len, int max_len, void *out,
                               int out_dtype, float *partials_out, int batch, int n_head,
                               int n_kv_head, int head_dim, float scale, int chunk_rows, void *stream) {
    // shapes first: the size arithmetic below must not run on nonsense
    if (batch <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head != 0 || max_len <= 0 || chunk_rows < 0 ||
        (head_dim != 64 && head_dim != 128))
        return fail(NIMLLM_ERR_ARG, "attn_decode_noalloc: bad shape B=%d Hq=%d Hkv=%d D=%d max_len=%d chunk_rows=%d",
                    batch, n_head, n_kv_head, head_dim, max_len, chunk_rows);
    // In host code the array's name is only a handle; the device address has to be asked for,
    // once per device, with that device current.  Racing first calls store the same address.
    static std::atomic<void *> scratch_ptr[64];
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64)
        return fail(NIMLLM_ERR_CUDA, "attn_decode_noalloc: no usable current device (%s)", cudaGetErrorString(e));
    void *scratch = scratch_ptr[dev].load(std::memory_order_acquire);
    if (!scratch) {
        e = cudaGetSymbolAddress(&scratch, g_builtin_scratch);
        if (e != cudaSuccess || !scratch)
            return fail(NIMLLM_ERR_CUDA, "attn_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                        cudaGetErrorString(e));
        scratch_ptr[dev].store(scratch, std::memory_order_release);
    }
    // The call runs if the records of one of the two kernels fit: the library's own split of the
    // batch (chunk_rows = 0, bf16 cache, Hq/Hkv <= 8) needs a fixed amount that depends on the
    // head shape only; otherwise the chunk grid needs one record per (chunk, sequence, head).
    // nimllm_attn_decode makes the same choice from the same two numbers.
    const bool bal_possible = chunk_rows == 0 && cache_dtype == NIMLLM_BF16 && n_head / n_kv_head <= 8;
    const size_t bal = bal_possible ? bal_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, seq_len != nullptr) : 0;
    const size_t split = split_workspace_bytes(batch, n_head, n_kv_head, head_dim, max_len, chunk_rows);
    const bool bal_fits = bal > 0 && bal <= kBuiltinScratchBytes;
    if (!bal_fits && split > kBuiltinScratchBytes)
        return fail(NIMLLM_ERR_WORKSPACE,
                    "attn_decode_noalloc: this call needs %zu bytes of chunk records (%zu for the library's own split) "
                    "but the built-in scratch holds %zu; use nimllm_attn_decode with a workspace, or a larger chunk_rows",
                    split, bal, kBuiltinScratchBytes);
    return nimllm_attn_decode(q, q_dtype, k_cache, v_cache, cache_dtype, kv_off, seq_stride, head_stride, seq_len,
                              max_len, out, out_dtype, partials_out, batch, n_head, n_kv_head, head_dim, scale,
                              chunk_rows, scratch, kBuiltinScratchBytes, stream);
}

int nimllm_attn_combine(const float *parts, int n_parts, int rows, int head_dim, int rec_stride_,
                        void *out, int out_dtype, float *partials_out, void *stream) {
    if (!parts || (!out && !partials_out)) return fail(NIMLLM_ERR_ARG, "attn_combine: null pointer");
    if (n_parts <= 0 || rows <= 0 || head_dim <= 0 || head_dim > 256 || rec_stride_ < head_dim + 2)
        return fail(NIMLLM_ERR_ARG, "attn_combine: bad shape n_parts=%d rows=%d D=%d stride=%d", n_parts,
                    rows, head_dim, rec_stride_);
    if (out && !dtype_ok(out_dtype)) return fail(NIMLLM_ERR_ARG, "attn_combine: unknown dtype");
    if (partials_out && rec_stride_ != rec_stride(head_dim))
        return fail(NIMLLM_ERR_ARG, "attn_combine: partials_out needs rec_stride == head_dim + 4");
    CombineParams c;
    c.parts = parts; c.seq_len = nullptr; c.out = out; c.partials_out = partials_out;
    c.out_dtype = out_dtype; c.n_parts = n_parts; c.rows = rows; c.D = head_dim; c.W = rec_stride_;
    c.Hq = 1; c.chunk_rows = 1; c.max_len = 0;
    combine_kernel<<<(rows + 3) / 4, 128, 0, (cudaStream_t)stream>>>(c);
    NIMLLM_CHECK_LAUNCH("attn_combine");
    return NIMLLM_OK;
}

}  // extern "C"
