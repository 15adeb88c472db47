// prefill_f32.cu -- causal GQA attention in fp32 on the CUDA cores.
//
// The <= 1e-4 parity path for the reference's fp32 forward() attention block
// (src/model.nim:498-508: per query head gather, cublasSgemm_v2 QK^T, gpu_causal_mask,
// gpu_softmax_fwd, cublasSgemm_v2 PV, scatter).  TF32 tensor-core products cannot hold
// 1e-4, so this path multiplies and accumulates in fp32.  It is flash-style: no S x S
// matrix is written; K/V tiles are staged in shared memory and an online softmax keeps
// (max, sum, output) per query row.  Two kernels: 16 query rows per CTA for small launches,
// 64 rows with register tiling once there is about a tile per SM.  Heads are read and written in place in
// the reference's [tokens, heads*D] layout, which removes the gather / scatter kernels
// (src/kernels.cu:349-365,439-449).  Also backs the reference's unused single-head entry
// gpu_flash_attn_fwd (src/kernels.cu:703-755).
#include "common.cuh"

namespace nimllm {

namespace {

constexpr int BM = 16;  // query rows per CTA (4 per warp)
constexpr int BN = 32;  // key rows per tile (one per lane)

template <int D>
__global__ void __launch_bounds__(128) prefill_f32_kernel(const float *__restrict__ q,
                                                          const float *__restrict__ k,
                                                          const float *__restrict__ v,
                                                          float *__restrict__ out,
                                                          float *__restrict__ lse, int S, int Hq,
                                                          int Hkv, float scale_log2e, int causal) {
    constexpr int RPW = BM / 4;  // rows per warp
    constexpr int DPL = D / 32;  // output columns per lane
    __shared__ __align__(16) float Qs[BM][D];
    __shared__ float Ks[BN][D + 1];
    __shared__ __align__(16) float Vs[BN][D];
    __shared__ __align__(16) float Ps[4][BN][RPW];

    const int tile_m = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (Hq / Hkv);
    const int E = Hq * D, Ekv = Hkv * D;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = tile_m * BM;
    const float *qb = q + (int64_t)b * S * E + (int64_t)h * D;
    const float *kb = k + (int64_t)b * S * Ekv + (int64_t)kvh * D;
    const float *vb = v + (int64_t)b * S * Ekv + (int64_t)kvh * D;

    for (int i = threadIdx.x; i < BM * D / 4; i += 128) {
        int r = i / (D / 4), c = (i % (D / 4)) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < S) x = *reinterpret_cast<const float4 *>(qb + (int64_t)(row0 + r) * E + c);
        *reinterpret_cast<float4 *>(&Qs[r][c]) = x;
    }

    float m[RPW], l[RPW], o[RPW][DPL];
#pragma unroll
    for (int r = 0; r < RPW; r++) {
        m[r] = -INFINITY; l[r] = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; d++) o[r][d] = 0.f;
    }

    const int last_row = min(row0 + BM, S) - 1;
    const int kv_end = causal ? last_row + 1 : S;  // keys [0, kv_end)
    for (int j0 = 0; j0 < kv_end; j0 += BN) {
        __syncthreads();
        for (int i = threadIdx.x; i < BN * D / 4; i += 128) {
            int r = i / (D / 4), c = (i % (D / 4)) * 4;
            float4 kx = make_float4(0.f, 0.f, 0.f, 0.f), vx = kx;
            if (j0 + r < S) {
                kx = *reinterpret_cast<const float4 *>(kb + (int64_t)(j0 + r) * Ekv + c);
                vx = *reinterpret_cast<const float4 *>(vb + (int64_t)(j0 + r) * Ekv + c);
            }
            Ks[r][c] = kx.x; Ks[r][c + 1] = kx.y; Ks[r][c + 2] = kx.z; Ks[r][c + 3] = kx.w;
            *reinterpret_cast<float4 *>(&Vs[r][c]) = vx;
        }
        __syncthreads();

        // scores of this lane's key against the warp's RPW query rows
        float s[RPW];
#pragma unroll
        for (int r = 0; r < RPW; r++) s[r] = 0.f;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
            float k0 = Ks[lane][d], k1 = Ks[lane][d + 1], k2 = Ks[lane][d + 2], k3 = Ks[lane][d + 3];
#pragma unroll
            for (int r = 0; r < RPW; r++) {
                float4 qv = *reinterpret_cast<const float4 *>(&Qs[warp * RPW + r][d]);
                s[r] = fmaf(qv.x, k0, s[r]); s[r] = fmaf(qv.y, k1, s[r]);
                s[r] = fmaf(qv.z, k2, s[r]); s[r] = fmaf(qv.w, k3, s[r]);
            }
        }
        const int key = j0 + lane;
        float p[RPW];
#pragma unroll
        for (int r = 0; r < RPW; r++) {
            const int qi = row0 + warp * RPW + r;
            const bool valid = key < S && (!causal || key <= qi);
            float sv = valid ? s[r] * scale_log2e : -INFINITY;
            float mx = sv;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            float m_new = fmaxf(m[r], mx);
            float safe = (m_new == -INFINITY) ? 0.f : m_new;
            float corr = ex2(m[r] - safe);
            p[r] = ex2(sv - safe);
            float sum = p[r];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            l[r] = l[r] * corr + sum;
            m[r] = m_new;
#pragma unroll
            for (int d = 0; d < DPL; d++) o[r][d] *= corr;
        }
        __syncwarp();
        if (RPW == 4) *reinterpret_cast<float4 *>(&Ps[warp][lane][0]) = make_float4(p[0], p[1], p[2], p[3]);
        __syncwarp();
#pragma unroll 8
        for (int j = 0; j < BN; j++) {
            float4 pj = *reinterpret_cast<const float4 *>(&Ps[warp][j][0]);
#pragma unroll
            for (int d = 0; d < DPL; d++) {
                float vv = Vs[j][lane + 32 * d];
                o[0][d] = fmaf(pj.x, vv, o[0][d]); o[1][d] = fmaf(pj.y, vv, o[1][d]);
                o[2][d] = fmaf(pj.z, vv, o[2][d]); o[3][d] = fmaf(pj.w, vv, o[3][d]);
            }
        }
    }

#pragma unroll
    for (int r = 0; r < RPW; r++) {
        const int qi = row0 + warp * RPW + r;
        if (qi >= S) continue;
        const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
#pragma unroll
        for (int d = 0; d < DPL; d++)
            out[((int64_t)b * S + qi) * E + (int64_t)h * D + lane + 32 * d] = o[r][d] * inv;
        if (lse && lane == 0)
            lse[((int64_t)b * Hq + h) * S + qi] = l[r] > 0.f ? (m[r] + log2f(l[r])) * kLn2 : -INFINITY;
    }
}

// ---------------------------------------------------------------------- register-tiled form
// The same arithmetic for launches large enough to fill the GPU with 64-row query tiles.  The kernel
// above reads shared memory once per two multiply-adds; here a thread owns a 4 x (BN / 8) block of the
// score tile and a 4 x (D / 8) block of the output, so every 16-byte shared-memory read feeds
// ten multiply-adds.  Thread (rg, cg) of the 16 x 8 thread grid takes query rows rg + 16 i, keys
// cg + 8 j and output columns cg * 4 + 32 u + e: with rows padded by 4 floats those strides keep the
// 16-byte reads of a quarter-warp on different banks.
// packed fp32 arithmetic (two IEEE fp32 operations per instruction); the halves of a float4 are register pairs
__device__ __forceinline__ uint64_t pair_of(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
__device__ __forceinline__ void unpair(uint64_t v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }

template <int D, int BN>
__global__ void __launch_bounds__(128) prefill_f32_tiled_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                                                const float *__restrict__ v, float *__restrict__ out,
                                                                float *__restrict__ lse, int S, int Hq, int Hkv,
                                                                float scale_log2e, int causal) {
    constexpr int TM = 64;               // query rows per CTA
    constexpr int LD = D + 4;            // row pitch of the Q, K, V tiles
    constexpr int LP = BN + 4;           // row pitch of the P tile
    constexpr int NJ = BN / 8;           // keys per thread
    constexpr int NU = D / 32;           // groups of four output columns per thread
    constexpr bool kPacked = D == 128;   // packed fp32 multiply-adds: measured 1.24 -> 1.13 ms at D = 128, a loss at D = 64
    extern __shared__ __align__(16) float tile_smem[];
    float *Qs = tile_smem, *Ks = Qs + TM * LD, *Vs = Ks + BN * LD, *Ps = Vs + BN * LD;

    const int tile_m = gridDim.x - 1 - blockIdx.x;      // heaviest tiles (most keys) first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (Hq / Hkv);
    const int E = Hq * D, Ekv = Hkv * D;
    const int rg = threadIdx.x >> 3, cg = threadIdx.x & 7;
    const int row0 = tile_m * TM;
    const float *qb = q + (int64_t)b * S * E + (int64_t)h * D;
    const float *kb = k + (int64_t)b * S * Ekv + (int64_t)kvh * D;
    const float *vb = v + (int64_t)b * S * Ekv + (int64_t)kvh * D;

    for (int i = threadIdx.x; i < TM * D / 4; i += 128) {
        const int r = i / (D / 4), c = (i % (D / 4)) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < S) x = *reinterpret_cast<const float4 *>(qb + (int64_t)(row0 + r) * E + c);
        *reinterpret_cast<float4 *>(Qs + r * LD + c) = x;
    }

    float m[4], l[4], o[4][NU * 4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        m[i] = -INFINITY; l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < NU * 4; c++) o[i][c] = 0.f;
    }

    const int last_row = min(row0 + TM, S) - 1;
    const int kv_end = causal ? last_row + 1 : S;
    for (int j0 = 0; j0 < kv_end; j0 += BN) {
        __syncthreads();                                  // the previous tile's K and V have been used
        for (int i = threadIdx.x; i < BN * D / 4; i += 128) {
            const int r = i / (D / 4), c = (i % (D / 4)) * 4;
            float4 kx = make_float4(0.f, 0.f, 0.f, 0.f), vx = kx;
            if (j0 + r < S) {
                kx = *reinterpret_cast<const float4 *>(kb + (int64_t)(j0 + r) * Ekv + c);
                vx = *reinterpret_cast<const float4 *>(vb + (int64_t)(j0 + r) * Ekv + c);
            }
            *reinterpret_cast<float4 *>(Ks + r * LD + c) = kx;
            *reinterpret_cast<float4 *>(Vs + r * LD + c) = vx;
        }
        __syncthreads();

        float s[4][NJ], s_odd[4][NJ];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < NJ; j++) { s[i][j] = 0.f; s_odd[i][j] = 0.f; }
#pragma unroll 2
        for (int d = 0; d < D; d += 4) {
            float4 qf[4], kf[NJ];
#pragma unroll
            for (int i = 0; i < 4; i++) qf[i] = *reinterpret_cast<const float4 *>(Qs + (rg + 16 * i) * LD + d);
#pragma unroll
            for (int j = 0; j < NJ; j++) kf[j] = *reinterpret_cast<const float4 *>(Ks + (cg + 8 * j) * LD + d);
            if constexpr (kPacked) {
                // packed multiply-adds on the halves of the float4 reads: even columns in s, odd ones in s_odd
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const uint64_t q01 = pair_of(qf[i].x, qf[i].y), q23 = pair_of(qf[i].z, qf[i].w);
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        uint64_t a = pair_of(s[i][j], s_odd[i][j]);
                        a = fma2(q23, pair_of(kf[j].z, kf[j].w), fma2(q01, pair_of(kf[j].x, kf[j].y), a));
                        unpair(a, s[i][j], s_odd[i][j]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < NJ; j++) {
                        s[i][j] = fmaf(qf[i].x, kf[j].x, s[i][j]); s[i][j] = fmaf(qf[i].y, kf[j].y, s[i][j]);
                        s[i][j] = fmaf(qf[i].z, kf[j].z, s[i][j]); s[i][j] = fmaf(qf[i].w, kf[j].w, s[i][j]);
                    }
            }
        }
        if constexpr (kPacked) {
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < NJ; j++) s[i][j] += s_odd[i][j];
        }
        // online softmax per row: the 8 threads of a row group sit in 8 neighbouring lanes
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int qi = row0 + rg + 16 * i;
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const int key = j0 + cg + 8 * j;
                const bool valid = key < S && (!causal || key <= qi);
                s[i][j] = valid ? s[i][j] * scale_log2e : -INFINITY;
                mx = fmaxf(mx, s[i][j]);
            }
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float m_new = fmaxf(m[i], mx);
            const float safe = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = ex2(m[i] - safe);
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; j++) {
                const float pv = ex2(s[i][j] - safe);
                sum += pv;
                Ps[(rg + 16 * i) * LP + cg + 8 * j] = pv;
            }
#pragma unroll
            for (int off = 1; off < 8; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            l[i] = l[i] * corr + sum;
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < NU * 4; c++) o[i][c] *= corr;
        }
        __syncwarp();                                     // a row's probabilities are written and read by the same 8 lanes
#pragma unroll 2
        for (int j = 0; j < BN; j += 4) {
            float4 pf[4];
#pragma unroll
            for (int i = 0; i < 4; i++) pf[i] = *reinterpret_cast<const float4 *>(Ps + (rg + 16 * i) * LP + j);
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                float4 vf[NU];
#pragma unroll
                for (int u = 0; u < NU; u++) vf[u] = *reinterpret_cast<const float4 *>(Vs + (j + jj) * LD + cg * 4 + 32 * u);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float pj = jj == 0 ? pf[i].x : jj == 1 ? pf[i].y : jj == 2 ? pf[i].z : pf[i].w;
                    if constexpr (kPacked) {
                        const uint64_t pp = pair_of(pj, pj);
#pragma unroll
                        for (int u = 0; u < NU; u++) {
                            unpair(fma2(pp, pair_of(vf[u].x, vf[u].y), pair_of(o[i][4 * u], o[i][4 * u + 1])), o[i][4 * u], o[i][4 * u + 1]);
                            unpair(fma2(pp, pair_of(vf[u].z, vf[u].w), pair_of(o[i][4 * u + 2], o[i][4 * u + 3])), o[i][4 * u + 2], o[i][4 * u + 3]);
                        }
                    } else {
#pragma unroll
                        for (int u = 0; u < NU; u++) {
                            o[i][4 * u] = fmaf(pj, vf[u].x, o[i][4 * u]); o[i][4 * u + 1] = fmaf(pj, vf[u].y, o[i][4 * u + 1]);
                            o[i][4 * u + 2] = fmaf(pj, vf[u].z, o[i][4 * u + 2]); o[i][4 * u + 3] = fmaf(pj, vf[u].w, o[i][4 * u + 3]);
                        }
                    }
                }
            }
        }
        __syncwarp();                                     // before the next tile's probabilities overwrite these
    }

#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int qi = row0 + rg + 16 * i;
        if (qi >= S) continue;
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
#pragma unroll
        for (int u = 0; u < NU; u++)
            *reinterpret_cast<float4 *>(out + ((int64_t)b * S + qi) * E + (int64_t)h * D + cg * 4 + 32 * u) =
                make_float4(o[i][4 * u] * inv, o[i][4 * u + 1] * inv, o[i][4 * u + 2] * inv, o[i][4 * u + 3] * inv);
        if (lse && cg == 0)
            lse[((int64_t)b * Hq + h) * S + qi] = l[i] > 0.f ? (m[i] + log2f(l[i])) * kLn2 : -INFINITY;
    }
}

template <int D, int BN>
int launch_tiled(const float *q, const float *k, const float *v, float *out, float *lse, int B, int S, int Hq, int Hkv,
                 float sl, int causal, cudaStream_t st) {
    const size_t smem = ((size_t)(64 + 2 * BN) * (D + 4) + (size_t)64 * (BN + 4)) * sizeof(float);
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (smem > 48 * 1024 && dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(prefill_f32_tiled_kernel<D, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_prefill fp32: shared memory opt-in: %s", cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    dim3 grid((S + 63) / 64, Hq, B);
    prefill_f32_tiled_kernel<D, BN><<<grid, 128, smem, st>>>(q, k, v, out, lse, S, Hq, Hkv, sl, causal);
    NIMLLM_CHECK_LAUNCH("attn_prefill fp32");
    return NIMLLM_OK;
}

}  // namespace

int launch_prefill_f32(const float *q, const float *k, const float *v, float *out, float *lse,
                       int B, int S, int Hq, int Hkv, int D, float scale, int causal,
                       cudaStream_t st) {
    static_assert(BM == 16, "Ps stores 4 rows per warp as one float4");
    dim3 grid((S + BM - 1) / BM, Hq, B);
    const float sl = scale * kLog2e;
    // the 64-row tiles need a launch with about one of them per SM (measured: 9 heads x 1024 tokens = 144 tiles
    // 117 -> 90 us, 9 x 512 = 72 tiles no difference); smaller launches keep the 16-row CTAs (a 32-row form of
    // the tiled kernel was measured for them: 61 against 51 us at 9 x 512)
    if ((int64_t)((S + 63) / 64) * Hq * B >= sm_count() / 2) {
        if (D == 64) return launch_tiled<64, 64>(q, k, v, out, lse, B, S, Hq, Hkv, sl, causal, st);
        if (D == 128) return launch_tiled<128, 32>(q, k, v, out, lse, B, S, Hq, Hkv, sl, causal, st);
        if (D == 32) return launch_tiled<32, 64>(q, k, v, out, lse, B, S, Hq, Hkv, sl, causal, st);
    }
    if (D == 32) prefill_f32_kernel<32><<<grid, 128, 0, st>>>(q, k, v, out, lse, S, Hq, Hkv, sl, causal);
    else if (D == 64) prefill_f32_kernel<64><<<grid, 128, 0, st>>>(q, k, v, out, lse, S, Hq, Hkv, sl, causal);
    else if (D == 128) prefill_f32_kernel<128><<<grid, 128, 0, st>>>(q, k, v, out, lse, S, Hq, Hkv, sl, causal);
    else return fail(NIMLLM_ERR_UNSUPPORTED, "prefill fp32: head_dim %d (32, 64, 128 are built)", D);
    NIMLLM_CHECK_LAUNCH("attn_prefill fp32");
    return NIMLLM_OK;
}

}  // namespace nimllm
