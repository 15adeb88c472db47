// matvec.cu -- the steps either side of decode attention, HBM-bound on the weight bytes.
//
// Replaces, for one new token per sequence (forwardCached with newTokens == 1):
//   * the three projections + RoPE + cache append of src/model.nim:775-815 (quantMatvec /
//     gpuSgemm x3, ropeFwd x2, 2*nKvHead cudaMemcpy) by ONE launch that reads xNorm and
//     wq | wk | wv, rotates q and k in registers and stores rotated K / raw V straight into
//     the cache row -- q, kNew and vNew never make the round trip through HBM;
//   * the output projection + residual of src/model.nim:843-849 (quantMatvec / gpuSgemm,
//     gpu_add) by one launch;
//   * the reference's quantised mat-vec launchers gpu_matvec_q4_0 / gpu_matvec_q8_0
//     (src/kernels.cu:941-1060), same names and arguments.
//
// Weight formats: fp32 and bf16 rows, and the reference's block formats -- Q4_0 {half d;
// uint8 qs[16]} = 18 bytes and Q8_0 {half d; int8 qs[32]} = 34 bytes per 32 weights
// (src/kernels.cu:898-901,1013-1016), value = d * (nibble - 8) or d * q.
//
// One warp owns one output row (or the rotation pair of rows f, f + D/2 of a head) and serves
// up to kMaxBatch input vectors with it, so a weight byte is fetched once per launch tile.
// Lanes stride over the row in units of 16 bytes (fp32 / bf16) or of block pairs read as
// aligned 32-bit words (Q4_0: 9 words, Q8_0: 17 words per 64 weights; single blocks through
// 16-bit loads when a row holds an odd number of blocks).  Block rows of a multiple of 16 bytes
// (cols a multiple of 256) are fetched 16 bytes per lane and passed through a per-warp buffer in
// shared memory instead (rows_dot_wide).  The input vectors sit in shared memory, padded by two
// floats per 64 for the block formats so that lanes reading different block pairs hit different
// banks; a block's even and odd weights are accumulated as packed fp32 pairs (fma.rn.f32x2).  A warp takes several rows per pass (their loads are in flight
// together, and every input value read from shared memory serves all of them).
//
// Two forms of every kernel: the weights loaded straight into registers (few input vectors), or
// staged through shared memory by the copy engine (eight input vectors per tile; see
// use_staged_matvec / use_staged_qkv for the measured crossover).
#include <cuda_fp16.h>

#include "common.cuh"
#include "tcgen05.cuh"

namespace nimllm {
namespace {
using namespace tc;       // mbarrier and shared-memory address helpers

constexpr int kMaxBatch = 8;      // input vectors served per weight fetch
constexpr int kMvWarps = 8;
constexpr int kStWarps = 8;       // warps of a staged kernel's CTA (one CTA per SM; 12 and 16 warps were measured: no gain)
__device__ int g_matvec_status = 0;   // sticky: 1 after a weight copy did not arrive within the wait limit

enum { W_F32 = 0, W_BF16 = 1, W_Q8_0 = 2, W_Q4_0 = 3 };

__host__ __device__ inline size_t row_bytes(int wt, int cols) {
    return wt == W_F32 ? (size_t)cols * 4 : wt == W_BF16 ? (size_t)cols * 2 : wt == W_Q8_0 ? (size_t)(cols / 32) * 34
                                                                                             : (size_t)(cols / 32) * 18;
}
// index of x[j] in shared memory: two pad floats per 64 for the block formats, so that lanes working
// on consecutive block pairs (66 floats apart) read different banks with their 8-byte loads
template <int WT> __device__ __forceinline__ int xs_index(int j) { return (WT >= W_Q8_0) ? j + 2 * (j >> 6) : j; }
template <int WT> __host__ __device__ inline int xs_stride(int cols) { return (WT >= W_Q8_0) ? cols + 2 * (cols / 64) + 4 : cols; }

// 4- and 2-byte loads of block data: neighbouring lanes and the loads of one lane share 32-byte
// sectors, so these allocate in L1 (every sector then comes out of L2 once per SM, not once per load)
__device__ __forceinline__ uint32_t ldg_u32(const void *p) {
    uint32_t r;
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ uint32_t ldg_u16(const void *p) {
    uint16_t r;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}
// the same from the staging ring in shared memory
__device__ __forceinline__ uint32_t lds_u32(const void *p) {
    uint32_t r;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ uint32_t lds_u16(const void *p) {
    uint16_t r;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(r) : "r"(smem_u32(p)));
    return r;
}
__device__ __forceinline__ uint4 lds_v4(const void *p) {
    uint4 r;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(smem_u32(p)));
    return r;
}
template <bool SM> __device__ __forceinline__ uint32_t ld_u32(const void *p) { return SM ? lds_u32(p) : ldg_u32(p); }
template <bool SM> __device__ __forceinline__ uint32_t ld_u16(const void *p) { return SM ? lds_u16(p) : ldg_u16(p); }
template <bool SM> __device__ __forceinline__ uint4 ld_v4(const void *p) { return SM ? lds_v4(p) : ldg_stream(p); }
__device__ __forceinline__ float half_bits_to_float(uint32_t h) { return __half2float(__ushort_as_half((unsigned short)(h & 0xffffu))); }

// acc[r][b] += sum_e wv[r][e] * x_b[j0 + e] for N consecutive weights of R rows: every input value
// is read from shared memory once and used for all R rows
template <int R, int NB, int N, bool VEC>
__device__ __forceinline__ void fma_chunk(const float (&wv)[R][N], const float *xs, int xs_ld, int j0, float (&acc)[R][NB]) {
#pragma unroll
    for (int b = 0; b < NB; b++) {
        float xv[N];
        if (VEC) {                                           // unpadded layout, j0 a multiple of 4: 16-byte reads
#pragma unroll
            for (int e = 0; e < N; e += 4) {
                const float4 t = *reinterpret_cast<const float4 *>(xs + b * xs_ld + j0 + e);
                xv[e] = t.x; xv[e + 1] = t.y; xv[e + 2] = t.z; xv[e + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int e = 0; e < N; e++) xv[e] = xs[b * xs_ld + j0 + e];
        }
#pragma unroll
        for (int e = 0; e < N; e++)
#pragma unroll
            for (int r = 0; r < R; r++) acc[r][b] = fmaf(wv[r][e], xv[e], acc[r][b]);
    }
}

// Four (Q8_0) or eight (Q4_0) quantised values of one 32-bit word of a block as floats (the block's
// scale is applied to the block's sum, as the reference's kernels do).  Q4_0: weight 2i = low nibble
// of byte i, weight 2i+1 = high nibble, minus 8 (src/kernels.cu:966-970); Q8_0: int8
// (src/kernels.cu:1033-1036).  No integer-to-float conversion instruction (a quarter-rate pipe): a
// byte b placed into the mantissa of 2^23 is the float 8388608 + b, and one exact subtraction takes
// the offset out.
__device__ __forceinline__ float byte_as_float(uint32_t word, int i) {         // 8388608 + byte i of word
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(word), "r"(0x4B000000u), "r"(0x7440u | (uint32_t)i));
    return __uint_as_float(r);
}
template <int WT> __device__ __forceinline__ void dequant_word(uint32_t q, float *out) {
    if (WT == W_Q4_0) {
        const uint32_t lo = q & 0x0F0F0F0Fu, hi = (q >> 4) & 0x0F0F0F0Fu;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[2 * i] = byte_as_float(lo, i) - 8388616.f;          // nibble - 8
            out[2 * i + 1] = byte_as_float(hi, i) - 8388616.f;
        }
    } else {
        const uint32_t u = q ^ 0x80808080u;                  // int8 + 128 as unsigned bytes
#pragma unroll
        for (int i = 0; i < 4; i++) out[i] = byte_as_float(u, i) - 8388736.f;
    }
}
// acc += d * part for the finished block of every row
template <int R, int NB> __device__ __forceinline__ void add_block(const float (&d)[R], float (&part)[R][NB], float (&acc)[R][NB]) {
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int b = 0; b < NB; b++) { acc[r][b] = fmaf(d[r], part[r][b], acc[r][b]); part[r][b] = 0.f; }
}

// Packed fp32 arithmetic (two IEEE fp32 operations per instruction, each rounded like the scalar form).
__device__ __forceinline__ uint64_t pack2(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) { uint64_t r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }
__device__ __forceinline__ float sum2(uint64_t v) { float lo, hi; asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); return lo + hi; }
// the quantised values of one 32-bit word as pairs of consecutive weights (same byte trick as dequant_word)
template <int WT> __device__ __forceinline__ void dequant_word2(uint32_t q, uint64_t *out) {
    if (WT == W_Q4_0) {
        const uint32_t lo = q & 0x0F0F0F0Fu, hi = (q >> 4) & 0x0F0F0F0Fu;
        const uint64_t k2 = pack2(-8388616.f, -8388616.f);               // nibble - 8
#pragma unroll
        for (int i = 0; i < 4; i++) out[i] = add2(pack2(byte_as_float(lo, i), byte_as_float(hi, i)), k2);
    } else {
        const uint32_t u = q ^ 0x80808080u;                              // int8 + 128 as unsigned bytes
        const uint64_t k2 = pack2(-8388736.f, -8388736.f);
#pragma unroll
        for (int i = 0; i < 2; i++) out[i] = add2(pack2(byte_as_float(u, 2 * i), byte_as_float(u, 2 * i + 1)), k2);
    }
}
// One block pair (64 weights) of R rows, read as aligned 32-bit words {d0 | q0[0..1]} q0.. {q0 tail | d1} q1..;
// `base` = index of the pair's first input value in the padded shared-memory layout (even: the input
// values are read two at a time).  Even and odd weights of a block are summed separately (packed fp32).
template <int WT, int NB, int R, bool SM>
__device__ __forceinline__ void pair_dot(const unsigned char *const (&pp)[R], const float *xs, int xs_ld, int base, float (&acc)[R][NB]) {
    constexpr int QW = WT == W_Q4_0 ? 4 : 8;             // 32-bit words of quantised values per block
    constexpr int N = 32 / QW;                           // weights per word
    uint32_t w[R][2 * QW + 1];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int i = 0; i < 2 * QW + 1; i++) w[r][i] = ld_u32<SM>(pp[r] + 4 * i);
#pragma unroll
    for (int blk = 0; blk < 2; blk++) {
        uint64_t part[R][NB];
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) part[r][b] = 0ull;              // (+0, +0)
#pragma unroll
        for (int i = 0; i < QW; i++) {
            uint64_t wp[R][N / 2];
#pragma unroll
            for (int r = 0; r < R; r++)
                dequant_word2<WT>(blk == 0 ? (w[r][i] >> 16) | (w[r][i + 1] << 16) : w[r][QW + 1 + i], wp[r]);
#pragma unroll
            for (int b = 0; b < NB; b++)
#pragma unroll
                for (int h = 0; h < N / 2; h++) {
                    const uint64_t xp = *reinterpret_cast<const uint64_t *>(xs + b * xs_ld + base + blk * 32 + i * N + 2 * h);
#pragma unroll
                    for (int r = 0; r < R; r++) part[r][b] = fma2(wp[r][h], xp, part[r][b]);
                }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
            const float d = half_bits_to_float(blk == 0 ? w[r][0] : w[r][QW] >> 16);
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = fmaf(d, sum2(part[r][b]), acc[r][b]);
        }
    }
}

// Partial dot products of R weight rows with NB input vectors: this lane's share (lanes stride over
// the row, the loads of all R rows are in flight together); the caller adds the lanes up.
template <int WT, int NB, int R, bool SM = false>
__device__ __forceinline__ void rows_dot(const unsigned char *const (&row)[R], int cols, const float *xs, int xs_ld, int lane,
                                         float (&acc)[R][NB]) {
    if (WT == W_F32 || WT == W_BF16) {
        constexpr int N = WT == W_F32 ? 4 : 8;               // weights per 16-byte load
        constexpr int EB = WT == W_F32 ? 4 : 2;
        for (int j = lane * N; j < cols; j += 64 * N) {      // two units per lane and round: 2 R loads in flight
            const int j2 = j + 32 * N;
            const bool has2 = j2 < cols;
            uint4 u[2][R];
#pragma unroll
            for (int r = 0; r < R; r++) {
                u[0][r] = ld_v4<SM>(row[r] + (size_t)j * EB);
                u[1][r] = has2 ? ld_v4<SM>(row[r] + (size_t)j2 * EB) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
                if (h == 1 && !has2) break;
                float wv[R][N];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    if (WT == W_F32) {
                        wv[r][0] = __uint_as_float(u[h][r].x); wv[r][1] = __uint_as_float(u[h][r].y);
                        wv[r][2] = __uint_as_float(u[h][r].z); wv[r][3] = __uint_as_float(u[h][r].w);
                    } else {
                        Elem<__nv_bfloat16>::unpack(u[h][r], wv[r]);
                    }
                }
                fma_chunk<R, NB, N, true>(wv, xs, xs_ld, h ? j2 : j, acc);
            }
        }
    } else {
        constexpr int BS = WT == W_Q4_0 ? 18 : 34;           // bytes per block
        constexpr int QW = WT == W_Q4_0 ? 4 : 8;             // 32-bit words of quantised values per block
        constexpr int N = 32 / QW;                           // weights per word
        const int bpr = cols >> 5;
        bool aligned = (bpr & 1) == 0;
#pragma unroll
        for (int r = 0; r < R; r++) aligned = aligned && ((uintptr_t)row[r] & 3) == 0;
        if (aligned) {
            for (int pr = lane; pr < (bpr >> 1); pr += 32) {
                const unsigned char *pp[R];
#pragma unroll
                for (int r = 0; r < R; r++) pp[r] = row[r] + (size_t)pr * (2 * BS);
                pair_dot<WT, NB, R, SM>(pp, xs, xs_ld, pr * 66, acc);      // 64 weights + 2 pad floats per pair
            }
        } else {
            // rows with an odd number of blocks: single blocks through 16-bit loads
            for (int bk = lane; bk < bpr; bk += 32) {
                float part[R][NB], d[R];
#pragma unroll
                for (int r = 0; r < R; r++) {
                    d[r] = half_bits_to_float(ld_u16<SM>(row[r] + (size_t)bk * BS));
#pragma unroll
                    for (int b = 0; b < NB; b++) part[r][b] = 0.f;
                }
#pragma unroll
                for (int i = 0; i < QW; i++) {
                    float wv[R][N];
#pragma unroll
                    for (int r = 0; r < R; r++) {
                        const unsigned char *p = row[r] + (size_t)bk * BS;
                        dequant_word<WT>(ld_u16<SM>(p + 2 + 4 * i) | (ld_u16<SM>(p + 4 + 4 * i) << 16), wv[r]);
                    }
                    fma_chunk<R, NB, N, false>(wv, xs, xs_ld, bk * 32 + 2 * (bk >> 1) + i * N, part);
                }
                add_block<R, NB>(d, part, acc);
            }
        }
    }
}

// Block-format rows whose length in bytes is a multiple of 16 (cols a multiple of 256): the warp fetches
// a segment of 32 block pairs of each row with 16-byte loads, lanes on consecutive 16-byte pieces (every
// 32-byte sector is asked for once, not once per 32-bit word of a pair), passes it through a buffer of
// its own in shared memory and reads its pair from there (lanes 68 or 36 bytes apart: odd word strides,
// no bank conflicts).  The next segment's loads are in flight while the current one is worked on, and
// the first segment can be fetched before the input vectors are staged.
template <int WT> struct Wide {
    static constexpr int BS = WT == W_Q4_0 ? 18 : 34;
    static constexpr int kSegBytes = 32 * 2 * BS;                    // 2176 or 1152
    static constexpr int kPieces = (kSegBytes / 16 + 31) / 32;       // 16-byte pieces per lane: 5 or 3
    static constexpr int kBufBytes = kSegBytes + 16;                 // per row and warp
};
template <int WT, int R>
__device__ __forceinline__ void wide_fetch(uint4 (&pre)[R][Wide<WT>::kPieces], const unsigned char *const (&row)[R], int seg, int npairs,
                                           int lane) {
    const int pairs = min(32, npairs - seg * 32);
    const int pieces = (pairs * 2 * Wide<WT>::BS + 15) >> 4;         // the row ends on a 16-byte boundary: never past it
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int k = 0; k < Wide<WT>::kPieces; k++) {
            const int c = lane + 32 * k;
            if (c < pieces) pre[r][k] = ldg_stream(row[r] + (size_t)seg * Wide<WT>::kSegBytes + 16 * c);
        }
}
template <int WT, int NB, int R>
__device__ __forceinline__ void rows_dot_wide(const unsigned char *const (&row)[R], int cols, const float *xs, int xs_ld, int lane,
                                              float (&acc)[R][NB], unsigned char *wbuf, uint4 (&pre)[R][Wide<WT>::kPieces], bool fetched) {
    using Wd = Wide<WT>;
    const int npairs = cols >> 6;
    const int nseg = (npairs + 31) >> 5;
    if (!fetched) wide_fetch<WT, R>(pre, row, 0, npairs, lane);
    for (int seg = 0; seg < nseg; seg++) {
        const int pairs = min(32, npairs - seg * 32);
        const int pieces = (pairs * 2 * Wd::BS + 15) >> 4;
        __syncwarp();                                               // the buffer's previous contents have been used
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int k = 0; k < Wd::kPieces; k++) {
                const int c = lane + 32 * k;
                if (c < pieces) *reinterpret_cast<uint4 *>(wbuf + r * Wd::kBufBytes + 16 * c) = pre[r][k];
            }
        __syncwarp();
        if (seg + 1 < nseg) wide_fetch<WT, R>(pre, row, seg + 1, npairs, lane);
        if (lane < pairs) {
            const unsigned char *pp[R];
#pragma unroll
            for (int r = 0; r < R; r++) pp[r] = wbuf + r * Wd::kBufBytes + lane * (2 * Wd::BS);
            pair_dot<WT, NB, R, true>(pp, xs, xs_ld, (seg * 32 + lane) * 66, acc);
        }
    }
}

template <int R, int NB> __device__ __forceinline__ void warp_sum2(float (&acc)[R][NB]) {
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) acc[r][b] += __shfl_xor_sync(0xffffffffu, acc[r][b], off);
}

// the input vectors of this batch tile into shared memory (layout of xs_index)
template <int WT>
__device__ __forceinline__ void stage_x(float *xs, const float *x, int cols, int x_ld, int nb) {
    const int ld = xs_stride<WT>(cols);
    // 16-byte loads, four per thread in flight (cols is a multiple of 4 for every weight type; a group of
    // four floats never straddles a 64-float pad boundary).  x rows are 16-byte aligned when x and x_ld are.
    const int c4 = cols >> 2, n4 = nb * c4;
    if ((((uintptr_t)x | ((uintptr_t)x_ld << 2)) & 15) == 0) {
        for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * blockDim.x;
                if (i < n4) {
                    const int b = i / c4, j4 = i - b * c4;
                    v[u] = *reinterpret_cast<const float4 *>(x + (size_t)b * x_ld + 4 * j4);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * blockDim.x;
                if (i < n4) {
                    const int b = i / c4, j = 4 * (i - b * c4);
                    float *d = xs + b * ld + xs_index<WT>(j);
                    if (WT >= W_Q8_0) { d[0] = v[u].x; d[1] = v[u].y; d[2] = v[u].z; d[3] = v[u].w; }
                    else *reinterpret_cast<float4 *>(d) = v[u];
                }
            }
        }
    } else {
        for (int i = threadIdx.x; i < nb * cols; i += blockDim.x) {
            const int b = i / cols, j = i - b * cols;
            xs[b * ld + xs_index<WT>(j)] = x[(size_t)b * x_ld + j];
        }
    }
}

// ------------------------------------------------------------------ weights staged by bulk copies
// The weight bytes reach the SM through the copy engine, not through the warps' load instructions:
// every warp runs a ring of its own -- lane 0 issues cp.async.bulk copies of the next row segments
// into shared memory (completion counted on an mbarrier of the slot), the warp computes on the
// segment that has arrived.  Many KB per warp are in flight without a register holding them, and the
// block formats' 34- and 18-byte blocks are read from shared memory at full rate (lanes 68 or 36
// bytes apart: odd word strides, no bank conflicts) instead of as scattered 4-byte global loads.
//
// A job is two weight rows (the rotation pair f, f + D/2 of a head, or two neighbouring rows); an
// item is segment s of both rows.  A bulk copy wants 16-byte aligned addresses and sizes: a segment
// is copied from its address rounded down to 16 bytes up to its end rounded up, clipped to the last
// 16-byte boundary inside the matrix; the few bytes past that boundary come through the lanes.
struct SlabGeom {
    int cols, segw, nseg;     // weights per row, per segment, segments per row
    int nstage, slot_half;    // ring depth per warp, bytes of one row's buffer in a slot (a slot = 2 of them)
};
__host__ __device__ inline int seg_weights(int wt) { return wt == W_F32 ? 512 : wt == W_BF16 ? 1024 : wt == W_Q8_0 ? 2048 : 4096; }

__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t ldg_u8(const void *p) {
    uint32_t r;
    asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
// waits for copies that are in flight whatever the abort flag says (a CTA must not exit under them)
__device__ __forceinline__ bool mbar_wait_drain(uint64_t *bar, uint32_t parity) {
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0;; ++it) {
        if (mbar_try(bar, parity)) return true;
        if ((it & 255) == 255 && globaltimer_ns() - t0 > 1000000000ull) return false;
    }
}

// rows_of(jj, row, wend): global pointers to the two rows of this warp's jj-th job and the ends of
// their matrices; finish(jj, acc): the lanes' partial sums of a finished job.
template <int WT, typename RowsOf>
__device__ __forceinline__ void slab_issue(uint8_t *ring, uint64_t *full, const SlabGeom &g, int k, int lane, RowsOf rows_of) {
    const int jj = k / g.nseg, s = k - jj * g.nseg, slot = k % g.nstage;
    const unsigned char *row[2], *wend[2];
    rows_of(jj, row, wend);
    const int c0 = s * g.segw, nc = min(g.segw, g.cols - c0);
    const size_t off = row_bytes(WT, c0);
    const uint32_t len = (uint32_t)row_bytes(WT, nc);
    uint8_t *dst = ring + (size_t)slot * 2 * g.slot_half;
    uintptr_t ga0[2], ge0[2];
    uint32_t tx = 0;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uintptr_t ga = (uintptr_t)row[r] + off, ge = ga + len;
        const uintptr_t ge_up = (ge + 15) & ~(uintptr_t)15, w_dn = (uintptr_t)wend[r] & ~(uintptr_t)15;
        ga0[r] = ga & ~(uintptr_t)15;
        ge0[r] = ge_up < w_dn ? ge_up : w_dn;
        tx += (uint32_t)(ge0[r] - ga0[r]);
        // bytes past the last 16-byte boundary of the matrix (at most 15): through the lanes
        const int tail = ge > ge0[r] ? (int)(ge - ge0[r]) : 0;
        if (lane < tail) dst[r * g.slot_half + (ge0[r] - ga0[r]) + lane] = (uint8_t)ldg_u8((const void *)(ge0[r] + lane));
    }
    if (lane == 0) {
        // the slot was read (and its tail bytes written) through the generic proxy
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_expect_tx(&full[slot], tx);
#pragma unroll
        for (int r = 0; r < 2; r++)
            if (ge0[r] > ga0[r]) bulk_load(dst + r * g.slot_half, (const void *)ga0[r], (uint32_t)(ge0[r] - ga0[r]), &full[slot]);
    }
}

// the first segments of a warp's jobs: issued before the input vectors are staged, so that the
// weights are on their way while x is copied
template <int WT, typename RowsOf>
__device__ __forceinline__ void slab_prime(uint8_t *ring, uint64_t *full, const SlabGeom &g, int n_jobs, int lane, RowsOf rows_of) {
    const int n_items = n_jobs * g.nseg;
    for (int k = 0; k < min(g.nstage, n_items); k++) slab_issue<WT>(ring, full, g, k, lane, rows_of);
}

template <int WT, int NB, typename RowsOf, typename Finish>
__device__ __forceinline__ void slab_pipeline(uint8_t *ring, uint64_t *full, const SlabGeom &g, const float *xs, int xs_ld,
                                              int n_jobs, int lane, volatile int *abort_flag, RowsOf rows_of, Finish finish) {
    const int n_items = n_jobs * g.nseg;
    float acc[2][NB];
#pragma unroll
    for (int r = 0; r < 2; r++)
#pragma unroll
        for (int b = 0; b < NB; b++) acc[r][b] = 0.f;
    int k = 0;
    for (; k < n_items; k++) {
        const int jj = k / g.nseg, s = k - jj * g.nseg, slot = k % g.nstage;
        if (!mbar_wait(&full[slot], (uint32_t)(k / g.nstage) & 1u, abort_flag)) break;
        __syncwarp();
        const unsigned char *row[2], *wend[2];
        rows_of(jj, row, wend);
        const int c0 = s * g.segw, nc = min(g.segw, g.cols - c0);
        const size_t off = row_bytes(WT, c0);
        const uint8_t *src = ring + (size_t)slot * 2 * g.slot_half;
        const unsigned char *srow[2] = {src + (((uintptr_t)row[0] + off) & 15), src + g.slot_half + (((uintptr_t)row[1] + off) & 15)};
        rows_dot<WT, NB, 2, true>(srow, nc, xs + xs_index<WT>(c0), xs_ld, lane, acc);
        if (s == g.nseg - 1) {
            finish(jj, acc);
#pragma unroll
            for (int r = 0; r < 2; r++)
#pragma unroll
                for (int b = 0; b < NB; b++) acc[r][b] = 0.f;
        }
        __syncwarp();
        if (k + g.nstage < n_items) slab_issue<WT>(ring, full, g, k + g.nstage, lane, rows_of);
    }
    if (k < n_items) {
        // a copy did not arrive within the limit: nothing more is computed or issued, but the CTA may
        // only exit once the copies already issued (items k .. k + nstage - 1) have landed
        if (lane == 0) atomicExch(&g_matvec_status, 1);
        for (int kk = k; kk < min(k + g.nstage, n_items); kk++)
            if (!mbar_wait_drain(&full[kk % g.nstage], (uint32_t)(kk / g.nstage) & 1u)) break;
    }
}

// shared memory of the staged kernels: x | barriers | rings
__device__ __forceinline__ void slab_setup(float *xs_base, int xs_floats, const SlabGeom &g, uint64_t *&full, uint8_t *&ring,
                                           volatile int *&abort_flag) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *p = reinterpret_cast<uint8_t *>(xs_base) + (((size_t)xs_floats * 4 + 127) & ~(size_t)127);
    uint64_t *bars = reinterpret_cast<uint64_t *>(p);                   // kStWarps x 8 barriers, then the abort flag
    abort_flag = reinterpret_cast<volatile int *>(bars + kStWarps * 8);
    full = bars + warp * 8;
    ring = p + 2048 + (size_t)warp * g.nstage * 2 * g.slot_half;
    if (lane == 0) {
        for (int i = 0; i < g.nstage; i++) mbar_init(&full[i], 1);
        if (warp == 0) *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
}

// ------------------------------------------------------------------ y = W x (+ residual)
struct MatvecParams {
    const unsigned char *w;
    const float *x;          // [batch, cols], row stride x_ld
    const float *resid;      // [batch, rows] or null (row stride y_ld)
    float *y;                // [batch, rows], row stride y_ld
    int rows, cols, x_ld, y_ld, batch;
};

// Three resident CTAs per SM are asked for (two with four and more input vectors), not the eight that fit:
// with only "256 threads" as the bound the compiler holds the kernel to 32 - 40 registers to keep full
// occupancy and then cannot keep a pass's loads in flight together (fp32 q/k/v at 4096-wide layers:
// 23.5 -> 18.6 us with this bound).  Two CTAs per SM were measured for the block formats too: the
// q/k/v grid of a 4096-wide layer (384 CTAs) then no longer fits one wave and the call gets slower.  bf16 with
// four input vectors keeps three as well (76 registers suffice; 23.6 against 33.1 us with two).
template <int WT, int NB, int R>                             // R rows per warp pass
__global__ void __launch_bounds__(kMvWarps * 32, ((NB >= 4 && WT != W_BF16) ? 2 : 3)) matvec_kernel(MatvecParams p) {
    extern __shared__ __align__(16) float xs[];
    const int b0 = blockIdx.y * NB;
    const int nb = min(NB, p.batch - b0);
    const int ld = xs_stride<WT>(p.cols);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t rb = row_bytes(WT, p.cols);
    constexpr bool kBlocks = WT >= W_Q8_0;
    constexpr int WTB = kBlocks ? WT : W_Q8_0;               // (the wide path is only instantiated for block formats)
    const bool wide = kBlocks && R == 2 && (rb & 15) == 0;
    unsigned char *wbuf = reinterpret_cast<unsigned char *>(xs) + (((size_t)NB * ld * 4 + 15) & ~(size_t)15) +
                          (size_t)warp * R * Wide<WTB>::kBufBytes;
    uint4 pre[R][Wide<WTB>::kPieces];
    const int first_row = (blockIdx.x * kMvWarps + warp) * R;
    if (kBlocks && wide && first_row < p.rows) {             // the first weights are on their way while x is staged
        const unsigned char *rows[R];
#pragma unroll
        for (int r = 0; r < R; r++) rows[r] = p.w + (size_t)min(first_row + r, p.rows - 1) * rb;
        wide_fetch<WTB, R>(pre, rows, 0, p.cols >> 6, lane);
    }
    // Launched as a programmatic dependent of the kernel before it in the stream: everything above reads
    // only the weights; the input vectors (and every buffer written below) may belong to that kernel, so
    // its completion is awaited here.  The kernel after this one may place its CTAs early when this one had
    // weights to fetch before the wait (block formats); placing them early otherwise only crowds the SMs
    // that finish first (measured: bf16 24.7 against 22.3 us per layer).
    grid_dependency_wait();
    if (kBlocks) launch_dependents();
    stage_x<WT>(xs, p.x + (size_t)b0 * p.x_ld, p.cols, p.x_ld, nb);
    for (int i = threadIdx.x + nb * ld; i < NB * ld; i += blockDim.x) xs[i] = 0.f;     // unused vectors read as zeros
    __syncthreads();
    for (int row0 = first_row; row0 < p.rows; row0 += gridDim.x * kMvWarps * R) {
        float acc[R][NB];
        const unsigned char *rows[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            rows[r] = p.w + (size_t)min(row0 + r, p.rows - 1) * rb;     // rows past the end repeat the last one, unstored
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.f;
        }
        if (kBlocks && wide) rows_dot_wide<WTB, NB, R>(rows, p.cols, xs, ld, lane, acc, wbuf, pre, row0 == first_row);
        else rows_dot<WT, NB, R>(rows, p.cols, xs, ld, lane, acc);
        warp_sum2<R, NB>(acc);
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int b = 0; b < NB; b++)
                if (lane == r * NB + b && b < nb && row0 + r < p.rows) {
                    const size_t o = (size_t)(b0 + b) * p.y_ld + row0 + r;
                    p.y[o] = acc[r][b] + (p.resid ? p.resid[o] : 0.f);
                }
    }
    if (!kBlocks) launch_dependents();
}

// jobs = pairs of neighbouring rows (2j, 2j + 1); an odd last row is paired with itself, unstored
template <int WT, int NB>
__global__ void __launch_bounds__(kStWarps * 32, 1) matvec_staged_kernel(MatvecParams p, SlabGeom g) {
    extern __shared__ __align__(128) float xs[];
    const int b0 = blockIdx.y * NB;
    const int nb = min(NB, p.batch - b0);
    const int ld = xs_stride<WT>(p.cols);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t *full; uint8_t *ring; volatile int *abort_flag;
    slab_setup(xs, NB * ld, g, full, ring, abort_flag);
    const size_t rb = row_bytes(WT, p.cols);
    const unsigned char *w_end = p.w + (size_t)p.rows * rb;
    const int jobs = (p.rows + 1) >> 1;
    const int gw = blockIdx.x * kStWarps + warp, n_warps = gridDim.x * kStWarps;
    const int mine = gw < jobs ? (jobs - gw + n_warps - 1) / n_warps : 0;
    auto rows_of = [&](int jj, const unsigned char *(&row)[2], const unsigned char *(&wend)[2]) {
        const int r0 = 2 * (gw + jj * n_warps);
        row[0] = p.w + (size_t)r0 * rb;
        row[1] = p.w + (size_t)min(r0 + 1, p.rows - 1) * rb;
        wend[0] = wend[1] = w_end;
    };
    auto finish = [&](int jj, float (&acc)[2][NB]) {
        warp_sum2<2, NB>(acc);
        const int r0 = 2 * (gw + jj * n_warps);
#pragma unroll
        for (int r = 0; r < 2; r++)
#pragma unroll
            for (int b = 0; b < NB; b++)
                if (lane == r * NB + b && b < nb && r0 + r < p.rows) {
                    const size_t o = (size_t)(b0 + b) * p.y_ld + r0 + r;
                    p.y[o] = acc[r][b] + (p.resid ? p.resid[o] : 0.f);
                }
    };
    slab_prime<WT>(ring, full, g, mine, lane, rows_of);      // weights on their way while x is staged
    // Launched as a programmatic dependent of the kernel before it in the stream: everything above reads
    // only the weights; the input vectors (and every buffer written below) may belong to that kernel, so
    // its completion is awaited here; the kernel after this one may place its CTAs from now on.
    grid_dependency_wait();
    launch_dependents();
    stage_x<WT>(xs, p.x + (size_t)b0 * p.x_ld, p.cols, p.x_ld, nb);
    for (int i = threadIdx.x + nb * ld; i < NB * ld; i += blockDim.x) xs[i] = 0.f;
    __syncthreads();
    slab_pipeline<WT, NB>(ring, full, g, xs, ld, mine, lane, abort_flag, rows_of, finish);
}

// ------------------------------------------------------------------ q | k | v = W x, RoPE, cache append
struct QkvParams {
    const unsigned char *wq, *wk, *wv;
    const float *x;                     // [batch, n_embd]
    float *q_out, *k_out, *v_out;       // [batch, Hq*D]; [batch, Hkv*D] or null
    const float *cos_tab, *sin_tab;
    const int32_t *seq_pos;
    void *k_cache, *v_cache;
    const int64_t *kv_off;
    int64_t seq_stride, head_stride;
    int pos0, cache_row0, max_seq;
    int batch, n_embd, Hq, Hkv, D;
};

template <typename T> __device__ __forceinline__ void store_cache(T *p, float v);
template <> __device__ __forceinline__ void store_cache<float>(float *p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_cache<__nv_bfloat16>(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// One warp task = RP neighbouring rotation pairs (f, f + D/2) of one head of q, k or v: 2 RP weight
// rows whose loads are in flight together (the block formats have short rows: two pairs per task).
template <int WT, int NB, typename CacheT>
__global__ void __launch_bounds__(kMvWarps * 32, ((NB >= 4 && WT != W_BF16) ? 2 : 3)) qkv_rope_append_kernel(QkvParams p) {
    constexpr int RP = 1;                                 // (two pairs per task were measured: no gain for the block formats)
    extern __shared__ __align__(16) float xs[];
    const int b0 = blockIdx.y * NB;
    const int nb = min(NB, p.batch - b0);
    const int ld = xs_stride<WT>(p.n_embd);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = p.D / 2;
    const int fpt = half / RP;                            // tasks per head
    const int tasks = (p.Hq + 2 * p.Hkv) * fpt;
    const size_t rb = row_bytes(WT, p.n_embd);
    constexpr bool kBlocks = WT >= W_Q8_0;
    constexpr int WTB = kBlocks ? WT : W_Q8_0;            // (the wide path is only instantiated for block formats)
    const bool wide = kBlocks && (rb & 15) == 0;
    unsigned char *wbuf = reinterpret_cast<unsigned char *>(xs) + (((size_t)NB * ld * 4 + 15) & ~(size_t)15) +
                          (size_t)warp * 2 * RP * Wide<WTB>::kBufBytes;
    uint4 pre[2 * RP][Wide<WTB>::kPieces];
    auto rows_of = [&](int t, const unsigned char *(&rows)[2 * RP]) {
        const int slot = t / fpt, f0 = (t - slot * fpt) * RP;
        const bool is_q = slot < p.Hq, is_k = !is_q && slot < p.Hq + p.Hkv;
        const int head = is_q ? slot : (is_k ? slot - p.Hq : slot - p.Hq - p.Hkv);
        const unsigned char *w = is_q ? p.wq : (is_k ? p.wk : p.wv);
#pragma unroll
        for (int r = 0; r < 2 * RP; r++) rows[r] = w + (size_t)(head * p.D + f0 + (r >> 1) + (r & 1) * half) * rb;      // pair r/2: rows f, f + D/2
    };
    const int first_task = blockIdx.x * kMvWarps + warp;
    if (kBlocks && wide && first_task < tasks) {          // the first weights are on their way while x is staged
        const unsigned char *rows[2 * RP];
        rows_of(first_task, rows);
        wide_fetch<WTB, 2 * RP>(pre, rows, 0, p.n_embd >> 6, lane);
    }
    // Launched as a programmatic dependent of the kernel before it in the stream: everything above reads
    // only the weights; the input vectors (and every buffer written below) may belong to that kernel, so
    // its completion is awaited here.  The kernel after this one may place its CTAs early when this one had
    // weights to fetch before the wait (block formats); placing them early otherwise only crowds the SMs
    // that finish first (measured: bf16 24.7 against 22.3 us per layer).
    grid_dependency_wait();
    if (kBlocks) launch_dependents();
    stage_x<WT>(xs, p.x + (size_t)b0 * p.n_embd, p.n_embd, p.n_embd, nb);
    for (int i = threadIdx.x + nb * ld; i < NB * ld; i += blockDim.x) xs[i] = 0.f;
    __syncthreads();
    for (int t = first_task; t < tasks; t += gridDim.x * kMvWarps) {
        const int slot = t / fpt, f0 = (t - slot * fpt) * RP;
        const bool is_q = slot < p.Hq, is_k = !is_q && slot < p.Hq + p.Hkv;
        const int head = is_q ? slot : (is_k ? slot - p.Hq : slot - p.Hq - p.Hkv);
        float acc[2 * RP][NB];
        const unsigned char *rows[2 * RP];
        rows_of(t, rows);
#pragma unroll
        for (int r = 0; r < 2 * RP; r++)
#pragma unroll
            for (int b = 0; b < NB; b++) acc[r][b] = 0.f;
        if (kBlocks && wide) rows_dot_wide<WTB, NB, 2 * RP>(rows, p.n_embd, xs, ld, lane, acc, wbuf, pre, t == first_task);
        else rows_dot<WT, NB, 2 * RP>(rows, p.n_embd, xs, ld, lane, acc);
        warp_sum2<2 * RP, NB>(acc);
#pragma unroll
        for (int pr = 0; pr < RP; pr++)
#pragma unroll
            for (int b = 0; b < NB; b++)
                if (lane == pr * NB + b && b < nb) {
                    const int bb = b0 + b, f = f0 + pr, row0 = head * p.D + f;
                    const int pos = p.seq_pos ? p.seq_pos[bb] : p.pos0;
                    float x0 = acc[2 * pr][b], x1 = acc[2 * pr + 1][b];
                    if ((is_q || is_k) && p.cos_tab) {
                        // the expression of src/kernels.cu:412-413 with sign = +1
                        const float c = p.cos_tab[(size_t)pos * half + f], s = p.sin_tab[(size_t)pos * half + f];
                        const float ra = x0 * c - x1 * s, rd = x0 * s + x1 * c;
                        x0 = ra; x1 = rd;
                    }
                    if (is_q) {
                        float *o = p.q_out + (size_t)bb * p.Hq * p.D + row0;
                        o[0] = x0; o[half] = x1;
                    } else {
                        float *o = is_k ? p.k_out : p.v_out;
                        if (o) { o[(size_t)bb * p.Hkv * p.D + row0] = x0; o[(size_t)bb * p.Hkv * p.D + row0 + half] = x1; }
                        const int crow = pos - p.cache_row0;
                        if (p.k_cache && crow >= 0 && crow < p.max_seq) {
                            const int64_t base = (p.kv_off ? p.kv_off[bb] : (int64_t)bb * p.seq_stride) + (int64_t)head * p.head_stride +
                                                 (int64_t)crow * p.D + f;
                            CacheT *dst = reinterpret_cast<CacheT *>(is_k ? p.k_cache : p.v_cache) + base;
                            store_cache<CacheT>(dst, x0);
                            store_cache<CacheT>(dst + half, x1);
                        }
                    }
                }
    }
    if (!kBlocks) launch_dependents();
}

// the same epilogue as qkv_rope_append_kernel, on weights staged through shared memory
template <int WT, int NB, typename CacheT>
__global__ void __launch_bounds__(kStWarps * 32, 1) qkv_rope_append_staged_kernel(QkvParams p, SlabGeom g) {
    extern __shared__ __align__(128) float xs[];
    const int b0 = blockIdx.y * NB;
    const int nb = min(NB, p.batch - b0);
    const int ld = xs_stride<WT>(p.n_embd);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint64_t *full; uint8_t *ring; volatile int *abort_flag;
    slab_setup(xs, NB * ld, g, full, ring, abort_flag);
    const int half = p.D / 2;
    const int jobs = (p.Hq + 2 * p.Hkv) * half;
    const size_t rb = row_bytes(WT, p.n_embd);
    const int gw = blockIdx.x * kStWarps + warp, n_warps = gridDim.x * kStWarps;
    const int mine = gw < jobs ? (jobs - gw + n_warps - 1) / n_warps : 0;
    auto rows_of = [&](int jj, const unsigned char *(&row)[2], const unsigned char *(&wend)[2]) {
        const int t = gw + jj * n_warps;
        const int slot = t / half, f = t - slot * half;
        const bool is_q = slot < p.Hq, is_k = !is_q && slot < p.Hq + p.Hkv;
        const int head = is_q ? slot : (is_k ? slot - p.Hq : slot - p.Hq - p.Hkv);
        const unsigned char *w = is_q ? p.wq : (is_k ? p.wk : p.wv);
        row[0] = w + (size_t)(head * p.D + f) * rb;
        row[1] = row[0] + (size_t)half * rb;
        wend[0] = wend[1] = w + (size_t)(is_q ? p.Hq : p.Hkv) * p.D * rb;
    };
    auto finish = [&](int jj, float (&acc)[2][NB]) {
        warp_sum2<2, NB>(acc);
        const int t = gw + jj * n_warps;
        const int slot = t / half, f = t - slot * half;
        const bool is_q = slot < p.Hq, is_k = !is_q && slot < p.Hq + p.Hkv;
        const int head = is_q ? slot : (is_k ? slot - p.Hq : slot - p.Hq - p.Hkv);
#pragma unroll
        for (int b = 0; b < NB; b++)
            if (lane == b && b < nb) {
                const int bb = b0 + b, row0 = head * p.D + f;
                const int pos = p.seq_pos ? p.seq_pos[bb] : p.pos0;
                float x0 = acc[0][b], x1 = acc[1][b];
                if ((is_q || is_k) && p.cos_tab) {
                    // the expression of src/kernels.cu:412-413 with sign = +1
                    const float c = p.cos_tab[(size_t)pos * half + f], s = p.sin_tab[(size_t)pos * half + f];
                    const float ra = x0 * c - x1 * s, rd = x0 * s + x1 * c;
                    x0 = ra; x1 = rd;
                }
                if (is_q) {
                    float *o = p.q_out + (size_t)bb * p.Hq * p.D + row0;
                    o[0] = x0; o[half] = x1;
                } else {
                    float *o = is_k ? p.k_out : p.v_out;
                    if (o) { o[(size_t)bb * p.Hkv * p.D + row0] = x0; o[(size_t)bb * p.Hkv * p.D + row0 + half] = x1; }
                    const int crow = pos - p.cache_row0;
                    if (p.k_cache && crow >= 0 && crow < p.max_seq) {
                        const int64_t base = (p.kv_off ? p.kv_off[bb] : (int64_t)bb * p.seq_stride) + (int64_t)head * p.head_stride +
                                             (int64_t)crow * p.D + f;
                        CacheT *dst = reinterpret_cast<CacheT *>(is_k ? p.k_cache : p.v_cache) + base;
                        store_cache<CacheT>(dst, x0);
                        store_cache<CacheT>(dst + half, x1);
                    }
                }
            }
    };
    slab_prime<WT>(ring, full, g, mine, lane, rows_of);      // weights on their way while x is staged
    // Launched as a programmatic dependent of the kernel before it in the stream: everything above reads
    // only the weights; the input vectors (and every buffer written below) may belong to that kernel, so
    // its completion is awaited here; the kernel after this one may place its CTAs from now on.
    grid_dependency_wait();
    launch_dependents();
    stage_x<WT>(xs, p.x + (size_t)b0 * p.n_embd, p.n_embd, p.n_embd, nb);
    for (int i = threadIdx.x + nb * ld; i < NB * ld; i += blockDim.x) xs[i] = 0.f;
    __syncthreads();
    slab_pipeline<WT, NB>(ring, full, g, xs, ld, mine, lane, abort_flag, rows_of, finish);
}

// ------------------------------------------------------------------ host side
template <int kWarps = kMvWarps, typename K, typename... P> int launch_with_smem(K kernel, dim3 grid, size_t smem, cudaStream_t st, const char *what, const P &...params) {
    if (smem > 48 * 1024) {
        // opt in once per kernel and device (the attribute is per function, per device)
        static thread_local const void *done[64][32];
        int dev = 0;
        cudaGetDevice(&dev);
        bool seen = false;
        if (dev >= 0 && dev < 64)
            for (int i = 0; i < 32 && done[dev][i]; i++) seen |= done[dev][i] == (const void *)kernel;
        if (!seen) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "%s: shared memory opt-in: %s", what, cudaGetErrorString(e));
            if (dev >= 0 && dev < 64)
                for (int i = 0; i < 32; i++)
                    if (!done[dev][i]) { done[dev][i] = (const void *)kernel; break; }
        }
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = dim3(kWarps * 32); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, params...);
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return NIMLLM_OK;
}

int batch_tile(int batch) { return batch >= 8 ? 8 : batch > 2 ? 4 : batch; }      // 1, 2, 4 or 8 vectors per weight fetch

template <int WT> size_t smem_for(int nb, int cols) { return (size_t)nb * xs_stride<WT>(cols) * sizeof(float); }
// the direct kernels' shared memory: x, and for the block formats two row buffers per warp
template <int WT> size_t smem_direct(int nb, int cols) {
    size_t b = (smem_for<WT>(nb, cols) + 15) & ~(size_t)15;
    if (WT >= W_Q8_0) b += (size_t)kMvWarps * 2 * Wide<(WT >= W_Q8_0 ? WT : W_Q8_0)>::kBufBytes;
    return b;
}

// ring geometry of the staged kernels for nb input vectors of `cols` floats; false when shared memory
// cannot hold the vectors plus two stages per warp
template <int WT> bool slab_geom(int nb, int cols, SlabGeom &g, size_t &smem) {
    g.cols = cols;
    g.segw = cols < seg_weights(WT) ? cols : seg_weights(WT);
    g.nseg = (cols + g.segw - 1) / g.segw;
    g.slot_half = (int)((row_bytes(WT, g.segw) + 32 + 127) & ~(size_t)127);
    const size_t xs_bytes = (smem_for<WT>(nb, cols) + 127) & ~(size_t)127;
    const size_t per_stage = (size_t)kStWarps * 2 * g.slot_half;
    if (xs_bytes + 2048 + 2 * per_stage > 227 * 1024) return false;
    size_t n = (227 * 1024 - xs_bytes - 2048) / per_stage;
    g.nstage = (int)(n > 8 ? 8 : n);
    smem = xs_bytes + 2048 + g.nstage * per_stage;
    return true;
}

// Which kernel runs (measured at 4096-wide layers, weights larger than L2): with one to four input vectors
// the direct loads win (16 and more warps per SM hide the latency of the short dependent chains better than
// the eight ring-owning warps do); with eight vectors the arithmetic per weight byte is large, the weights
// are better read from shared memory at full rate and one CTA per SM stages x once instead of once per
// 16 rows: 55.6 -> 39.5 us (Q8_0 q/k/v), 90.8 -> 58.2 us (fp32).  Q8_0 pairs with two and four vectors
// run out of registers in the direct form (31.2 us vs 18.3 us staged).
template <int WT> bool use_staged_matvec(int nb) { return nb >= 8; }
template <int WT> bool use_staged_qkv(int nb) { return nb >= 8 || (WT == W_Q8_0 && nb >= 2); }

template <int WT>
int launch_matvec_direct(const MatvecParams &p, cudaStream_t st) {
    const int nb = batch_tile(p.batch);
    const size_t smem = smem_direct<WT>(nb, p.cols);
    if (smem > 227 * 1024) return fail(NIMLLM_ERR_UNSUPPORTED, "matvec: %d input vectors of %d floats do not fit shared memory", nb, p.cols);
    // fp32 / bf16: four rows per warp pass when that still leaves two CTAs of work per SM, else two;
    // the block formats always take two (their rows pass through two buffers per warp)
    const bool r4 = WT < W_Q8_0 && nb < 8 && p.rows >= 2 * sm_count() * kMvWarps * 2;
    const int rows_per_cta = kMvWarps * (r4 ? 4 : 2);
    int gx = (p.rows + rows_per_cta - 1) / rows_per_cta;
    const int cap = sm_count() * 8;
    if (gx > cap) gx = cap;
    dim3 grid(gx, (p.batch + nb - 1) / nb);
    switch (nb) {
        case 1: return r4 ? launch_with_smem(matvec_kernel<WT, 1, 4>, grid, smem, st, "matvec", p)
                          : launch_with_smem(matvec_kernel<WT, 1, 2>, grid, smem, st, "matvec", p);
        case 2: return r4 ? launch_with_smem(matvec_kernel<WT, 2, 4>, grid, smem, st, "matvec", p)
                          : launch_with_smem(matvec_kernel<WT, 2, 2>, grid, smem, st, "matvec", p);
        case 4: return r4 ? launch_with_smem(matvec_kernel<WT, 4, 4>, grid, smem, st, "matvec", p)
                          : launch_with_smem(matvec_kernel<WT, 4, 2>, grid, smem, st, "matvec", p);
        default: return launch_with_smem(matvec_kernel<WT, 8, 2>, grid, smem, st, "matvec", p);
    }
}

template <int WT>
int launch_matvec_t(const MatvecParams &p, cudaStream_t st) {
    const int nb = batch_tile(p.batch);
    if (!use_staged_matvec<WT>(nb)) return launch_matvec_direct<WT>(p, st);
    SlabGeom g;
    size_t smem;
    if (!slab_geom<WT>(nb, p.cols, g, smem))
        return fail(NIMLLM_ERR_UNSUPPORTED, "matvec: %d input vectors of %d floats do not fit shared memory", nb, p.cols);
    const int jobs = (p.rows + 1) / 2;
    int gx = (jobs + kStWarps - 1) / kStWarps;
    if (gx > sm_count()) gx = sm_count();                      // one CTA per SM, every warp a ring of its own
    dim3 grid(gx, (p.batch + nb - 1) / nb);
    switch (nb) {
        case 1: return launch_with_smem<kStWarps>(matvec_staged_kernel<WT, 1>, grid, smem, st, "matvec", p, g);
        case 2: return launch_with_smem<kStWarps>(matvec_staged_kernel<WT, 2>, grid, smem, st, "matvec", p, g);
        case 4: return launch_with_smem<kStWarps>(matvec_staged_kernel<WT, 4>, grid, smem, st, "matvec", p, g);
        default: return launch_with_smem<kStWarps>(matvec_staged_kernel<WT, 8>, grid, smem, st, "matvec", p, g);
    }
}

int launch_matvec(int wt, const MatvecParams &p, cudaStream_t st) {
    switch (wt) {
        case W_F32: return launch_matvec_t<W_F32>(p, st);
        case W_BF16: return launch_matvec_t<W_BF16>(p, st);
        case W_Q8_0: return launch_matvec_t<W_Q8_0>(p, st);
        default: return launch_matvec_t<W_Q4_0>(p, st);
    }
}

template <int WT, typename CacheT>
int launch_qkv_direct(const QkvParams &p, cudaStream_t st) {
    const int nb = batch_tile(p.batch);
    const size_t smem = smem_direct<WT>(nb, p.n_embd);
    if (smem > 227 * 1024) return fail(NIMLLM_ERR_UNSUPPORTED, "qkv_rope_append: %d input vectors of %d floats do not fit shared memory", nb, p.n_embd);
    const int rp = 1;
    const int tasks = (p.Hq + 2 * p.Hkv) * (p.D / 2 / rp);
    int gx = (tasks + kMvWarps - 1) / kMvWarps;
    const int cap = sm_count() * 8;
    if (gx > cap) gx = cap;
    dim3 grid(gx, (p.batch + nb - 1) / nb);
    switch (nb) {
        case 1: return launch_with_smem(qkv_rope_append_kernel<WT, 1, CacheT>, grid, smem, st, "qkv_rope_append", p);
        case 2: return launch_with_smem(qkv_rope_append_kernel<WT, 2, CacheT>, grid, smem, st, "qkv_rope_append", p);
        case 4: return launch_with_smem(qkv_rope_append_kernel<WT, 4, CacheT>, grid, smem, st, "qkv_rope_append", p);
        default: return launch_with_smem(qkv_rope_append_kernel<WT, 8, CacheT>, grid, smem, st, "qkv_rope_append", p);
    }
}

template <int WT, typename CacheT>
int launch_qkv_t(const QkvParams &p, cudaStream_t st) {
    const int nb = batch_tile(p.batch);
    if (!use_staged_qkv<WT>(nb)) return launch_qkv_direct<WT, CacheT>(p, st);
    SlabGeom g;
    size_t smem;
    if (!slab_geom<WT>(nb, p.n_embd, g, smem))
        return fail(NIMLLM_ERR_UNSUPPORTED, "qkv_rope_append: %d input vectors of %d floats do not fit shared memory", nb, p.n_embd);
    const int jobs = (p.Hq + 2 * p.Hkv) * (p.D / 2);
    int gx = (jobs + kStWarps - 1) / kStWarps;
    if (gx > sm_count()) gx = sm_count();
    dim3 grid(gx, (p.batch + nb - 1) / nb);
    switch (nb) {
        case 1: return launch_with_smem<kStWarps>(qkv_rope_append_staged_kernel<WT, 1, CacheT>, grid, smem, st, "qkv_rope_append", p, g);
        case 2: return launch_with_smem<kStWarps>(qkv_rope_append_staged_kernel<WT, 2, CacheT>, grid, smem, st, "qkv_rope_append", p, g);
        case 4: return launch_with_smem<kStWarps>(qkv_rope_append_staged_kernel<WT, 4, CacheT>, grid, smem, st, "qkv_rope_append", p, g);
        default: return launch_with_smem<kStWarps>(qkv_rope_append_staged_kernel<WT, 8, CacheT>, grid, smem, st, "qkv_rope_append", p, g);
    }
}

template <typename CacheT>
int launch_qkv(int wt, const QkvParams &p, cudaStream_t st) {
    switch (wt) {
        case W_F32: return launch_qkv_t<W_F32, CacheT>(p, st);
        case W_BF16: return launch_qkv_t<W_BF16, CacheT>(p, st);
        case W_Q8_0: return launch_qkv_t<W_Q8_0, CacheT>(p, st);
        default: return launch_qkv_t<W_Q4_0, CacheT>(p, st);
    }
}

bool weight_shape_ok(int wt, int cols) {
    if (wt < W_F32 || wt > W_Q4_0 || cols <= 0) return false;
    return wt == W_F32 ? cols % 4 == 0 : wt == W_BF16 ? cols % 8 == 0 : cols % 32 == 0;
}

}  // namespace
}  // namespace nimllm

using namespace nimllm;

extern "C" {

int nimllm_matvec(const void *w, int w_type, const float *x, const float *residual, float *y, int batch, int rows,
                  int cols, void *stream) {
    if (!w || !x || !y) return fail(NIMLLM_ERR_ARG, "matvec: null pointer");
    if (batch <= 0 || rows <= 0 || !weight_shape_ok(w_type, cols))
        return fail(NIMLLM_ERR_ARG, "matvec: bad shape batch=%d rows=%d cols=%d for weight type %d (fp32 rows: cols %% 4, bf16: "
                                    "cols %% 8, Q8_0 / Q4_0: cols %% 32)", batch, rows, cols, w_type);
    if (((uintptr_t)w & 15) || ((uintptr_t)x & 3) || ((uintptr_t)y & 3))
        return fail(NIMLLM_ERR_ARG, "matvec: the weights must be 16-byte aligned");
    MatvecParams p;
    p.w = (const unsigned char *)w; p.x = x; p.resid = residual; p.y = y;
    p.rows = rows; p.cols = cols; p.x_ld = cols; p.y_ld = rows; p.batch = batch;
    return launch_matvec(w_type, p, (cudaStream_t)stream);
}

int nimllm_wo_residual(const float *attn_out, const void *wo, int w_type, const float *x_resid, float *x_out, int batch,
                       int n_embd, int n_in, void *stream) {
    if (!x_resid) return fail(NIMLLM_ERR_ARG, "wo_residual: null residual");
    return nimllm_matvec(wo, w_type, attn_out, x_resid, x_out, batch, n_embd, n_in, stream);
}

int nimllm_qkv_rope_append(const float *x_norm, const void *wq, const void *wk, const void *wv, int w_type, float *q_out,
                           float *k_out, float *v_out, const float *rope_cos, const float *rope_sin,
                           const int32_t *seq_pos, int pos0, void *k_cache, void *v_cache, int cache_dtype,
                           const int64_t *kv_off, int64_t seq_stride, int64_t head_stride, int cache_row0, int max_seq,
                           int batch, int n_embd, int n_head, int n_kv_head, int head_dim, void *stream) {
    if (!x_norm || !wq || !wk || !wv || !q_out) return fail(NIMLLM_ERR_ARG, "qkv_rope_append: null x / weights / q_out");
    if (batch <= 0 || n_head <= 0 || n_kv_head <= 0 || head_dim <= 0 || (head_dim & 3) || !weight_shape_ok(w_type, n_embd))
        return fail(NIMLLM_ERR_ARG, "qkv_rope_append: bad shape batch=%d n_embd=%d Hq=%d Hkv=%d D=%d weight type %d", batch,
                    n_embd, n_head, n_kv_head, head_dim, w_type);
    if ((rope_cos == nullptr) != (rope_sin == nullptr))
        return fail(NIMLLM_ERR_ARG, "qkv_rope_append: give both RoPE tables or neither");
    if ((k_cache == nullptr) != (v_cache == nullptr))
        return fail(NIMLLM_ERR_ARG, "qkv_rope_append: give both cache pointers or neither");
    if (!k_cache && (!k_out || !v_out)) return fail(NIMLLM_ERR_ARG, "qkv_rope_append: nowhere to put k and v");
    if (k_cache && (!dtype_ok(cache_dtype) || max_seq <= 0))
        return fail(NIMLLM_ERR_ARG, "qkv_rope_append: bad cache dtype or max_seq");
    if (((uintptr_t)wq | (uintptr_t)wk | (uintptr_t)wv) & 15)
        return fail(NIMLLM_ERR_ARG, "qkv_rope_append: the weights must be 16-byte aligned");
    QkvParams p;
    p.wq = (const unsigned char *)wq; p.wk = (const unsigned char *)wk; p.wv = (const unsigned char *)wv;
    p.x = x_norm; p.q_out = q_out; p.k_out = k_out; p.v_out = v_out;
    p.cos_tab = rope_cos; p.sin_tab = rope_sin; p.seq_pos = seq_pos;
    p.k_cache = k_cache; p.v_cache = v_cache; p.kv_off = kv_off; p.seq_stride = seq_stride; p.head_stride = head_stride;
    p.pos0 = pos0; p.cache_row0 = cache_row0; p.max_seq = max_seq;
    p.batch = batch; p.n_embd = n_embd; p.Hq = n_head; p.Hkv = n_kv_head; p.D = head_dim;
    if (k_cache && cache_dtype == NIMLLM_BF16) return launch_qkv<__nv_bfloat16>(w_type, p, (cudaStream_t)stream);
    return launch_qkv<float>(w_type, p, (cudaStream_t)stream);
}

int nimllm_matvec_status(int reset) {
    int st = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&st, g_matvec_status, sizeof(int));
    if (e == cudaSuccess && reset && st != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_matvec_status, &zero, sizeof(int));
    }
    if (e != cudaSuccess) return -fail(NIMLLM_ERR_CUDA, "matvec_status: %s", cudaGetErrorString(e));
    return st;
}

/* src/kernels.cu:996-1003 and :1053-1059: y[rows] = A[rows, cols] x[cols], legacy default stream, void */
void gpu_matvec_q4_0(const void *A, const float *x, float *y, int rows, int cols) {
    if (nimllm_matvec(A, W_Q4_0, x, nullptr, y, 1, rows, cols, nullptr))
        fprintf(stderr, "gpu_matvec_q4_0: %s\n", nimllm_attn_last_error());
}
void gpu_matvec_q8_0(const void *A, const float *x, float *y, int rows, int cols) {
    if (nimllm_matvec(A, W_Q8_0, x, nullptr, y, 1, rows, cols, nullptr))
        fprintf(stderr, "gpu_matvec_q8_0: %s\n", nimllm_attn_last_error());
}

}  // extern "C"
