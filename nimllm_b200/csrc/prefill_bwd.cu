// prefill_bwd.cu -- backward of the causal GQA attention block (fp32), flash-style.
//
// Replaces the per-query-head loop of backward() in the reference (src/model.nim:639-685): per
// head it re-materialises scores and probabilities [S, S], forms dWeights, runs softmax_bwd
// (src/kernels.cu:305-328), two more S x S products and accumulates dk / dv of the shared KV
// head with atomics (src/kernels.cu:451-461) -- four S x S fp32 matrices through HBM per head.
// Here nothing of size S x S leaves the SM: probabilities are recomputed tile by tile from the
// saved post-RoPE q, k and the forward's log-sum-exp,
//     p_ij  = exp(scale * q_i.k_j - lse_i)            (j <= i)
//     dS_ij = p_ij * (dO_i.v_j - dO_i.o_i)
//     dv_j += sum_i p_ij dO_i     dk_j += scale * sum_i dS_ij q_i     dq_i = scale * sum_j dS_ij k_j
// and the rotation is undone on dq and dk in the epilogue (gpu_rope_bwd, src/kernels.cu:425-431).
//
// Three kernels: delta_i = dO_i.o_i per (sequence, head, row); dk/dv with one CTA per (32 KV rows,
// KV head) walking the query heads of the group and the query tiles at or below the diagonal --
// so the sums over heads and rows happen in a fixed order in registers, no atomics, results are
// deterministic; dq with one CTA per (32 query rows, query head) walking the KV tiles.
// fp32 FMA on the CUDA cores: this is the <= 1e-4 parity path of the training configuration
// (S = 128..2048, D = 64), not a tensor-core kernel.  The dk/dv and dq kernels exist twice: on
// 32 x 32 tiles (every head size, small launches) and on 64 x 64 register-blocked tiles (head size 64,
// launches that fill the GPU).
#include "common.cuh"

namespace nimllm {

namespace {

constexpr int kT = 32;          // tile edge: query rows and KV rows per tile
constexpr int kThreads = 128;

struct BwdParams {
    const float *q, *k, *v, *out, *dout, *lse;
    const float *cos_tab, *sin_tab;
    float *delta;               // [B, Hq, S]
    float *dk_part, *dv_part;   // [G][B*S][Hkv*D] per-query-head partial sums when G > 1, else null
    float *dq, *dk, *dv;
    int B, S, Hq, Hkv, pos0;
    float scale;
};

__global__ void __launch_bounds__(128) bwd_delta_kernel(BwdParams p, int D) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);       // over B * S * Hq, head fastest
    const int lane = threadIdx.x & 31;
    if (row >= p.B * p.S * p.Hq) return;
    const int h = row % p.Hq;
    const int64_t bs = row / p.Hq;                              // b * S + i
    const float *o = p.out + bs * p.Hq * D + (int64_t)h * D;
    const float *d = p.dout + bs * p.Hq * D + (int64_t)h * D;
    float acc = 0.f;
    for (int c = lane; c < D; c += 32) acc += o[c] * d[c];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) {
        const int b = (int)(bs / p.S), i = (int)(bs % p.S);
        p.delta[((int64_t)b * p.Hq + h) * p.S + i] = acc;
    }
}

// Shared-memory tiles are [32][D + 4] floats: rows stay 16-byte aligned for 128-bit loads and
// consecutive rows start 4 banks apart, so the 8 lanes of a quarter-warp reading one float4 each
// from consecutive rows (or consecutive float4s of one row) never collide.
template <int D> constexpr int ld() { return D + 4; }

// rows [row0, row0+32) x D of a [B*S, width] matrix (head at column col0) into a tile
template <int D>
__device__ __forceinline__ void load_tile(float *dst, const float *src, int64_t seq_base, int row0, int S, int width, int col0) {
    for (int idx = threadIdx.x; idx < kT * (D / 4); idx += kThreads) {
        const int r = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < S) x = *reinterpret_cast<const float4 *>(src + (seq_base + row0 + r) * width + col0 + c4);
        *reinterpret_cast<float4 *>(dst + r * ld<D>() + c4) = x;
    }
}

// The same tile in two steps, so that the global loads of the next tile are in flight while the
// current one is being used: fetch into registers (D/16 float4 per thread), stash into the tile.
template <int D>
__device__ __forceinline__ void fetch_tile(float4 (&reg)[D / 16], const float *src, int64_t seq_base, int row0, int S, int width, int col0) {
#pragma unroll
    for (int k = 0; k < D / 16; k++) {
        const int idx = threadIdx.x + k * kThreads;
        const int r = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
        reg[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < S) reg[k] = *reinterpret_cast<const float4 *>(src + (seq_base + row0 + r) * width + col0 + c4);
    }
}
template <int D>
__device__ __forceinline__ void stash_tile(float *dst, const float4 (&reg)[D / 16]) {
#pragma unroll
    for (int k = 0; k < D / 16; k++) {
        const int idx = threadIdx.x + k * kThreads;
        const int r = idx / (D / 4), c4 = (idx % (D / 4)) * 4;
        *reinterpret_cast<float4 *>(dst + r * ld<D>() + c4) = reg[k];
    }
}

// P and dS tiles [32 q rows][32 kv cols] from the staged Q, dO (rows) and K, V (cols).
// Thread t computes row t/4, columns (t%4) + 4u, u < 8, four values of d per step.
template <int D>
__device__ __forceinline__ void score_tile(const float *Qs, const float *dOs, const float *Ks, const float *Vs,
                                           const float *lse_s, const float *delta_s, float *Ps, float *dSs,
                                           int q0, int k0, int S, float scale) {
    const int r = threadIdx.x >> 2, cg = threadIdx.x & 3;
    float s[8], dp[8];
#pragma unroll
    for (int u = 0; u < 8; u++) { s[u] = 0.f; dp[u] = 0.f; }
    const float *qr = Qs + r * ld<D>(), *dor = dOs + r * ld<D>();
#pragma unroll 4
    for (int d = 0; d < D; d += 4) {
        const float4 qv = *reinterpret_cast<const float4 *>(qr + d);
        const float4 dv = *reinterpret_cast<const float4 *>(dor + d);
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const float4 kv = *reinterpret_cast<const float4 *>(Ks + (cg + 4 * u) * ld<D>() + d);
            const float4 vv = *reinterpret_cast<const float4 *>(Vs + (cg + 4 * u) * ld<D>() + d);
            s[u] = fmaf(qv.x, kv.x, fmaf(qv.y, kv.y, fmaf(qv.z, kv.z, fmaf(qv.w, kv.w, s[u]))));
            dp[u] = fmaf(dv.x, vv.x, fmaf(dv.y, vv.y, fmaf(dv.z, vv.z, fmaf(dv.w, vv.w, dp[u]))));
        }
    }
    const int qi = q0 + r;
    const float l = lse_s[r], dl = delta_s[r];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        const int col = cg + 4 * u, kj = k0 + col;
        const bool live = qi < S && kj <= qi;
        const float pv = live ? expf(s[u] * scale - l) : 0.f;
        Ps[r * (kT + 1) + col] = pv;
        dSs[r * (kT + 1) + col] = pv * (dp[u] - dl);
    }
}

// A thread owns the float4 groups dsel + 4*kq (kq < D/16) of its row: x[4*kq + i] is column
// 4*(dsel + 4*kq) + i.  The rotation partner of column f < D/2 is f + D/2, i.e. group + D/8 =
// the same thread's kq + D/32.
template <int D>
__device__ __forceinline__ void unrotate(float *x, const float *cos_tab, const float *sin_tab, int pos, int dsel) {
    if (!cos_tab) return;
    static_assert(D % 32 == 0, "head_dim must be a multiple of 32");
#pragma unroll
    for (int kq = 0; kq < D / 32; kq++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int f = 4 * (dsel + 4 * kq) + i;
            const float c = cos_tab[(int64_t)pos * (D / 2) + f], s = -sin_tab[(int64_t)pos * (D / 2) + f];
            const float x0 = x[4 * kq + i], x1 = x[4 * (kq + D / 32) + i];
            x[4 * kq + i] = x0 * c - x1 * s;             // k_rope with sign = -1 (src/kernels.cu:399-413)
            x[4 * (kq + D / 32) + i] = x0 * s + x1 * c;
        }
}

template <int D>
__global__ void __launch_bounds__(kThreads) bwd_dkdv_kernel(BwdParams p) {
    extern __shared__ float smem[];
    float *Ks = smem, *Vs = Ks + kT * ld<D>(), *Qs = Vs + kT * ld<D>(), *dOs = Qs + kT * ld<D>();
    float *Ps = dOs + kT * ld<D>(), *dSs = Ps + kT * (kT + 1);
    float *lse_s = dSs + kT * (kT + 1), *delta_s = lse_s + kT;

    // blockIdx.y is a KV head (one CTA sums over the group's query heads) or, when the partial
    // buffers are given, a query head (G times the CTAs, a third of the walk each at G = 3; the
    // partials are added up in head order by bwd_reduce_kernel)
    const int jt = blockIdx.x, b = blockIdx.z;
    const int G = p.Hq / p.Hkv, E = p.Hq * D, Ekv = p.Hkv * D;
    const bool split = p.dk_part != nullptr;
    const int kvh = split ? (int)blockIdx.y / G : (int)blockIdx.y;
    const int h_first = split ? (int)blockIdx.y : kvh * G, n_heads = split ? 1 : G;
    const int k0 = jt * kT;
    const int64_t seq_base = (int64_t)b * p.S;
    const int n_tiles = (p.S + kT - 1) / kT;
    load_tile<D>(Ks, p.k, seq_base, k0, p.S, Ekv, kvh * D);
    load_tile<D>(Vs, p.v, seq_base, k0, p.S, Ekv, kvh * D);

    const int c = threadIdx.x >> 2, dsel = threadIdx.x & 3;      // this thread's KV row and column phase
    float dk[D / 4], dv[D / 4];
#pragma unroll
    for (int kk = 0; kk < D / 4; kk++) { dk[kk] = 0.f; dv[kk] = 0.f; }

    // (query head, query tile) pairs of this KV tile, in a fixed order; the next pair's rows are
    // fetched into registers while the current pair is being worked on
    const int per_h = n_tiles - jt, total = n_heads * per_h;
    float4 rq[D / 16], rdo[D / 16];
    float rl = 0.f, rd = 0.f;
    auto fetch = [&](int n) {
        const int h = h_first + n / per_h, q0 = (jt + n % per_h) * kT;
        fetch_tile<D>(rq, p.q, seq_base, q0, p.S, E, h * D);
        fetch_tile<D>(rdo, p.dout, seq_base, q0, p.S, E, h * D);
        if (threadIdx.x < kT) {
            const int qi = q0 + threadIdx.x;
            rl = qi < p.S ? p.lse[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
            rd = qi < p.S ? p.delta[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
        }
    };
    fetch(0);
    for (int n = 0; n < total; n++) {
        const int q0 = (jt + n % per_h) * kT;
        __syncthreads();                                         // previous pair fully consumed
        stash_tile<D>(Qs, rq);
        stash_tile<D>(dOs, rdo);
        if (threadIdx.x < kT) { lse_s[threadIdx.x] = rl; delta_s[threadIdx.x] = rd; }
        __syncthreads();
        if (n + 1 < total) fetch(n + 1);
        score_tile<D>(Qs, dOs, Ks, Vs, lse_s, delta_s, Ps, dSs, q0, k0, p.S, p.scale);
        __syncthreads();
        for (int r = 0; r < kT; r++) {
            const float pv = Ps[r * (kT + 1) + c], ds = dSs[r * (kT + 1) + c];
#pragma unroll
            for (int kq = 0; kq < D / 16; kq++) {
                const float4 o4 = *reinterpret_cast<const float4 *>(dOs + r * ld<D>() + 4 * (dsel + 4 * kq));
                const float4 q4 = *reinterpret_cast<const float4 *>(Qs + r * ld<D>() + 4 * (dsel + 4 * kq));
                dv[4 * kq + 0] = fmaf(pv, o4.x, dv[4 * kq + 0]); dv[4 * kq + 1] = fmaf(pv, o4.y, dv[4 * kq + 1]);
                dv[4 * kq + 2] = fmaf(pv, o4.z, dv[4 * kq + 2]); dv[4 * kq + 3] = fmaf(pv, o4.w, dv[4 * kq + 3]);
                dk[4 * kq + 0] = fmaf(ds, q4.x, dk[4 * kq + 0]); dk[4 * kq + 1] = fmaf(ds, q4.y, dk[4 * kq + 1]);
                dk[4 * kq + 2] = fmaf(ds, q4.z, dk[4 * kq + 2]); dk[4 * kq + 3] = fmaf(ds, q4.w, dk[4 * kq + 3]);
            }
        }
    }
    const int kj = k0 + c;
    if (kj < p.S) {
        float *dko, *dvo;
        if (split) {                                             // raw partial sums of this query head
            const int64_t off = (((int64_t)(h_first % G) * p.B * p.S) + seq_base + kj) * Ekv + (int64_t)kvh * D;
            dko = p.dk_part + off; dvo = p.dv_part + off;
        } else {
#pragma unroll
            for (int kk = 0; kk < D / 4; kk++) dk[kk] *= p.scale;
            unrotate<D>(dk, p.cos_tab, p.sin_tab, p.pos0 + kj, dsel);
            dko = p.dk + (seq_base + kj) * Ekv + (int64_t)kvh * D; dvo = p.dv + (seq_base + kj) * Ekv + (int64_t)kvh * D;
        }
#pragma unroll
        for (int kq = 0; kq < D / 16; kq++) {
            *reinterpret_cast<float4 *>(dko + 4 * (dsel + 4 * kq)) = make_float4(dk[4 * kq], dk[4 * kq + 1], dk[4 * kq + 2], dk[4 * kq + 3]);
            *reinterpret_cast<float4 *>(dvo + 4 * (dsel + 4 * kq)) = make_float4(dv[4 * kq], dv[4 * kq + 1], dv[4 * kq + 2], dv[4 * kq + 3]);
        }
    }
}

// dk, dv = sum over the G query heads of a KV head of the partials, in head order; dk is then
// scaled and un-rotated.  One thread per (row, KV head, rotation pair).
__global__ void __launch_bounds__(256) bwd_reduce_kernel(BwdParams p, int D) {
    const int half = D / 2, G = p.Hq / p.Hkv, Ekv = p.Hkv * D;
    const int64_t total = (int64_t)p.B * p.S * p.Hkv * half;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const int f = (int)(idx % half);
    const int kvh = (int)((idx / half) % p.Hkv);
    const int64_t row = idx / ((int64_t)half * p.Hkv);             // b * S + position
    const int64_t o = row * Ekv + (int64_t)kvh * D + f;
    const int64_t gstride = (int64_t)p.B * p.S * Ekv;
    float k0 = 0.f, k1 = 0.f, v0 = 0.f, v1 = 0.f;
    for (int g = 0; g < G; g++) {
        k0 += p.dk_part[g * gstride + o]; k1 += p.dk_part[g * gstride + o + half];
        v0 += p.dv_part[g * gstride + o]; v1 += p.dv_part[g * gstride + o + half];
    }
    k0 *= p.scale; k1 *= p.scale;
    if (p.cos_tab) {
        const int pos = p.pos0 + (int)(row % p.S);
        const float c = p.cos_tab[(int64_t)pos * half + f], s = -p.sin_tab[(int64_t)pos * half + f];
        const float a = k0 * c - k1 * s, d = k0 * s + k1 * c;      // k_rope with sign = -1
        k0 = a; k1 = d;
    }
    p.dk[o] = k0; p.dk[o + half] = k1;
    p.dv[o] = v0; p.dv[o + half] = v1;
}

template <int D>
__global__ void __launch_bounds__(kThreads) bwd_dq_kernel(BwdParams p) {
    extern __shared__ float smem[];
    float *Ks = smem, *Vs = Ks + kT * ld<D>(), *Qs = Vs + kT * ld<D>(), *dOs = Qs + kT * ld<D>();
    float *Ps = dOs + kT * ld<D>(), *dSs = Ps + kT * (kT + 1);
    float *lse_s = dSs + kT * (kT + 1), *delta_s = lse_s + kT;

    // the query tiles with the longest walk are launched first
    const int it = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int G = p.Hq / p.Hkv, E = p.Hq * D, Ekv = p.Hkv * D, kvh = h / G;
    const int q0 = it * kT;
    const int64_t seq_base = (int64_t)b * p.S;
    load_tile<D>(Qs, p.q, seq_base, q0, p.S, E, h * D);
    load_tile<D>(dOs, p.dout, seq_base, q0, p.S, E, h * D);
    if (threadIdx.x < kT) {
        const int qi = q0 + threadIdx.x;
        lse_s[threadIdx.x] = qi < p.S ? p.lse[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
        delta_s[threadIdx.x] = qi < p.S ? p.delta[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
    }
    const int r = threadIdx.x >> 2, dsel = threadIdx.x & 3;
    float dq[D / 4];
#pragma unroll
    for (int kk = 0; kk < D / 4; kk++) dq[kk] = 0.f;

    float4 rk[D / 16], rv[D / 16];
    fetch_tile<D>(rk, p.k, seq_base, 0, p.S, Ekv, kvh * D);
    fetch_tile<D>(rv, p.v, seq_base, 0, p.S, Ekv, kvh * D);
    for (int jt = 0; jt <= it; jt++) {
        const int k0 = jt * kT;
        __syncthreads();
        stash_tile<D>(Ks, rk);
        stash_tile<D>(Vs, rv);
        __syncthreads();
        if (jt < it) {                                           // next KV tile in flight during this one
            fetch_tile<D>(rk, p.k, seq_base, k0 + kT, p.S, Ekv, kvh * D);
            fetch_tile<D>(rv, p.v, seq_base, k0 + kT, p.S, Ekv, kvh * D);
        }
        score_tile<D>(Qs, dOs, Ks, Vs, lse_s, delta_s, Ps, dSs, q0, k0, p.S, p.scale);
        __syncthreads();
        for (int cc = 0; cc < kT; cc++) {
            const float ds = dSs[r * (kT + 1) + cc];
#pragma unroll
            for (int kq = 0; kq < D / 16; kq++) {
                const float4 k4 = *reinterpret_cast<const float4 *>(Ks + cc * ld<D>() + 4 * (dsel + 4 * kq));
                dq[4 * kq + 0] = fmaf(ds, k4.x, dq[4 * kq + 0]); dq[4 * kq + 1] = fmaf(ds, k4.y, dq[4 * kq + 1]);
                dq[4 * kq + 2] = fmaf(ds, k4.z, dq[4 * kq + 2]); dq[4 * kq + 3] = fmaf(ds, k4.w, dq[4 * kq + 3]);
            }
        }
    }
    const int qi = q0 + r;
    if (qi < p.S) {
#pragma unroll
        for (int kk = 0; kk < D / 4; kk++) dq[kk] *= p.scale;
        unrotate<D>(dq, p.cos_tab, p.sin_tab, p.pos0 + qi, dsel);
        float *o = p.dq + (seq_base + qi) * E + (int64_t)h * D;
#pragma unroll
        for (int kq = 0; kq < D / 16; kq++)
            *reinterpret_cast<float4 *>(o + 4 * (dsel + 4 * kq)) = make_float4(dq[4 * kq], dq[4 * kq + 1], dq[4 * kq + 2], dq[4 * kq + 3]);
    }
}

// ---------------------------------------------------------------------- register-tiled forms (head_dim 64)
// The same arithmetic on 64 x 64 tiles for launches that fill the GPU: thread (rg, cg) of a 16 x 8 thread
// grid owns a 4 x 8 block of the score tile (rows rg + 16 i, columns cg + 8 j) and 4 rows x 8 columns
// (cg * 4 + 32 u + e) of the accumulated gradient, so a 16-byte shared-memory read feeds about ten
// multiply-adds instead of three and a half.  The rotation partner f + 32 of column f is held by the same
// thread.  Tiles are [64][68] floats: the strides rg * 68 and cg * 68 put the 16-byte reads of a
// quarter-warp on different banks.
constexpr int kTT = 64;            // tile edge of the tiled kernels
constexpr int kTL = 64 + 4;        // row pitch of their [64][64] tiles

__device__ __forceinline__ void load_tile64(float *dst, const float *src, int64_t seq_base, int row0, int S, int width, int col0) {
    for (int i = threadIdx.x; i < kTT * 16; i += 128) {
        const int r = i >> 4, c = (i & 15) * 4;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < S) x = *reinterpret_cast<const float4 *>(src + (seq_base + row0 + r) * width + col0 + c);
        *reinterpret_cast<float4 *>(dst + r * kTL + c) = x;
    }
}
// Packed fp32 arithmetic (two IEEE fp32 multiply-adds per instruction): the halves of a float4 read from
// shared memory are register pairs as they are.
__device__ __forceinline__ uint64_t pair_of(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) { uint64_t r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
__device__ __forceinline__ void unpair(uint64_t v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
// acc[i][j] += A[rg + 16 i] . B[cg + 8 j] over the 64 columns of two [64][68] tiles (even and odd columns are
// summed separately and added at the end)
__device__ __forceinline__ void tile_dots(const float *A, const float *B, int rg, int cg, float (&acc)[4][8]) {
    uint64_t acc2[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc2[i][j] = 0ull;
#pragma unroll 2
    for (int d = 0; d < 64; d += 4) {
        float4 af[4], bf[8];
#pragma unroll
        for (int i = 0; i < 4; i++) af[i] = *reinterpret_cast<const float4 *>(A + (rg + 16 * i) * kTL + d);
#pragma unroll
        for (int j = 0; j < 8; j++) bf[j] = *reinterpret_cast<const float4 *>(B + (cg + 8 * j) * kTL + d);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const uint64_t a01 = pair_of(af[i].x, af[i].y), a23 = pair_of(af[i].z, af[i].w);
#pragma unroll
            for (int j = 0; j < 8; j++) acc2[i][j] = fma2(a23, pair_of(bf[j].z, bf[j].w), fma2(a01, pair_of(bf[j].x, bf[j].y), acc2[i][j]));
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) { float e, o; unpair(acc2[i][j], e, o); acc[i][j] += e + o; }
}
// g[i][4u + e] += sum_j W[rg + 16 i][j] * X[j][cg * 4 + 32 u + e]: the weights of a row are written and read by
// the same eight lanes
__device__ __forceinline__ void tile_accumulate(const float *W, const float *X, int rg, int cg, float (&g)[4][8]) {
    uint64_t g2[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) g2[i][c] = pair_of(g[i][2 * c], g[i][2 * c + 1]);
#pragma unroll 2
    for (int j = 0; j < 64; j += 4) {
        float4 wf[4];
#pragma unroll
        for (int i = 0; i < 4; i++) wf[i] = *reinterpret_cast<const float4 *>(W + (rg + 16 * i) * kTL + j);
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const float4 x0 = *reinterpret_cast<const float4 *>(X + (j + jj) * kTL + cg * 4);
            const float4 x1 = *reinterpret_cast<const float4 *>(X + (j + jj) * kTL + cg * 4 + 32);
            const uint64_t x01 = pair_of(x0.x, x0.y), x23 = pair_of(x0.z, x0.w), x45 = pair_of(x1.x, x1.y), x67 = pair_of(x1.z, x1.w);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float w = jj == 0 ? wf[i].x : jj == 1 ? wf[i].y : jj == 2 ? wf[i].z : wf[i].w;
                const uint64_t ww = pair_of(w, w);
                g2[i][0] = fma2(ww, x01, g2[i][0]); g2[i][1] = fma2(ww, x23, g2[i][1]);
                g2[i][2] = fma2(ww, x45, g2[i][2]); g2[i][3] = fma2(ww, x67, g2[i][3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < 4; c++) unpair(g2[i][c], g[i][2 * c], g[i][2 * c + 1]);
}
// scale, undo the rotation (columns f = cg * 4 + e and f + 32 are g[e] and g[4 + e]; k_rope with sign = -1,
// src/kernels.cu:399-413) and store one row of a gradient
__device__ __forceinline__ void finish_row64(float (&g)[8], float scale, const float *cos_tab, const float *sin_tab, int pos, int cg, float *dst) {
#pragma unroll
    for (int c = 0; c < 8; c++) g[c] *= scale;
    if (cos_tab) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int f = cg * 4 + e;
            const float c = cos_tab[(int64_t)pos * 32 + f], s = -sin_tab[(int64_t)pos * 32 + f];
            const float x0 = g[e], x1 = g[4 + e];
            g[e] = x0 * c - x1 * s;
            g[4 + e] = x0 * s + x1 * c;
        }
    }
    *reinterpret_cast<float4 *>(dst + cg * 4) = make_float4(g[0], g[1], g[2], g[3]);
    *reinterpret_cast<float4 *>(dst + cg * 4 + 32) = make_float4(g[4], g[5], g[6], g[7]);
}

// dq of 64 query rows of one query head: walk the KV tiles up to the diagonal
__global__ void __launch_bounds__(128) bwd_dq_tiled_kernel(BwdParams p) {
    constexpr int D = 64;
    extern __shared__ __align__(16) float smem[];
    float *Qs = smem, *dOs = Qs + kTT * kTL, *Ks = dOs + kTT * kTL, *Vs = Ks + kTT * kTL, *dSs = Vs + kTT * kTL;
    float *lse_s = dSs + kTT * kTL, *delta_s = lse_s + kTT;
    const int it = (int)gridDim.x - 1 - (int)blockIdx.x, h = blockIdx.y, b = blockIdx.z;     // longest walks first
    const int G = p.Hq / p.Hkv, E = p.Hq * D, Ekv = p.Hkv * D, kvh = h / G;
    const int q0 = it * kTT;
    const int64_t seq_base = (int64_t)b * p.S;
    const int rg = threadIdx.x >> 3, cg = threadIdx.x & 7;
    load_tile64(Qs, p.q, seq_base, q0, p.S, E, h * D);
    load_tile64(dOs, p.dout, seq_base, q0, p.S, E, h * D);
    if (threadIdx.x < kTT) {
        const int qi = q0 + threadIdx.x;
        lse_s[threadIdx.x] = qi < p.S ? p.lse[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
        delta_s[threadIdx.x] = qi < p.S ? p.delta[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
    }
    float dq[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < 8; c++) dq[i][c] = 0.f;
    for (int jt = 0; jt <= it; jt++) {
        const int k0 = jt * kTT;
        __syncthreads();                                         // the previous tile's K and V have been used
        load_tile64(Ks, p.k, seq_base, k0, p.S, Ekv, kvh * D);
        load_tile64(Vs, p.v, seq_base, k0, p.S, Ekv, kvh * D);
        __syncthreads();
        float s[4][8], dp[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) { s[i][j] = 0.f; dp[i][j] = 0.f; }
        tile_dots(Qs, Ks, rg, cg, s);
        tile_dots(dOs, Vs, rg, cg, dp);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = rg + 16 * i, qi = q0 + r;
            const float l = lse_s[r], dl = delta_s[r];
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int kj = k0 + cg + 8 * j;
                const bool live = qi < p.S && kj <= qi;
                const float pv = live ? expf(s[i][j] * p.scale - l) : 0.f;
                dSs[r * kTL + cg + 8 * j] = pv * (dp[i][j] - dl);
            }
        }
        __syncwarp();
        tile_accumulate(dSs, Ks, rg, cg, dq);
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int qi = q0 + rg + 16 * i;
        if (qi < p.S) finish_row64(dq[i], p.scale, p.cos_tab, p.sin_tab, p.pos0 + qi, cg, p.dq + (seq_base + qi) * E + (int64_t)h * D);
    }
}

// dk, dv of 64 KV rows: walk the query heads of the group (or the one query head, when partial sums per head are
// kept) and their query tiles from the diagonal down.  The score tile is formed transposed ([kv][q]) so that a
// thread's rows are KV rows.
__global__ void __launch_bounds__(128) bwd_dkdv_tiled_kernel(BwdParams p) {
    constexpr int D = 64;
    extern __shared__ __align__(16) float smem[];
    float *Ks = smem, *Vs = Ks + kTT * kTL, *Qs = Vs + kTT * kTL, *dOs = Qs + kTT * kTL, *Pt = dOs + kTT * kTL, *dSt = Pt + kTT * kTL;
    float *lse_s = dSt + kTT * kTL, *delta_s = lse_s + kTT;
    const int jt = blockIdx.x, b = blockIdx.z;
    const int G = p.Hq / p.Hkv, E = p.Hq * D, Ekv = p.Hkv * D;
    const bool split = p.dk_part != nullptr;
    const int kvh = split ? (int)blockIdx.y / G : (int)blockIdx.y;
    const int h_first = split ? (int)blockIdx.y : kvh * G, n_heads = split ? 1 : G;
    const int k0 = jt * kTT;
    const int64_t seq_base = (int64_t)b * p.S;
    const int n_tiles = (p.S + kTT - 1) / kTT;
    const int rg = threadIdx.x >> 3, cg = threadIdx.x & 7;
    load_tile64(Ks, p.k, seq_base, k0, p.S, Ekv, kvh * D);
    load_tile64(Vs, p.v, seq_base, k0, p.S, Ekv, kvh * D);
    float dk[4][8], dv[4][8];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < 8; c++) { dk[i][c] = 0.f; dv[i][c] = 0.f; }
    const int per_h = n_tiles - jt, total = n_heads * per_h;
    for (int n = 0; n < total; n++) {
        const int h = h_first + n / per_h, q0 = (jt + n % per_h) * kTT;
        __syncthreads();                                         // the previous pair's tiles have been used
        load_tile64(Qs, p.q, seq_base, q0, p.S, E, h * D);
        load_tile64(dOs, p.dout, seq_base, q0, p.S, E, h * D);
        if (threadIdx.x < kTT) {
            const int qi = q0 + threadIdx.x;
            lse_s[threadIdx.x] = qi < p.S ? p.lse[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
            delta_s[threadIdx.x] = qi < p.S ? p.delta[((int64_t)b * p.Hq + h) * p.S + qi] : 0.f;
        }
        __syncthreads();
        float s[4][8], dp[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 8; j++) { s[i][j] = 0.f; dp[i][j] = 0.f; }
        tile_dots(Ks, Qs, rg, cg, s);                            // s[i][j] = k[kv row i] . q[query j]
        tile_dots(Vs, dOs, rg, cg, dp);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int r = rg + 16 * i, kj = k0 + r;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const int c = cg + 8 * j, qi = q0 + c;
                const bool live = qi < p.S && kj <= qi;
                const float pv = live ? expf(s[i][j] * p.scale - lse_s[c]) : 0.f;
                Pt[r * kTL + c] = pv;
                dSt[r * kTL + c] = pv * (dp[i][j] - delta_s[c]);
            }
        }
        __syncwarp();
        tile_accumulate(Pt, dOs, rg, cg, dv);
        tile_accumulate(dSt, Qs, rg, cg, dk);
        __syncwarp();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int kj = k0 + rg + 16 * i;
        if (kj >= p.S) continue;
        if (split) {                                             // raw partial sums of this query head
            const int64_t off = (((int64_t)(h_first % G) * p.B * p.S) + seq_base + kj) * Ekv + (int64_t)kvh * D;
            *reinterpret_cast<float4 *>(p.dk_part + off + cg * 4) = make_float4(dk[i][0], dk[i][1], dk[i][2], dk[i][3]);
            *reinterpret_cast<float4 *>(p.dk_part + off + cg * 4 + 32) = make_float4(dk[i][4], dk[i][5], dk[i][6], dk[i][7]);
            *reinterpret_cast<float4 *>(p.dv_part + off + cg * 4) = make_float4(dv[i][0], dv[i][1], dv[i][2], dv[i][3]);
            *reinterpret_cast<float4 *>(p.dv_part + off + cg * 4 + 32) = make_float4(dv[i][4], dv[i][5], dv[i][6], dv[i][7]);
        } else {
            const int64_t off = (seq_base + kj) * Ekv + (int64_t)kvh * D;
            finish_row64(dk[i], p.scale, p.cos_tab, p.sin_tab, p.pos0 + kj, cg, p.dk + off);
            *reinterpret_cast<float4 *>(p.dv + off + cg * 4) = make_float4(dv[i][0], dv[i][1], dv[i][2], dv[i][3]);
            *reinterpret_cast<float4 *>(p.dv + off + cg * 4 + 32) = make_float4(dv[i][4], dv[i][5], dv[i][6], dv[i][7]);
        }
    }
}

int launch_bwd_tiled64(const BwdParams &p, cudaStream_t st) {
    const size_t smem_dq = (size_t)(5 * kTT * kTL + 2 * kTT) * sizeof(float), smem_kv = (size_t)(6 * kTT * kTL + 2 * kTT) * sizeof(float);
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(bwd_dkdv_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(bwd_dq_tiled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq);
        if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_prefill_bwd: shared memory opt-in: %s", cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    const int n_tiles = (p.S + kTT - 1) / kTT;
    const int rows = p.B * p.S * p.Hq;
    bwd_delta_kernel<<<(rows + 3) / 4, 128, 0, st>>>(p, 64);
    NIMLLM_CHECK_LAUNCH("attn_prefill_bwd delta");
    bwd_dkdv_tiled_kernel<<<dim3(n_tiles, p.dk_part ? p.Hq : p.Hkv, p.B), 128, smem_kv, st>>>(p);
    NIMLLM_CHECK_LAUNCH("attn_prefill_bwd dk dv");
    if (p.dk_part) {
        const int64_t n = (int64_t)p.B * p.S * p.Hkv * 32;
        bwd_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(p, 64);
        NIMLLM_CHECK_LAUNCH("attn_prefill_bwd reduce");
    }
    bwd_dq_tiled_kernel<<<dim3(n_tiles, p.Hq, p.B), 128, smem_dq, st>>>(p);
    NIMLLM_CHECK_LAUNCH("attn_prefill_bwd dq");
    return NIMLLM_OK;
}

template <int D>
int launch_bwd(const BwdParams &p, cudaStream_t st) {
    const size_t smem = (size_t)(4 * kT * ld<D>() + 2 * kT * (kT + 1) + 2 * kT) * sizeof(float);
    static bool attr_set[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(bwd_dkdv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_prefill_bwd: shared memory opt-in: %s", cudaGetErrorString(e));
        attr_set[dev] = true;
    }
    const int n_tiles = (p.S + kT - 1) / kT;
    const int rows = p.B * p.S * p.Hq;
    bwd_delta_kernel<<<(rows + 3) / 4, 128, 0, st>>>(p, D);
    NIMLLM_CHECK_LAUNCH("attn_prefill_bwd delta");
    bwd_dkdv_kernel<D><<<dim3(n_tiles, p.dk_part ? p.Hq : p.Hkv, p.B), kThreads, smem, st>>>(p);
    NIMLLM_CHECK_LAUNCH("attn_prefill_bwd dk dv");
    if (p.dk_part) {
        const int64_t n = (int64_t)p.B * p.S * p.Hkv * (D / 2);
        bwd_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(p, D);
        NIMLLM_CHECK_LAUNCH("attn_prefill_bwd reduce");
    }
    bwd_dq_kernel<D><<<dim3(n_tiles, p.Hq, p.B), kThreads, smem, st>>>(p);
    NIMLLM_CHECK_LAUNCH("attn_prefill_bwd dq");
    return NIMLLM_OK;
}

}  // namespace
}  // namespace nimllm

using namespace nimllm;

extern "C" {

// delta [B, Hq, S], then (for grouped heads) per-query-head partial dk and dv: 2 * [G][B*S][Hkv*D]
// = 2 * B*S*Hq*D floats
size_t nimllm_attn_prefill_bwd_workspace_bytes(int batch, int seq_len, int n_head, int head_dim) {
    if (batch <= 0 || seq_len <= 0 || n_head <= 0 || head_dim <= 0) return 0;
    size_t delta = ((size_t)batch * seq_len * n_head * sizeof(float) + 255) / 256 * 256;
    return delta + 2 * (size_t)batch * seq_len * n_head * head_dim * sizeof(float);
}

int nimllm_attn_prefill_bwd(const float *q_rot, const float *k_rot, const float *v, const float *out,
                            const float *dout, const float *lse, const float *rope_cos, const float *rope_sin,
                            int pos0, float *dq, float *dk, float *dv, int batch, int seq_len, int n_head,
                            int n_kv_head, int head_dim, float scale, void *workspace, size_t workspace_bytes,
                            void *stream) {
    if (!q_rot || !k_rot || !v || !out || !dout || !lse || !dq || !dk || !dv)
        return fail(NIMLLM_ERR_ARG, "attn_prefill_bwd: null pointer (q, k, v, out, dout, lse, dq, dk, dv are all required)");
    if (batch <= 0 || seq_len <= 0 || n_head <= 0 || n_kv_head <= 0 || n_head % n_kv_head != 0)
        return fail(NIMLLM_ERR_ARG, "attn_prefill_bwd: bad shape B=%d S=%d Hq=%d Hkv=%d", batch, seq_len, n_head, n_kv_head);
    if (head_dim != 32 && head_dim != 64 && head_dim != 128)
        return fail(NIMLLM_ERR_UNSUPPORTED, "attn_prefill_bwd: head_dim %d (32, 64 and 128 are built)", head_dim);
    if ((rope_cos == nullptr) != (rope_sin == nullptr))
        return fail(NIMLLM_ERR_ARG, "attn_prefill_bwd: rope_cos and rope_sin go together");
    if (batch > 65535 || n_head > 65535) return fail(NIMLLM_ERR_UNSUPPORTED, "attn_prefill_bwd: batch or head count > 65535");
    const size_t need = nimllm_attn_prefill_bwd_workspace_bytes(batch, seq_len, n_head, head_dim);
    if (!workspace || workspace_bytes < need)
        return fail(NIMLLM_ERR_WORKSPACE, "attn_prefill_bwd: workspace %zu bytes, need %zu", workspace_bytes, need);
    if (((uintptr_t)q_rot | (uintptr_t)k_rot | (uintptr_t)v | (uintptr_t)out | (uintptr_t)dout | (uintptr_t)dq | (uintptr_t)dk |
         (uintptr_t)dv | (uintptr_t)workspace) & 15)
        return fail(NIMLLM_ERR_ARG, "attn_prefill_bwd: q, k, v, out, dout, dq, dk, dv and the workspace must be 16-byte aligned");
    BwdParams p;
    p.q = q_rot; p.k = k_rot; p.v = v; p.out = out; p.dout = dout; p.lse = lse;
    p.cos_tab = rope_cos; p.sin_tab = rope_sin; p.delta = (float *)workspace;
    {
        const size_t delta_bytes = ((size_t)batch * seq_len * n_head * sizeof(float) + 255) / 256 * 256;
        const size_t part = (size_t)batch * seq_len * n_head * head_dim;      // floats per partial buffer
        float *base = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(workspace) + delta_bytes);
        const bool grouped = n_head != n_kv_head;
        p.dk_part = grouped ? base : nullptr;
        p.dv_part = grouped ? base + part : nullptr;
    }
    p.dq = dq; p.dk = dk; p.dv = dv;
    p.B = batch; p.S = seq_len; p.Hq = n_head; p.Hkv = n_kv_head; p.pos0 = pos0;
    p.scale = scale > 0.f ? scale : 1.0f / sqrtf((float)head_dim);
    cudaStream_t st = (cudaStream_t)stream;
    if (head_dim == 32) return launch_bwd<32>(p, st);
    // 64 x 64 tiles once there is about one query tile per two SMs, the 32 x 32 tiles below that
    if (head_dim == 64 && (int64_t)((seq_len + 63) / 64) * n_head * batch >= sm_count() / 2) return launch_bwd_tiled64(p, st);
    if (head_dim == 64) return launch_bwd<64>(p, st);
    return launch_bwd<128>(p, st);
}

}  // extern "C"
