// prefill_tc2.cu -- causal GQA prefill attention on CTA pairs (bf16, D = 128, tcgen05 cta_group::2).
//
// Same computation and warp roles as prefill_tc.cu (see there for the softmax and the RoPE
// prologue), but two CTAs on neighbouring SMs form a cluster and work as one MMA unit:
//
//   * a pair owns 512 consecutive query rows of one (sequence, query head) as two 256-row
//     tiles; of each tile the even CTA holds rows 0..127 and the odd CTA rows 128..255 -- in its
//     own shared memory (Q), its own TMEM (S, P, O) and its own softmax warps;
//   * every MMA is issued once, by one thread of the even CTA, with M = 256: S_w = Q_w K_j^T and
//     O_w += P_w V_j run on both SMs' tensor cores.  The B operand is split between the CTAs:
//     each loads only HALF of every K tile (64 of its 128 KV rows) and half of every V tile (64 of
//     its 128 columns) and the hardware reads the other half from the partner's shared memory.
//     So a K/V tile fetched once serves 512 query rows instead of 256, and the B-operand traffic
//     out of each SM's shared memory is halved -- the two limits measured on the one-CTA kernel.
//
// Barriers.  K/V "full" barriers live in the even CTA: both producers' TMA loads count their
// bytes there (cp.async.bulk.tensor with cta_group::2, no multicast).  "Empty", "S ready" and
// "O ready" are raised in both CTAs at once by tcgen05.commit with a CTA mask.  "P ready" and
// "Q staged" are counted in the even CTA; the odd CTA's warps arrive there remotely.  Every wait
// is bounded as in prefill_tc.cu; a cluster barrier before the TMEM release keeps either CTA's
// shared memory and TMEM alive until its partner is done.
#include "tcgen05.cuh"

namespace nimllm {

namespace {

using namespace tc;

constexpr int kD = 128;
constexpr int kBM = 128;                      // query rows per CTA and tile (= TMEM lanes)
constexpr int kBN = 128;                      // KV rows per tile
constexpr int kSlots = 8;                     // ring of half tiles: K_0 V_0 K_1 V_1 ...
constexpr int kQTileBytes = kBM * kD * 2;     // 32 KiB
constexpr int kHalfBytes = kBN * kD;          // 16 KiB: half of a K tile (64 rows) or of a V tile (64 columns)
constexpr int kThreads = 384;
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;

struct Smem {
    uint8_t q[2][kQTileBytes];
    uint8_t kv[kSlots][kHalfBytes];
    uint64_t q_full, kv_full[kSlots], kv_empty[kSlots];
    uint64_t s_full[2], p_ready[2], o_full[2], drain;
    uint32_t tmem_base;
    volatile int abort_flag;
};

struct PairParams {
    __nv_bfloat16 *q;
    __nv_bfloat16 *out;
    float *lse;
    const float *cos_tab, *sin_tab;
    int *status;
    int B, S, Hq, Hkv, pos0;
    int rotate_q, write_back_q;
    float scale_log2e;
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
prefill_tc2_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                   const __grid_constant__ CUtensorMap v_map, PairParams p) {
    extern __shared__ uint8_t smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs, 1: partner
    const int G = p.Hq / p.Hkv;
    const int n_groups = (p.S + 4 * kBM - 1) / (4 * kBM);      // groups of 512 query rows
    // heaviest groups first; consecutive pairs walk the query heads of one sequence
    const int pair_id = (int)blockIdx.x >> 1;
    const int per_group = p.Hq * p.B;
    const int t = n_groups - 1 - pair_id / per_group;
    const int rem = pair_id % per_group;
    const int b = rem / p.Hq, h = rem % p.Hq;
    const int kvh = h / G;
    const int nkv_total = (p.S + kBN - 1) / kBN;
    const int row_base = t * 4 * kBM;                  // first query row of the pair
    const bool active1 = row_base + 2 * kBM < p.S;
    const int n0 = min(4 * t + 2, nkv_total);          // KV tiles of the 256-row tile 0 / 1
    const int n1 = active1 ? min(4 * t + 4, nkv_total) : 0;
    const int nmax = max(n0, n1);
    volatile int *abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, p.rotate_q ? 16 : 1);
        for (int s = 0; s < kSlots; s++) { mbar_init(&sm.kv_full[s], 1); mbar_init(&sm.kv_empty[s], 1); }
        for (int w = 0; w < 2; w++) {
            mbar_init(&sm.s_full[w], 1); mbar_init(&sm.p_ready[w], 8); mbar_init(&sm.o_full[w], 1);
        }
        mbar_init(&sm.drain, 1);
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        // the same warp of both CTAs: one allocation that covers the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the partner's barriers are initialised before anything is signalled there
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    if (warp == 8) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        if (lane == 0) {
            const int qx = h * kD, kx = kvh * kD;
            if (!p.rotate_q) {
                const uint32_t qbar = map_to_cta(&sm.q_full, 0);
                if (rank == 0) mbar_expect_tx(&sm.q_full, (active1 ? 2 : 1) * 2 * kQTileBytes);
                for (int w = 0; w < (active1 ? 2 : 1); w++) {
                    const int y = b * p.S + row_base + w * 2 * kBM + (int)rank * kBM;
                    tma_load_2d_pair(sm.q[w], &q_map, qx, y, qbar);
                    tma_load_2d_pair(sm.q[w] + kBoxBytes, &q_map, qx + 64, y, qbar);
                }
            }
            // ring position u = 2j for K_j, 2j + 1 for V_j
            for (int u = 0; u < 2 * nmax; u++) {
                const int slot = u % kSlots, ph = (u / kSlots) & 1;
                const int y = b * p.S + (u >> 1) * kBN;
                if (!mbar_wait(&sm.kv_empty[slot], ph ^ 1, abort_flag)) break;
                const uint32_t full = map_to_cta(&sm.kv_full[slot], 0);
                if (rank == 0) mbar_expect_tx(&sm.kv_full[slot], 2 * kHalfBytes);
                if (u & 1) {
                    // V_j: this CTA's 64 columns of the 128 KV rows
                    tma_load_2d_pair(sm.kv[slot], &v_map, kx + (int)rank * 64, y, full);
                } else {
                    // K_j: this CTA's 64 KV rows, both 64-column boxes (8 KiB each)
                    tma_load_2d_pair(sm.kv[slot], &k_map, kx, y + (int)rank * 64, full);
                    tma_load_2d_pair(sm.kv[slot] + kHalfBytes / 2, &k_map, kx + 64, y + (int)rank * 64, full);
                }
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer (even CTA only)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc_qk = instr_desc(2 * kBM, kBN, 0, 0);
            constexpr uint32_t idesc_pv = instr_desc(2 * kBM, kD, 0, 1);
            const uint32_t q_addr[2] = {smem_u32(sm.q[0]), smem_u32(sm.q[1])};
            const uint32_t s_tmem[2] = {tmem + 0, tmem + 128};
            const uint32_t o_tmem[2] = {tmem + 256, tmem + 384};
            const int n_w[2] = {n0, n1};
            bool ok = mbar_wait(&sm.q_full, 0, abort_flag);
            tc_fence_after();

            // S_w = Q_w K^T: 8 steps of 16 along D.  A: this CTA's 128 query rows (two 16 KiB boxes);
            // B: this CTA's 64 KV rows (two 8 KiB boxes); K-major, 1024 bytes between 8-row groups
            auto issue_qk = [&](int w, int slot) {
                const uint32_t ka = smem_u32(sm.kv[slot]);
#pragma unroll
                for (int ks = 0; ks < kD / 16; ks++) {
                    const uint32_t a_off = (ks >> 2) * kBoxBytes + (ks & 3) * 32;
                    const uint32_t b_off = (ks >> 2) * (kHalfBytes / 2) + (ks & 3) * 32;
                    mma_ss_pair(s_tmem[w], smem_desc(q_addr[w] + a_off, 16, 1024), smem_desc(ka + b_off, 16, 1024), idesc_qk, ks > 0);
                }
                tc_commit_pair(&sm.s_full[w]);
            };
            // O_w += P_w V: 8 steps of 16 KV rows; P from each CTA's TMEM, V MN-major: this CTA's
            // 64 columns, 16 rows = 2048 bytes per step
            auto issue_pv = [&](int w, int slot, int j) {
                const uint32_t va = smem_u32(sm.kv[slot]);
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ks++)
                    mma_ts_pair(o_tmem[w], s_tmem[w] + ks * 8, smem_desc(va + ks * 2048, kHalfBytes, 1024), idesc_pv,
                                (j > 0 || ks > 0) ? 1u : 0u);
                if (j == n_w[w] - 1) tc_commit_pair(&sm.o_full[w]);
            };
            auto wait_full = [&](int u) { return mbar_wait(&sm.kv_full[u % kSlots], (u / kSlots) & 1, abort_flag); };
            auto release = [&](int u) { tc_commit_pair(&sm.kv_empty[u % kSlots]); };

            if (ok && nmax > 0) ok = wait_full(0);
            if (ok && nmax > 0) {
                tc_fence_after();
                if (n0 > 0) issue_qk(0, 0);
                if (n1 > 0) issue_qk(1, 0);
                release(0);
            }
            for (int j = 0; ok && j < nmax; j++) {
                const int uv = 2 * j + 1, ukn = 2 * j + 2;
                const bool next = j + 1 < nmax;
                if (!(ok = wait_full(uv))) break;
                if (next && !(ok = wait_full(ukn))) break;
#pragma unroll
                for (int w = 0; w < 2; w++) {
                    if (j < n_w[w]) {
                        if (!(ok = mbar_wait(&sm.p_ready[w], j & 1, abort_flag))) break;
                        tc_fence_after();
                        issue_pv(w, uv % kSlots, j);
                    }
                    if (w == 1) release(uv);
                    if (j + 1 < n_w[w]) issue_qk(w, ukn % kSlots);
                }
                if (!ok) break;
                if (next) release(ukn);
            }
            tc_commit_pair_local(&sm.drain);
            mbar_wait(&sm.drain, 0, abort_flag);
        }
    } else if (warp < 8) {
        // ---------------------------------------------------------------- softmax groups (both CTAs)
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int w = warp >> 2;                       // 256-row tile of this group
        const int r = (warp & 3) * 32 + lane;          // row inside this CTA's half = TMEM lane
        const int tile_row0 = row_base + w * 2 * kBM + (int)rank * kBM;
        const int qrow = tile_row0 + r;
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + (w ? 128u : 0u);
        const uint32_t o_addr = lane_base + (w ? 384u : 256u);
        const int n = w ? n1 : n0;
        const int diag = tile_row0 / kBN;              // KV tile holding this half's diagonal; later tiles are masked out
        const float c = p.scale_log2e;
        const uint32_t p_ready_bar = map_to_cta(&sm.p_ready[w], 0);
        bool ok = true;

        if (p.rotate_q) {
            // stage this CTA's two 128-row Q tiles with RoPE (8 lanes per row, coalesced)
            const int c8 = (lane & 7) * 8;
#pragma unroll 1
            for (int half_i = 0; half_i < 2; half_i++) {
                uint4 lo[4], hi[4];
                float4 cs0[4], cs1[4], sn0[4], sn1[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int row = (half_i * 4 + u) * 32 + warp * 4 + (lane >> 3);     // 0..255: tile = row >> 7
                    const int pos = row_base + (row >> 7) * 2 * kBM + (int)rank * kBM + (row & 127);
                    lo[u] = hi[u] = make_uint4(0, 0, 0, 0);
                    cs0[u] = cs1[u] = sn0[u] = sn1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (pos < p.S) {
                        const __nv_bfloat16 *qg = p.q + ((int64_t)b * p.S + pos) * p.Hq * kD + (int64_t)h * kD + c8;
                        const float *ct = p.cos_tab + (int64_t)(p.pos0 + pos) * (kD / 2) + c8;
                        const float *st = p.sin_tab + (int64_t)(p.pos0 + pos) * (kD / 2) + c8;
                        lo[u] = *reinterpret_cast<const uint4 *>(qg);
                        hi[u] = *reinterpret_cast<const uint4 *>(qg + kD / 2);
                        cs0[u] = *reinterpret_cast<const float4 *>(ct);
                        cs1[u] = *reinterpret_cast<const float4 *>(ct + 4);
                        sn0[u] = *reinterpret_cast<const float4 *>(st);
                        sn1[u] = *reinterpret_cast<const float4 *>(st + 4);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int row = (half_i * 4 + u) * 32 + warp * 4 + (lane >> 3);
                    const int tile_i = row >> 7, rr = row & 127;
                    const int pos = row_base + tile_i * 2 * kBM + (int)rank * kBM + rr;
                    const float cs[8] = {cs0[u].x, cs0[u].y, cs0[u].z, cs0[u].w, cs1[u].x, cs1[u].y, cs1[u].z, cs1[u].w};
                    const float sn[8] = {sn0[u].x, sn0[u].y, sn0[u].z, sn0[u].w, sn1[u].x, sn1[u].y, sn1[u].z, sn1[u].w};
                    float x0[8], x1[8], a[8], d[8];
                    Elem<__nv_bfloat16>::unpack(lo[u], x0);
                    Elem<__nv_bfloat16>::unpack(hi[u], x1);
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        a[i] = x0[i] * cs[i] - x1[i] * sn[i];
                        d[i] = x0[i] * sn[i] + x1[i] * cs[i];
                    }
                    const uint4 rlo = make_uint4(pack_bf16(a[0], a[1]), pack_bf16(a[2], a[3]), pack_bf16(a[4], a[5]), pack_bf16(a[6], a[7]));
                    const uint4 rhi = make_uint4(pack_bf16(d[0], d[1]), pack_bf16(d[2], d[3]), pack_bf16(d[4], d[5]), pack_bf16(d[6], d[7]));
                    if (p.write_back_q && pos < p.S) {
                        __nv_bfloat16 *qg = p.q + ((int64_t)b * p.S + pos) * p.Hq * kD + (int64_t)h * kD + c8;
                        *reinterpret_cast<uint4 *>(qg) = rlo;
                        *reinterpret_cast<uint4 *>(qg + kD / 2) = rhi;
                    }
                    *reinterpret_cast<uint4 *>(sm.q[tile_i] + tile_offset(rr, c8)) = rlo;
                    *reinterpret_cast<uint4 *>(sm.q[tile_i] + tile_offset(rr, c8 + kD / 2)) = rhi;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(&sm.q_full, 0));
        }

        float m_ref = -INFINITY, l = 0.f;
        bool first = true;                             // no tile with an unmasked column seen yet
        for (int j = 0; j < n; j++) {
            if (!(ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_full[w], j & 1, abort_flag)))) break;
            tc_fence_after();
            if (j > diag) {
                // wholly above this half's diagonal (only the even CTA's last tile): P = 0
                uint32_t z[32];
#pragma unroll
                for (int i = 0; i < 32; i++) z[i] = 0u;
                tmem_st32(s_addr, z);
                tmem_st32(s_addr + 32, z);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { if (rank == 0) mbar_arrive(&sm.p_ready[w]); else mbar_arrive_cluster(p_ready_bar); }
                continue;
            }
            const bool masked = (j == diag);
            const int col0 = j * kBN;

            uint32_t v[128];
            tmem_ld32(s_addr, v);
            tmem_ld32(s_addr + 32, v + 32);
            tmem_ld32(s_addr + 64, v + 64);
            tmem_ld32(s_addr + 96, v + 96);
            tc_wait_ld();

            float mx;
            if (masked) {
                float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 128; i += 2) {
                    if (col0 + i <= qrow) m0 = fmaxf(m0, __uint_as_float(v[i]));
                    if (col0 + i + 1 <= qrow) m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
                }
                mx = fmaxf(m0, m1);
            } else {
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 128; i += 8) {
                    m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                    m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                    m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                    m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            const float mx_s = mx * c;
            float corr = 1.f;
            bool grow = false;
            if (first) {
                m_ref = mx_s;
                first = false;
            } else if (mx_s > m_ref + kRescaleThreshold) {
                corr = ex2(m_ref - mx_s);
                m_ref = mx_s;
                l *= corr;
                grow = true;
            }
            if (__any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                for (int ch = 0; ch < 4; ch++) {
                    uint32_t o[32];
                    tmem_ld32(o_addr + ch * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tmem_st32(o_addr + ch * 32, o);
                }
                tc_wait_st();
            }

            const float neg_m = -m_ref;
            float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
            uint32_t pk[64];
#pragma unroll
            for (int i = 0; i < 128; i += 4) {
                float x[4], e[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    x[u] = fmaf(__uint_as_float(v[i + u]), c, neg_m);
                    if (masked && col0 + i + u > qrow) x[u] = -INFINITY;
                    e[u] = ex2(x[u]);
                }
                sum0 += e[0]; sum1 += e[1]; sum2 += e[2]; sum3 += e[3];
                pk[i >> 1] = pack_bf16(e[0], e[1]);
                pk[(i >> 1) + 1] = pack_bf16(e[2], e[3]);
            }
            tmem_st32(s_addr, pk);
            tmem_st32(s_addr + 32, pk + 32);
            l += (sum0 + sum1) + (sum2 + sum3);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (rank == 0) mbar_arrive(&sm.p_ready[w]); else mbar_arrive_cluster(p_ready_bar); }
        }

        if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(&sm.o_full[w], 0, abort_flag));
        if (ok && n > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16 *og = p.out + ((int64_t)b * p.S + qrow) * p.Hq * kD + (int64_t)h * kD;
#pragma unroll 1
            for (int ch = 0; ch < 4; ch++) {
                uint32_t v[32];
                tmem_ld32(o_addr + ch * 32, v);
                tc_wait_ld();
                if (qrow < p.S) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 o4 = make_uint4(
                            pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv),
                            pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv),
                            pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv),
                            pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv));
                        *reinterpret_cast<uint4 *>(og + ch * 32 + i) = o4;
                    }
                }
            }
            if (p.lse && qrow < p.S)
                p.lse[((int64_t)b * p.Hq + h) * p.S + qrow] = l > 0.f ? (m_ref + log2f(l)) * kLn2 : -INFINITY;
        }
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    }

    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // neither CTA leaves (or frees TMEM) while its partner may still touch it
    if (threadIdx.x == 0 && sm.abort_flag) atomicExch(p.status, 1);
    if (warp == 9) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn2() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// 2-D bf16 tensor [rows, cols] row-major; box = 64 columns x box_rows rows, 128-byte swizzle
int make_map2(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn2();
    if (!fn) return fail(NIMLLM_ERR_CUDA, "attn_prefill: cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NIMLLM_ERR_CUDA, "attn_prefill: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return NIMLLM_OK;
}

}  // namespace

int g_prefill_variant = 1;

int launch_prefill_tc2(void *q, const void *k, const void *v, void *out, float *lse, const float *cos_tab,
                       const float *sin_tab, int pos0, int write_back_q, int B, int S, int Hq, int Hkv, int D,
                       float scale, void *workspace, size_t workspace_bytes, cudaStream_t st) {
    if (D != kD) return fail(NIMLLM_ERR_UNSUPPORTED, "attn_prefill bf16: head_dim %d (the tensor-core kernel is built for 128)", D);
    if (!workspace || workspace_bytes < 256) return fail(NIMLLM_ERR_WORKSPACE, "attn_prefill bf16: workspace %zu bytes, need 256", workspace_bytes);
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        return fail(NIMLLM_ERR_ARG, "attn_prefill bf16: q, k, v, out must be 16-byte aligned");
    if ((int64_t)B * S > 0x7fffffff) return fail(NIMLLM_ERR_UNSUPPORTED, "attn_prefill bf16: B*S too large");

    static bool attr_set[64] = {false};
    const size_t smem_bytes = sizeof(Smem) + 1024;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_prefill bf16: shared memory opt-in: %s", cudaGetErrorString(e));
        attr_set[dev] = true;
    }

    CUtensorMap q_map, k_map, v_map;
    int rc;
    if ((rc = make_map2(&q_map, q, (uint64_t)B * S, (uint64_t)Hq * D, 128))) return rc;
    if ((rc = make_map2(&k_map, k, (uint64_t)B * S, (uint64_t)Hkv * D, 64))) return rc;
    if ((rc = make_map2(&v_map, v, (uint64_t)B * S, (uint64_t)Hkv * D, 128))) return rc;

    PairParams p;
    p.q = (__nv_bfloat16 *)q; p.out = (__nv_bfloat16 *)out; p.lse = lse;
    p.cos_tab = cos_tab; p.sin_tab = sin_tab;
    p.status = (int *)workspace;
    p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.pos0 = pos0;
    p.rotate_q = cos_tab ? 1 : 0;
    p.write_back_q = write_back_q;
    p.scale_log2e = scale * kLog2e;

    cudaError_t e = cudaMemsetAsync(workspace, 0, 4, st);
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_prefill bf16: %s", cudaGetErrorString(e));
    const int n_groups = (S + 4 * kBM - 1) / (4 * kBM);
    dim3 grid((unsigned)n_groups * Hq * B * 2);       // clusters of two CTAs (compile-time cluster dims)
    prefill_tc2_kernel<<<grid, kThreads, smem_bytes, st>>>(q_map, k_map, v_map, p);
    NIMLLM_CHECK_LAUNCH("attn_prefill bf16 (CTA pairs)");
    return NIMLLM_OK;
}

}  // namespace nimllm

extern "C" void nimllm_attn_debug_prefill_variant(int which) { nimllm::g_prefill_variant = which; }
