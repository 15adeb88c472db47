// prefill_tc.cu -- causal GQA prefill attention on the Blackwell tensor cores (bf16, D = 128 or 64).
//
// Replaces, for bf16 activations, the per-query-head loop of forward() in the reference
// (src/model.nim:498-508: gather, cublasSgemm_v2 QK^T, gpu_causal_mask, gpu_softmax_fwd,
// cublasSgemm_v2 PV, scatter -- two S x S matrices through HBM per head) with one
// flash-style kernel: no score matrix leaves the SM.
//
// One CTA owns 256 consecutive query rows of one (sequence, query head) as two 128-row
// tiles and walks the KV sequence in 128-row tiles up to the causal diagonal.
//
//   warp 8      TMA producer: K_j tiles into a 3-slot ring, V_j tiles into a 2-slot ring
//               (cp.async.bulk.tensor, 128-byte swizzle, mbarrier transaction counts; a slot is
//               released by tcgen05.commit when the MMAs that read it have completed).  Q tiles by
//               TMA as well when no RoPE is asked for.
//   warp 9      MMA issuer, converged, one elected lane executes the tcgen05 instructions:
//               S = Q_w K_j^T (both operands from shared memory) and O_w += P_w V_j (P from TMEM,
//               V MN-major from shared memory), cta_group::1, kind::f16, M = N = 128, K = 16, fp32
//               accumulators in TMEM.
//   warps 0-3 / 4-7   softmax group of query tile 0 / 1, one thread per query row (= one TMEM
//               lane).  Per KV tile: ONE TMEM round trip brings the 128 scores of the row into
//               registers (setmaxnreg moves registers from warps 8-11 to these), row max, P =
//               exp2(S*c - m) rounded to bf16 into the tile's own P columns, where the PV MMA
//               reads it as its A operand.  O is rescaled only when a row maximum grows by more
//               than 2^8 (the exact softmax is restored by the final division by the running
//               sum); the epilogue normalises, rounds and writes O.
//
// TMEM (512 columns): S | P0 P1 | O0 | O1.  The two query tiles SHARE the one S accumulator: a
// score tile only has to live until its softmax group has pulled it into registers, and the two
// groups take turns.  Because P has columns of its own, Q_w K_{j+1}^T is computed while the
// softmax of tile j still runs, and P_w V_j while the softmax of tile j+1 runs: a group goes from
// one tile's softmax straight into the next one's, and no MMA sits on that chain.  Order of the
// issuer: S fills alternate between the tiles (each waits only for the previous fill to have been
// read out), every end of a softmax triggers that tile's PV and the other tile's next fill.
//
// RoPE: K arrives already rotated (the pre-pass that also fills the KV cache rotates it in
// place, as the reference does and stores); Q is rotated by this kernel's prologue while it is
// staged into the swizzled shared-memory tile (coalesced, 8 lanes per row), and written back
// only when the caller keeps it (save_cache).
//
// Every wait on an mbarrier is bounded: after ~2 s without progress the CTA raises an abort
// flag, all roles leave their loops, TMEM is released and a status word is set.
#include "tcgen05.cuh"

namespace nimllm {

namespace {

using namespace tc;
// packed fp32 arithmetic: two IEEE fp32 operations per instruction, each rounded like its scalar form
__device__ __forceinline__ uint64_t pair2(float a, float b) { uint64_t r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b)); return r; }
__device__ __forceinline__ void unpair2(uint64_t v, float &a, float &b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2_f32(uint64_t a, uint64_t b, uint64_t c) { uint64_t r; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c)); return r; }
__device__ __forceinline__ uint64_t add2_f32(uint64_t a, uint64_t b) { uint64_t r; asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b)); return r; }

// Sticky per-device status of the bf16 prefill: becomes 1 when a bounded wait inside a launch gave
// up (the outputs of that launch are then incomplete) and stays 1 until the host clears it through
// nimllm_attn_prefill_status.
__device__ int g_prefill_status = 0;

constexpr int kBM = 128;           // query rows per tile (= TMEM lanes)
constexpr int kBN = 128;           // KV rows per tile
constexpr int kKSlots = 3;          // ring of K tiles
constexpr int kVSlots = 2;          // ring of V tiles
// head_dim kD is a template parameter (128 or 64): a [128 x kD] bf16 tile is kD/64 swizzled 64-column
// boxes of 16 KiB
template <int kD> constexpr int tile_bytes() { return kBN * kD * 2; }
constexpr int kThreads = 384;                // 8 softmax warps + one warpgroup holding producer, MMA issuer, 2 idle
constexpr uint32_t kTmemCols = 512;
constexpr int kBarSFree = 1, kBarPReady = 2;     // named barriers (0 is __syncthreads): 128 arriving threads + the issuing warp
constexpr uint32_t kColS = 0, kColP = 128, kColO = 256;   // S (shared by both tiles) | P0 P1 | O0 O1
constexpr float kRescaleThreshold = 8.0f;    // log2 units: O is rescaled when a row maximum grows by more

template <int kD> struct Smem {
    // tiles first: 1024-byte alignment is required by the 128-byte swizzle atoms
    uint8_t q[2][tile_bytes<kD>()];
    uint8_t k[kKSlots][tile_bytes<kD>()];
    uint8_t v[kVSlots][tile_bytes<kD>()];
    uint64_t q_full[2], k_full[kKSlots], k_empty[kKSlots], v_full[kVSlots], v_empty[kVSlots];
    uint64_t s_full[2], pv_done[2], o_full[2], drain;
    uint32_t tmem_base;
    volatile int abort_flag;
};

struct PrefillParams {
    __nv_bfloat16 *q;        // [B, S, Hq*D], read by the prologue when it rotates Q
    __nv_bfloat16 *out;      // [B, S, Hq*D]
    float *lse;              // [B, Hq, S] or null
    const float *cos_tab, *sin_tab;  // rows pos0.. used when rotate_q
    int B, S, Hq, Hkv, pos0;
    int rotate_q;            // 1: stage Q through registers with RoPE; 0: Q is loaded by TMA
    int write_back_q;        // with rotate_q: also store the rotated Q to global
    float scale_log2e;
};

// ------------------------------------------------------------------ kernel
template <int kD>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap k_map,
                  const __grid_constant__ CUtensorMap v_map, PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    static_assert(kD == 64 || kD == 128, "head_dim 64 or 128");
    constexpr int kTileBytes = tile_bytes<kD>();
    constexpr int kBoxes = kD / 64;
    Smem<kD> &sm = *reinterpret_cast<Smem<kD> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = p.Hq / p.Hkv;
    const int n_pairs = (p.S + 2 * kBM - 1) / (2 * kBM);
    // Schedule: heaviest query-tile pairs first (their CTAs run 2t + 2 KV tiles); consecutive
    // CTAs walk the query heads of one sequence, so the heads sharing a KV head stream its
    // tiles out of L2 together.  (Grouping all CTAs of one KV head instead was measured: same
    // K/V feed rate, worse balance.)
    const int per_pair = p.Hq * p.B;
    const int t = n_pairs - 1 - (int)blockIdx.x / per_pair;
    const int rem = (int)blockIdx.x % per_pair;
    const int b = rem / p.Hq, h = rem % p.Hq;
    const int kvh = h / G;
    const int nkv_total = (p.S + kBN - 1) / kBN;
    const int row_base = t * 2 * kBM;                 // first query row of tile 0
    const bool active1 = row_base + kBM < p.S;
    const int n0 = min(2 * t + 1, nkv_total);
    const int n1 = active1 ? min(2 * t + 2, nkv_total) : 0;
    const int nmax = max(n0, n1);
    volatile int *abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full[0], p.rotate_q ? 8 : 1);
        mbar_init(&sm.q_full[1], p.rotate_q ? 8 : 1);
        for (int s = 0; s < kKSlots; s++) { mbar_init(&sm.k_full[s], 1); mbar_init(&sm.k_empty[s], 1); }
        for (int s = 0; s < kVSlots; s++) { mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_empty[s], 1); }
        for (int w = 0; w < 2; w++) {
            mbar_init(&sm.s_full[w], 1); mbar_init(&sm.pv_done[w], 1);
            mbar_init(&sm.o_full[w], 1);
        }
        mbar_init(&sm.drain, 1);
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm.tmem_base;

    // Registers follow the work: the softmax warpgroups hold a whole row of S (128 values) plus
    // the packed P, the third warpgroup only issues copies and MMAs.  168 per thread at launch;
    // setmaxnreg.inc can only take what the CTA's own warps gave back with setmaxnreg.dec, and it
    // blocks (for ever) when that is not enough: 4 warps x (168 - 72) = 8 warps x (216 - 168).
    if (warp == 8) {
        // ---------------------------------------------------------------- TMA producer
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        if (lane == 0) {
            const int qx = h * kD, kx = kvh * kD;
            const int y0 = b * p.S + row_base;
            if (!p.rotate_q) {
                mbar_expect_tx(&sm.q_full[0], kTileBytes);
                if (active1) mbar_expect_tx(&sm.q_full[1], kTileBytes);
                for (int bx = 0; bx < kBoxes; bx++) {
                    tma_load_2d(sm.q[0] + bx * kBoxBytes, &q_map, qx + bx * 64, y0, &sm.q_full[0]);
                    if (active1) tma_load_2d(sm.q[1] + bx * kBoxBytes, &q_map, qx + bx * 64, y0 + kBM, &sm.q_full[1]);
                }
            }
            // K_j goes to slot j % kKSlots (phase (j / kKSlots) & 1), V_j to slot j % kVSlots; loads
            // are issued in the order the issuer first needs them: K_0 K_1 V_0 K_2 V_1 K_3 ...
            auto load = [&](uint8_t *dst, const CUtensorMap *map, int j, uint64_t *full) {
                mbar_expect_tx(full, kTileBytes);
                for (int bx = 0; bx < kBoxes; bx++)
                    tma_load_2d(dst + bx * kBoxBytes, map, kx + bx * 64, b * p.S + j * kBN, full);
            };
            bool ok = true;
            for (int j = 0; ok && j <= nmax; j++) {
                if (j < nmax) {
                    if (!(ok = mbar_wait(&sm.k_empty[j % kKSlots], ((j / kKSlots) & 1) ^ 1, abort_flag))) break;
                    load(sm.k[j % kKSlots], &k_map, j, &sm.k_full[j % kKSlots]);
                }
                if (j >= 1) {
                    const int jv = j - 1;
                    if (!(ok = mbar_wait(&sm.v_empty[jv % kVSlots], ((jv / kVSlots) & 1) ^ 1, abort_flag))) break;
                    load(sm.v[jv % kVSlots], &v_map, jv, &sm.v_full[jv % kVSlots]);
                }
            }
        }
    } else if (warp == 9) {
        // ---------------------------------------------------------------- MMA issuer
        // The warp stays converged: descriptors are warp-uniform values (no per-lane copies to
        // move into uniform registers), the tcgen05 instructions execute in one elected lane.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        {
            const uint32_t leader = elect_one();
            constexpr uint32_t idesc_qk = instr_desc(kBM, kBN, 0, 0);   // A, B K-major
            constexpr uint32_t idesc_pv = instr_desc(kBM, kD, 0, 1);    // A from TMEM, B (V) MN-major
            // descriptor words: start address >> 4 | leading byte offset >> 4 << 16 in the low word,
            // stride byte offset 1024 B, version 1 and the 128-byte swizzle in the high word
            constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
            constexpr uint32_t kLboK = 1u << 16;                         // K-major operands: 16 B
            constexpr uint32_t kLboV = (uint32_t)(kBoxBytes >> 4) << 16; // MN-major V: 64-column boxes 16 KiB apart
            const uint32_t q_lo0 = ((smem_u32(sm.q[0]) >> 4) & 0x3FFFu) | kLboK, q_lo1 = ((smem_u32(sm.q[1]) >> 4) & 0x3FFFu) | kLboK;
            const uint32_t k_base = smem_u32(sm.k[0]), v_base = smem_u32(sm.v[0]);
            const uint32_t s_tmem = tmem + kColS;
            bool ok = true;
            // S = Q_w K_j^T : kD/16 steps of 16 along D; both operands K-major, 128-byte swizzle,
            // 1024 bytes between 8-row groups; a step advances 32 bytes inside the 128-byte row
            auto issue_fill = [&](int w, int j) {
                tc_fence_after();
                const uint32_t k_lo = (((k_base + (uint32_t)(j % kKSlots) * kTileBytes) >> 4) & 0x3FFFu) | kLboK;
#pragma unroll
                for (int ks = 0; ks < kD / 16; ks++) {
                    const uint32_t c = (uint32_t)((ks >> 2) * (kBoxBytes >> 4) + (ks & 3) * 2);
                    mma_ss_if(leader, s_tmem, make_desc((w ? q_lo1 : q_lo0) + c, kDescHi), make_desc(k_lo + c, kDescHi), idesc_qk, ks > 0);
                }
                tc_commit_if(leader, w ? &sm.s_full[1] : &sm.s_full[0]);
                // K_j is done with once the last tile that attends it has its scores: tile 1 when
                // it is active (it always attends at least as many KV tiles), else tile 0
                if (w == 1 || j >= n1) tc_commit_if(leader, &sm.k_empty[j % kKSlots]);
            };
            // O_w += P_w V_j : 8 steps of 16 KV rows; P (bf16 pairs, 8 columns per step) from TMEM,
            // V MN-major: 16 rows = 2048 bytes per step
            auto issue_pv = [&](int w, int j) {
                tc_fence_after();
                const uint32_t v_lo = (((v_base + (uint32_t)(j % kVSlots) * kTileBytes) >> 4) & 0x3FFFu) | kLboV;
#pragma unroll
                for (int ks = 0; ks < kBN / 16; ks++)
                    mma_ts_if(leader, tmem + kColO + (w ? 128u : 0u), tmem + kColP + (w ? 64u : 0u) + ks * 8,
                              make_desc(v_lo + ks * 128, kDescHi), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
                tc_commit_if(leader, w ? &sm.pv_done[1] : &sm.pv_done[0]);   // P_w may be overwritten, O_w may be rescaled
                if (j == (w ? n1 : n0) - 1) tc_commit_if(leader, w ? &sm.o_full[1] : &sm.o_full[0]);
            };

            // Hand-overs from the softmax groups (scores read out of TMEM, P stored) come through
            // named hardware barriers: a look at a shared-memory barrier costs this warp several
            // hundred cycles while the tensor cores stream operands out of shared memory, a
            // barrier.sync a few tens.  The order is fixed and is the order of the events: every
            // end of a softmax (tile w, KV tile i) is followed by that group reading its next
            // scores, which lets the OTHER tile's next scores be computed, and by P_w(i) V_i.
            int fills = 0, k_known = -1, v_known = -1;
            auto fill = [&](int w, int j) {
                if (!ok) return;
                if (fills > 0) { named_sync(kBarSFree, 160); if (*abort_flag) { ok = false; return; } }
                // each tile's Q has a barrier of its own: tile 0 starts while tile 1 is still being rotated
                if (j == 0 && !(ok = mbar_wait(&sm.q_full[w], 0, abort_flag))) return;
                if (j > k_known) {
                    if (!(ok = mbar_wait(&sm.k_full[j % kKSlots], (j / kKSlots) & 1, abort_flag))) return;
                    k_known = j;
                }
                issue_fill(w, j);
                fills++;
            };
            auto pv = [&](int w, int j) {
                if (!ok) return;
                named_sync(kBarPReady + w, 160);
                if (*abort_flag) { ok = false; return; }
                if (j > v_known) {
                    if (!(ok = mbar_wait(&sm.v_full[j % kVSlots], (j / kVSlots) & 1, abort_flag))) return;
                    v_known = j;
                }
                issue_pv(w, j);
            };
            if (0 < n0) fill(0, 0);
            if (0 < n1) fill(1, 0);
            if (1 < n0) fill(0, 1);
            for (int i = 0; ok && i < nmax; i++) {
                // tile 0 finished the softmax of KV tile i and took S_0(i+1) out of TMEM
                if (i + 1 < n1) fill(1, i + 1);
                if (i < n0) pv(0, i);
                // look ahead (the answers come back while this warp sits in the next barrier)
                if (i + 2 < nmax && i + 2 > k_known && mbar_test(&sm.k_full[(i + 2) % kKSlots], ((i + 2) / kKSlots) & 1)) k_known = i + 2;
                // tile 1 finished the softmax of KV tile i and took S_1(i+1) out of TMEM
                if (i + 2 < n0) fill(0, i + 2);
                if (i < n1) pv(1, i);
                if (ok) tc_commit_if(leader, &sm.v_empty[i % kVSlots]);
                if (i + 1 < nmax && i + 1 > v_known && mbar_test(&sm.v_full[(i + 1) % kVSlots], ((i + 1) / kVSlots) & 1)) v_known = i + 1;
            }
            // every MMA issued by this warp has completed once this commit arrives
            tc_commit_if(leader, &sm.drain);
            mbar_wait(&sm.drain, 0, abort_flag);
        }
    } else if (warp < 8) {
        // ---------------------------------------------------------------- softmax groups
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
        const int w = warp >> 2;                       // query tile of this group
        const int r = (warp & 3) * 32 + lane;          // row inside the tile = TMEM lane
        const int qrow = row_base + w * kBM + r;       // query position inside the sequence
        const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_addr = lane_base + kColS;
        const uint32_t p_addr = lane_base + kColP + (w ? 64u : 0u);
        const uint32_t o_addr = lane_base + kColO + (w ? 128u : 0u);
        const int n = w ? n1 : n0;
        const int diag = 2 * t + w;                    // KV tile holding this tile's diagonal
        const float c = p.scale_log2e;
        bool ok = true;

        if (p.rotate_q) {
            // Stage both Q tiles through registers, all 256 softmax threads together: kD/16 lanes
            // per row, lane c of a row owns columns [8c, 8c+8) and their rotation partners
            // [kD/2+8c, kD/2+8c+8), so global reads (q and the cos/sin rows) are fully coalesced and
            // the bf16 results drop into the swizzled tile without bank conflicts.  Rotated
            // values also go back to global when the caller keeps Q (saveCache).
            constexpr int kLpr = kD / 16;                      // lanes per row
            constexpr int kRpw = 32 / kLpr;                    // rows per warp and step; 8 warps cover 8 * kRpw rows
            const int c8 = (lane % kLpr) * 8;
#pragma unroll 1
            for (int half_i = 0; half_i < kLpr / 4; half_i++) {      // batches of four steps
                // all 24 loads of four steps are issued before any of them is used
                uint4 lo[4], hi[4];
                float4 cs0[4], cs1[4], sn0[4], sn1[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int row = (half_i * 4 + u) * (8 * kRpw) + warp * kRpw + lane / kLpr;     // 0..255 over both tiles
                    const int pos = row_base + row;
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
                    const int row = (half_i * 4 + u) * (8 * kRpw) + warp * kRpw + lane / kLpr;
                    const int tile_i = row >> 7, rr = row & 127;
                    const int pos = row_base + row;
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
                // a batch of four steps covers 128 rows at head size 128 (= one query tile: hand it
                // over now) and all 256 rows at head size 64; the generic-proxy stores are made
                // visible to the tensor core's async proxy first
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    if (kLpr / 4 == 2) mbar_arrive(&sm.q_full[half_i]);
                    else { mbar_arrive(&sm.q_full[0]); mbar_arrive(&sm.q_full[1]); }
                }
            }
        }

        float m_ref = -INFINITY, l = 0.f;
        for (int j = 0; j < n; j++) {
            // warp-uniform outcome: the aligned TMEM instructions below need the whole warp
            if (!(ok = __all_sync(0xffffffffu, mbar_wait(&sm.s_full[w], j & 1, abort_flag)))) break;
            tc_fence_after();
            const bool masked = (j == diag);
            const int col0 = j * kBN;

            // the whole row of S in registers with ONE TMEM round trip (four loads in flight)
            uint32_t v[128];
            tmem_ld32(s_addr, v);
            tmem_ld32(s_addr + 32, v + 32);
            tmem_ld32(s_addr + 64, v + 64);
            tmem_ld32(s_addr + 96, v + 96);
            tc_wait_ld();
            // the scores are in registers: the other tile's next scores may take their place
            tc_fence_before();
            __syncwarp();
            named_arrive(kBarSFree, 160);

            // the diagonal tile: columns past the row's own position drop out (exp2(-inf) = 0); every
            // other tile goes straight to the unmasked code below
            if (masked) {
#pragma unroll
                for (int i = 0; i < 128; i++)
                    if (col0 + i > qrow) v[i] = 0xff800000u;
            }
            // row maximum of the raw scores, four independent chains
            float mx;
            {
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
            if (j == 0) {
                m_ref = mx_s;
            } else if (mx_s > m_ref + kRescaleThreshold) {
                corr = ex2(m_ref - mx_s);
                m_ref = mx_s;
                l *= corr;
                grow = true;
            }
            if (__any_sync(0xffffffffu, grow)) {
                // rare: bring O down to the new reference maximum, once the PV products of the
                // tile before (issued while this softmax was starting) have landed in O
                if (!(ok = __all_sync(0xffffffffu, mbar_wait(&sm.pv_done[w], (j - 1) & 1, abort_flag)))) break;
                tc_fence_after();
#pragma unroll 1
                for (int ch = 0; ch < kD / 32; ch++) {
                    uint32_t o[32];
                    tmem_ld32(o_addr + ch * 32, o);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                    tmem_st32(o_addr + ch * 32, o);
                }
                tc_wait_st();
            }

            // P = exp2(S*c - m_ref) as bf16 pairs, for the tile's own P columns
            const float neg_m = -m_ref;
            uint64_t sum01 = 0ull, sum23 = 0ull;
            const uint64_t c2 = pair2(c, c), nm2 = pair2(neg_m, neg_m);
            uint32_t pk[64];
            bool p_free = (j == 0);
#pragma unroll
            for (int i = 0; i < 128; i += 4) {
                // half-way: has the PV of the tile before finished with the P columns?  (asked here,
                // so that the answer is back when the stores below need it)
                if (i == 64 && j > 0) p_free = mbar_test(&sm.pv_done[w], (j - 1) & 1);
                // scale-and-shift and the row sum as packed fp32 operations (two per instruction)
                float x[4], e[4];
                unpair2(fma2_f32(pair2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), c2, nm2), x[0], x[1]);
                unpair2(fma2_f32(pair2(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])), c2, nm2), x[2], x[3]);
#pragma unroll
                for (int u = 0; u < 4; u++) e[u] = ex2(x[u]);
                sum01 = add2_f32(sum01, pair2(e[0], e[1]));
                sum23 = add2_f32(sum23, pair2(e[2], e[3]));
                pk[i >> 1] = pack_bf16(e[0], e[1]);
                pk[(i >> 1) + 1] = pack_bf16(e[2], e[3]);
            }
            {
                float sum0, sum1, sum2, sum3;
                unpair2(sum01, sum0, sum1); unpair2(sum23, sum2, sum3);
                l += (sum0 + sum1) + (sum2 + sum3);
            }
            // P_w(j-1) must have been consumed (its PV was issued when the previous softmax ended)
            if (j > 0) {
                if (!__all_sync(0xffffffffu, p_free) &&
                    !(ok = __all_sync(0xffffffffu, mbar_wait(&sm.pv_done[w], (j - 1) & 1, abort_flag)))) break;
                tc_fence_after();
            }
            tmem_st32(p_addr, pk);
            tmem_st32(p_addr + 32, pk + 32);
            tc_wait_st();
            tc_fence_before();
            named_arrive(kBarPReady + w, 160);
        }

        if (!ok) {
            // giving up: the issuing warp may sit in one of the named barriers this group feeds;
            // let it through (it looks at the abort flag behind every barrier)
            named_arrive(kBarSFree, 160);
            named_arrive(kBarPReady + w, 160);
        }
        // epilogue: O / l -> bf16 -> global
        if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait(&sm.o_full[w], 0, abort_flag));
        if (ok && n > 0) {
            tc_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            __nv_bfloat16 *og = p.out + ((int64_t)b * p.S + qrow) * p.Hq * kD + (int64_t)h * kD;
#pragma unroll 1
            for (int ch = 0; ch < kD / 32; ch++) {
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
    }

    else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");   // warps 10, 11: same warpgroup as 8, 9
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && sm.abort_flag) atomicExch(&g_prefill_status, 1);
    if (warp == 9) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

// 2-D bf16 tensor [rows, cols] row-major; box = 64 columns x 128 rows, 128-byte swizzle.
int make_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(NIMLLM_ERR_CUDA, "attn_prefill: cuTensorMapEncodeTiled is not available");
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {64, 128};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NIMLLM_ERR_CUDA, "attn_prefill: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return NIMLLM_OK;
}

// The descriptors of the most recent operands are kept (a model's layers call with the same few
// buffers again and again): a hit costs a lookup instead of three driver calls.
struct MapKey { const void *base; uint64_t rows, cols; };
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
thread_local MapSlot g_maps[8];
thread_local int g_map_next = 0;

int cached_map(CUtensorMap *map, const void *base, uint64_t rows, uint64_t cols) {
    for (int i = 0; i < 8; i++)
        if (g_maps[i].used && g_maps[i].key.base == base && g_maps[i].key.rows == rows && g_maps[i].key.cols == cols) {
            *map = g_maps[i].map;
            return NIMLLM_OK;
        }
    const int rc = make_map(map, base, rows, cols);
    if (rc) return rc;
    MapSlot &s = g_maps[g_map_next];
    g_map_next = (g_map_next + 1) % 8;
    s.key = MapKey{base, rows, cols}; s.map = *map; s.used = true;
    return NIMLLM_OK;
}

template <int kD>
int launch_prefill_tc_d(void *q, const void *k, const void *v, void *out, float *lse, const float *cos_tab,
                        const float *sin_tab, int pos0, int write_back_q, int B, int S, int Hq, int Hkv,
                        float scale, cudaStream_t st) {
    static bool attr_set[64] = {false};
    const size_t smem_bytes = sizeof(Smem<kD>) + 1024;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaError_t e = cudaFuncSetAttribute(prefill_tc_kernel<kD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
        if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_prefill bf16: shared memory opt-in: %s", cudaGetErrorString(e));
        attr_set[dev] = true;
    }

    CUtensorMap q_map, k_map, v_map;
    int rc;
    if ((rc = cached_map(&q_map, q, (uint64_t)B * S, (uint64_t)Hq * kD))) return rc;
    if ((rc = cached_map(&k_map, k, (uint64_t)B * S, (uint64_t)Hkv * kD))) return rc;
    if ((rc = cached_map(&v_map, v, (uint64_t)B * S, (uint64_t)Hkv * kD))) return rc;

    PrefillParams p;
    p.q = (__nv_bfloat16 *)q; p.out = (__nv_bfloat16 *)out; p.lse = lse;
    p.cos_tab = cos_tab; p.sin_tab = sin_tab;
    p.B = B; p.S = S; p.Hq = Hq; p.Hkv = Hkv; p.pos0 = pos0;
    p.rotate_q = cos_tab ? 1 : 0;
    p.write_back_q = write_back_q;
    p.scale_log2e = scale * kLog2e;

    const int n_pairs = (S + 2 * kBM - 1) / (2 * kBM);
    dim3 grid((unsigned)n_pairs * Hq * B);
    prefill_tc_kernel<kD><<<grid, kThreads, smem_bytes, st>>>(q_map, k_map, v_map, p);
    NIMLLM_CHECK_LAUNCH("attn_prefill bf16");
    return NIMLLM_OK;
}

}  // namespace

int launch_prefill_tc(void *q, const void *k, const void *v, void *out, float *lse, const float *cos_tab,
                      const float *sin_tab, int pos0, int write_back_q, int B, int S, int Hq, int Hkv, int D,
                      float scale, cudaStream_t st) {
    if (D != 64 && D != 128)
        return fail(NIMLLM_ERR_UNSUPPORTED, "attn_prefill bf16: head_dim %d (the tensor-core kernel is built for 64 and 128)", D);
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        return fail(NIMLLM_ERR_ARG, "attn_prefill bf16: q, k, v, out must be 16-byte aligned");
    if ((int64_t)B * S > 0x7fffffff) return fail(NIMLLM_ERR_UNSUPPORTED, "attn_prefill bf16: B*S too large");
    if (D == 64)
        return launch_prefill_tc_d<64>(q, k, v, out, lse, cos_tab, sin_tab, pos0, write_back_q, B, S, Hq, Hkv, scale, st);
    return launch_prefill_tc_d<128>(q, k, v, out, lse, cos_tab, sin_tab, pos0, write_back_q, B, S, Hq, Hkv, scale, st);
}

// Reads (and with reset != 0 clears) the sticky status word of the current device.  Synchronises
// the device: call it where the host waits for results anyway.
int prefill_tc_status(int reset, int *status_out) {
    int st = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&st, g_prefill_status, sizeof(int));
    if (e == cudaSuccess && reset && st != 0) {
        const int zero = 0;
        e = cudaMemcpyToSymbol(g_prefill_status, &zero, sizeof(int));
    }
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_prefill_status: %s", cudaGetErrorString(e));
    *status_out = st;
    return NIMLLM_OK;
}

}  // namespace nimllm
