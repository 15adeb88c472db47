// common.cuh -- shared host/device helpers of the attention library (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/nimllm_attn.h"

namespace nimllm {

// ---- error reporting (thread-local message behind nimllm_attn_last_error) ----
void set_error(const char *fmt, ...);
int fail(int code, const char *fmt, ...);

#define NIMLLM_CHECK_LAUNCH(what)                                                      \
    do {                                                                               \
        cudaError_t e_ = cudaGetLastError();                                           \
        if (e_ != cudaSuccess)                                                         \
            return ::nimllm::fail(NIMLLM_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e_)); \
    } while (0)

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// one partial record: o[D] (normalised), m (natural-log domain), l, 2 pad floats
__host__ __device__ inline int rec_stride(int D) { return D + 4; }

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
}

// 16-byte streaming load that does not allocate in L1 (KV rows are read once)
__device__ __forceinline__ uint4 ldg_stream(const void *p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <typename T> struct Elem;
template <> struct Elem<float> {
    static constexpr int kVec = 4;  // elements per 16 bytes
    __device__ static void unpack(const uint4 &u, float *f) {
        f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
    }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kVec = 8;
    __device__ static void unpack(const uint4 &u, float *f) {
        f[0] = bf16lo(u.x); f[1] = bf16hi(u.x); f[2] = bf16lo(u.y); f[3] = bf16hi(u.y);
        f[4] = bf16lo(u.z); f[5] = bf16hi(u.z); f[6] = bf16lo(u.w); f[7] = bf16hi(u.w);
    }
};

__device__ __forceinline__ float load_as_f32(const void *base, int dtype, int64_t i) {
    return dtype == NIMLLM_F32 ? reinterpret_cast<const float *>(base)[i]
                               : __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(base)[i]);
}
__device__ __forceinline__ void store_from_f32(void *base, int dtype, int64_t i, float x) {
    if (dtype == NIMLLM_F32) reinterpret_cast<float *>(base)[i] = x;
    else reinterpret_cast<__nv_bfloat16 *>(base)[i] = __float2bfloat16_rn(x);
}

// ---- programmatic dependent launch: a kernel launched with the programmatic-serialization
// attribute may start while its predecessor still runs; it must not touch the predecessor's
// results before grid_dependency_wait().  launch_dependents() lets the successor's CTAs be
// scheduled early.  Both are no-ops in a launch without the attribute.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- where a kernel stores finished (o, m, l) records for the other ranks of a KV-sequence-
// sharded decode (peer.cu owns the buffers).  Buffer of a rank: 2 slots of [world][rows_max][W]
// floats, then kPeerMaxWorld flag words, then {CTA ticket, call counter}.
constexpr int kPeerMaxWorld = 16;
struct PeerPush {
    float *const *peers;     // device table: base of every rank's buffer (own entry included)
    int rank, world, rows_max, W;
    size_t slot_floats;      // world * rows_max * W
};
__device__ __forceinline__ unsigned int *peer_ctl(const PeerPush &px, int r) {
    return reinterpret_cast<unsigned int *>(px.peers[r] + 2 * px.slot_floats);
}
// call counter of this launch; the counter lives in device memory and is advanced by the last
// CTA of the pushing launch, so a captured CUDA graph can replay the step
__device__ __forceinline__ unsigned int peer_push_epoch(const PeerPush &px) { return peer_ctl(px, px.rank)[kPeerMaxWorld + 1] + 1u; }
// this rank's records in rank r's buffer (double-slotted by the counter's parity, so a fast
// rank's next call cannot overwrite records a slow rank is still merging)
__device__ __forceinline__ float *peer_push_slot(const PeerPush &px, int r, unsigned int epoch) {
    return px.peers[r] + (size_t)(epoch & 1u) * px.slot_floats + (size_t)px.rank * px.rows_max * px.W;
}
// called by every thread of every CTA after its stores: the last CTA to get here advances the
// counter and raises this rank's flag on every peer (plain stores + system-scope release)
__device__ __forceinline__ void peer_push_publish(const PeerPush &px, unsigned int epoch) {
    // the CTA's stores happen-before thread 0 through the barrier; its system-scope fence then orders all of
    // them (fences are cumulative) before the counter and, in the last CTA, before the flags
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        unsigned int *ctl = peer_ctl(px, px.rank) + kPeerMaxWorld;
        if (atomicAdd(&ctl[0], 1u) == gridDim.x - 1) {
            ctl[0] = 0u;
            ctl[1] = epoch;
            __threadfence_system();
            for (int r = 0; r < px.world; r++)
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peer_ctl(px, r) + px.rank), "r"(epoch) : "memory");
        }
    }
}

inline size_t dtype_size(int dtype) { return dtype == NIMLLM_F32 ? 4 : 2; }
inline bool dtype_ok(int dtype) { return dtype == NIMLLM_F32 || dtype == NIMLLM_BF16; }

int sm_count();  // multiprocessors of the current device (cached per device)

// ---- kernel launchers implemented in the .cu files (device pointers, validated args) ----
int launch_rope_append(void *q, int Hq, void *k_new, const void *v_new, int act_dtype,
                       int write_back_k, const float *cos_tab, const float *sin_tab,
                       const int32_t *seq_pos, int pos0, void *k_cache, void *v_cache,
                       int cache_dtype, const int64_t *kv_off, int64_t seq_stride,
                       int64_t head_stride, int cache_row0, int max_seq, int B, int n, int Hkv,
                       int D, cudaStream_t st, const int32_t *page_table = nullptr, int max_pages = 0,
                       int page_shift = 0, int n_pages = 0);

int launch_prefill_f32(const float *q, const float *k, const float *v, float *out, float *lse,
                       int B, int S, int Hq, int Hkv, int D, float scale, int causal,
                       cudaStream_t st);

int launch_prefill_tc(void *q, const void *k, const void *v, void *out, float *lse,
                      const float *cos_tab, const float *sin_tab, int pos0, int write_back_q,
                      int B, int S, int Hq, int Hkv, int D, float scale, cudaStream_t st);

int prefill_tc_status(int reset, int *status_out);

}  // namespace nimllm

struct nimllm_peer_exchange;
namespace nimllm {
PeerPush peer_push_of(const nimllm_peer_exchange *x);
int peer_rows_max(const nimllm_peer_exchange *x);
int peer_head_dim(const nimllm_peer_exchange *x);
}  // namespace nimllm
