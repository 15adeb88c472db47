// peer.cu -- exchange and merge of KV-sequence-shard partials over NVLink peer memory.
//
// No counterpart in the reference (single GPU, no collective anywhere in src/).  When one long
// sequence's KV rows are sharded over the GPUs of a box, every rank's decode produces one
// (o, m, l) record per (sequence, query head); each rank needs all of them to finish the
// softmax.  Instead of an all-gather collective followed by a merge launch, every rank
//   1. stores its records straight into a slot of EVERY peer's exchange buffer (plain 16-byte
//      stores to peer-mapped memory over NVLink / NVSwitch), fences, and -- when its last CTA is
//      done -- raises its flag on every peer;
//   2. waits, bounded, until all peers' flags for this call have arrived, and merges the records
//      out of its own memory.
// Flags carry a call counter (never reset); buffers are double-slotted by its parity so that a
// fast rank's next call cannot overwrite records a slow rank is still merging.  No multicast
// loads, no multimem: ordinary stores, system-scope fences and acquire loads.  The wait gives up
// after about a second, sets a status word and returns; it never traps or spins forever.
#include <string.h>

#include "common.cuh"

struct nimllm_peer_exchange {
    int rank, world, rows_max, W, device;
    size_t slot_floats;          // world * rows_max * W
    size_t bytes;                // 2 slots of records + flags + ticket
    float *local;                // this rank's buffer (cudaMalloc)
    void *peer_base[16];         // mapped base of every rank's buffer (own entry = local)
    bool imported[16];
    float **peer_table_dev;      // device copy of peer_base
    unsigned long long wait_limit_ns;   // how long wait_combine_kernel polls before it gives up
};

namespace nimllm {
namespace {

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// records [rows, W] of this rank -> slot `rank` of every peer's buffer; the last CTA to finish
// publishes the call counter in every peer's flag word for this rank
//
// The call counter lives in device memory (word kPeerMaxWorld + 1 after the flags) and is advanced by
// the push kernel itself, so a captured CUDA graph can replay the pair of launches.
__global__ void __launch_bounds__(256) push_kernel(const float *__restrict__ rec, PeerPush px, int rows) {
    const unsigned int epoch = peer_push_epoch(px);   // stable until the last CTA of this launch writes it back
    const int n4 = rows * px.W / 4;
    const float4 *src = reinterpret_cast<const float4 *>(rec);
    for (int r = 0; r < px.world; r++) {
        float4 *dst = reinterpret_cast<float4 *>(peer_push_slot(px, r, epoch));
        for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += gridDim.x * blockDim.x) dst[i] = src[i];
    }
    peer_push_publish(px, epoch);
}

// one warp per output row: wait for every rank's flag, then log-sum-exp merge of the world
// records of the row (same arithmetic as combine_kernel in decode.cu)
__global__ void __launch_bounds__(128) wait_combine_kernel(const float *buf, int world, int rows, int rows_max,
                                                           int D, int W, size_t slot_floats, void *out, int out_dtype,
                                                           int *status, unsigned long long limit_ns) {
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    // launched as a programmatic dependent of the kernel that pushes: everything above is free to
    // run early, the pusher's writes (the call counter below) are visible after this point
    grid_dependency_wait();
    if (row >= rows) return;
    const unsigned int *flags = reinterpret_cast<const unsigned int *>(buf + 2 * slot_floats);
    const unsigned int epoch = __ldcg(flags + kPeerMaxWorld + 1);   // written by this rank's push kernel, which has completed
    const int slot = (int)(epoch & 1u);
    bool ok = true;
    if (lane < world) {
        // counters only grow: a peer that is already one call ahead has left this call's records
        // untouched in this slot (its next call uses the other one)
        unsigned long long t0 = 0;
        for (unsigned int it = 0;; ++it) {
            unsigned int f = ld_acquire_sys(flags + lane);
            if ((int)(f - epoch) >= 0) break;
            if ((it & 1023) == 1023) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                else if (now - t0 > limit_ns) { ok = false; break; }
            }
        }
    }
    if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) atomicExch(status, 1);
        return;
    }
    const float *base = buf + (size_t)slot * slot_floats + (size_t)row * W;
    const size_t pstride = (size_t)rows_max * W;
    float mi = -INFINITY, li = 0.f;
    // peers wrote these records while this kernel may already have been running: read them from
    // L2 (the point their stores arrive at), never through a non-coherent path
    if (lane < world) { mi = __ldcg(base + lane * pstride + D); li = __ldcg(base + lane * pstride + D + 1); }
    float M = li > 0.f ? mi : -INFINITY;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float safe = (M == -INFINITY) ? 0.f : M;
    const float w_mine = li > 0.f ? li * ex2((mi - safe) * kLog2e) : 0.f;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.f;
    float wsum = 0.f;
    for (int p = 0; p < world; p++) {
        const float w = __shfl_sync(0xffffffffu, w_mine, p);
        wsum += w;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int d = lane + 32 * j;
            if (d < D) acc[j] = fmaf(w, __ldcg(base + p * pstride + d), acc[j]);
        }
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) {
        const int d = lane + 32 * j;
        if (d < D) store_from_f32(out, out_dtype, (int64_t)row * D + d, acc[j] * inv);
    }
}

}  // namespace
}  // namespace nimllm

using namespace nimllm;

extern "C" {

nimllm_peer_exchange *nimllm_peer_exchange_create(int rank, int world, int rows_max, int head_dim) {
    if (rank < 0 || world < 1 || world > kPeerMaxWorld || rank >= world || rows_max <= 0 || head_dim <= 0 || head_dim % 4) {
        set_error("peer_exchange_create: bad arguments");
        return nullptr;
    }
    nimllm_peer_exchange *x = new nimllm_peer_exchange();
    x->rank = rank; x->world = world; x->rows_max = rows_max; x->W = rec_stride(head_dim);
    x->slot_floats = (size_t)world * rows_max * x->W;
    x->bytes = (2 * x->slot_floats + 2 * kPeerMaxWorld) * sizeof(float);
    cudaGetDevice(&x->device);
    if (cudaMalloc((void **)&x->local, x->bytes) != cudaSuccess || cudaMemset(x->local, 0, x->bytes) != cudaSuccess ||
        cudaMalloc((void **)&x->peer_table_dev, kPeerMaxWorld * sizeof(float *)) != cudaSuccess) {
        set_error("peer_exchange_create: cudaMalloc failed");
        delete x;
        return nullptr;
    }
    x->wait_limit_ns = 1000000000ull;
    for (int r = 0; r < kPeerMaxWorld; r++) { x->peer_base[r] = nullptr; x->imported[r] = false; }
    x->peer_base[rank] = x->local;
    cudaDeviceSynchronize();
    return x;
}

/* 64-byte handle another process on the box can open */
int nimllm_peer_exchange_export(nimllm_peer_exchange *x, void *handle_out) {
    if (!x || !handle_out) return fail(NIMLLM_ERR_ARG, "peer_exchange_export: null argument");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, x->local);
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "peer_exchange_export: %s", cudaGetErrorString(e));
    static_assert(sizeof(h) == 64, "IPC handle size");
    memcpy(handle_out, &h, 64);
    return NIMLLM_OK;
}

int nimllm_peer_exchange_import(nimllm_peer_exchange *x, int peer_rank, const void *handle) {
    if (!x || !handle || peer_rank < 0 || peer_rank >= x->world)
        return fail(NIMLLM_ERR_ARG, "peer_exchange_import: bad argument");
    if (peer_rank == x->rank) return NIMLLM_OK;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "peer_exchange_import(rank %d): %s", peer_rank, cudaGetErrorString(e));
    x->peer_base[peer_rank] = p;
    x->imported[peer_rank] = true;
    return NIMLLM_OK;
}

/* a peer that lives in THIS process on the same device (tests, or several ranks driven by one
 * process): its buffer is used directly, no IPC handle */
int nimllm_peer_exchange_import_local(nimllm_peer_exchange *x, int peer_rank, nimllm_peer_exchange *peer) {
    if (!x || !peer || peer_rank < 0 || peer_rank >= x->world || peer->rank != peer_rank || peer->world != x->world ||
        peer->rows_max != x->rows_max || peer->W != x->W)
        return fail(NIMLLM_ERR_ARG, "peer_exchange_import_local: the two buffers do not describe the same exchange");
    if (peer_rank == x->rank) return NIMLLM_OK;
    x->peer_base[peer_rank] = peer->local;
    x->imported[peer_rank] = false;           // nothing to close
    return NIMLLM_OK;
}

/* how long a wait for the peers' records may last before it gives up (default 1000 ms) */
int nimllm_peer_exchange_set_wait_limit(nimllm_peer_exchange *x, int milliseconds) {
    if (!x || milliseconds <= 0) return fail(NIMLLM_ERR_ARG, "peer_exchange_set_wait_limit: bad argument");
    x->wait_limit_ns = (unsigned long long)milliseconds * 1000000ull;
    return NIMLLM_OK;
}

/* after every peer has been imported */
int nimllm_peer_exchange_ready(nimllm_peer_exchange *x) {
    if (!x) return fail(NIMLLM_ERR_ARG, "peer_exchange_ready: null handle");
    for (int r = 0; r < x->world; r++)
        if (!x->peer_base[r]) return fail(NIMLLM_ERR_ARG, "peer_exchange_ready: rank %d was not imported", r);
    cudaError_t e = cudaMemcpy(x->peer_table_dev, x->peer_base, kPeerMaxWorld * sizeof(float *), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "peer_exchange_ready: %s", cudaGetErrorString(e));
    return NIMLLM_OK;
}

void nimllm_peer_exchange_destroy(nimllm_peer_exchange *x) {
    if (!x) return;
    cudaDeviceSynchronize();
    for (int r = 0; r < x->world; r++)
        if (x->imported[r]) cudaIpcCloseMemHandle(x->peer_base[r]);
    cudaFree(x->peer_table_dev);
    cudaFree(x->local);
    delete x;
}

}  // extern "C"

namespace nimllm {
PeerPush peer_push_of(const nimllm_peer_exchange *x) {
    PeerPush px;
    px.peers = x->peer_table_dev; px.rank = x->rank; px.world = x->world; px.rows_max = x->rows_max; px.W = x->W;
    px.slot_floats = x->slot_floats;
    return px;
}
int peer_rows_max(const nimllm_peer_exchange *x) { return x->rows_max; }
int peer_head_dim(const nimllm_peer_exchange *x) { return x->W - 4; }
}  // namespace nimllm

extern "C" {

/* bounded wait for every rank's records of this call, then the merge: out [rows, D] */
int nimllm_attn_wait_combine(nimllm_peer_exchange *x, int rows, void *out, int out_dtype, int *status_dev, void *stream) {
    if (!x || !out || !status_dev) return fail(NIMLLM_ERR_ARG, "attn_wait_combine: null argument");
    if (rows <= 0 || rows > x->rows_max) return fail(NIMLLM_ERR_ARG, "attn_wait_combine: rows %d outside 1..%d", rows, x->rows_max);
    if (!dtype_ok(out_dtype)) return fail(NIMLLM_ERR_ARG, "attn_wait_combine: unknown dtype");
    const int D = x->W - 4;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((rows + 3) / 4); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = 0; cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, wait_combine_kernel, (const float *)x->local, x->world, rows, x->rows_max, D, x->W,
                                       x->slot_floats, out, out_dtype, status_dev, x->wait_limit_ns);
    if (e != cudaSuccess) return fail(NIMLLM_ERR_CUDA, "attn_wait_combine: %s", cudaGetErrorString(e));
    return NIMLLM_OK;
}

/* records [rows, D+4] of this rank in, merged output [rows, D] out; status_dev (device int,
 * caller-zeroed) becomes 1 if a peer's records did not arrive within the wait limit */
int nimllm_attn_combine_peers(nimllm_peer_exchange *x, const float *rec_local, int rows, void *out, int out_dtype,
                              int *status_dev, void *stream) {
    if (!x || !rec_local || !out || !status_dev) return fail(NIMLLM_ERR_ARG, "attn_combine_peers: null argument");
    if (rows <= 0 || rows > x->rows_max) return fail(NIMLLM_ERR_ARG, "attn_combine_peers: rows %d outside 1..%d", rows, x->rows_max);
    if (!dtype_ok(out_dtype)) return fail(NIMLLM_ERR_ARG, "attn_combine_peers: unknown dtype");
    if ((uintptr_t)rec_local & 15) return fail(NIMLLM_ERR_ARG, "attn_combine_peers: records must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    int blocks = (rows * x->W / 4 + 255) / 256;
    if (blocks > 32) blocks = 32;
    push_kernel<<<blocks, 256, 0, st>>>(rec_local, peer_push_of(x), rows);
    NIMLLM_CHECK_LAUNCH("attn_combine_peers push");
    return nimllm_attn_wait_combine(x, rows, out, out_dtype, status_dev, stream);
}

}  // extern "C"
