// attn_host.cpp -- see attn_host.hpp.  Also exports a small extern "C" shim so that the test
// suite can drive this layer through ctypes.
#include "attn_host.hpp"

#include <cuda_runtime.h>

#include <cmath>
#include <stdexcept>

namespace nimllm {

Arena::Arena(size_t bytes) : cap_(bytes) {
    if (cudaMalloc((void **)&base_, bytes) != cudaSuccess) throw std::runtime_error("Arena: cudaMalloc failed");
    cudaMemset(base_, 0, bytes);
}
Arena::~Arena() { cudaFree(base_); }

void *Arena::bytes(size_t n) {
    size_t aligned = (off_ + 127) / 128 * 128;                       // src/autograd.nim:39-41
    if (aligned + n > cap_) throw std::runtime_error("Arena exhausted");
    off_ = aligned + n;
    return base_ + aligned;
}
GpuBuf Arena::trackedCreate(size_t numel) { return GpuBuf{bytes(numel * sizeof(float)), numel}; }
void Arena::freeStepAllocations() {                                  // src/autograd.nim:53-61
    if (off_) cudaMemsetAsync(base_, 0, off_, 0);
    off_ = 0;
}

static GpuBuf gpuCreate(size_t numel) {                              // src/gpu.nim:126-131
    GpuBuf b;
    b.numel = numel;
    if (cudaMalloc(&b.data, numel * sizeof(float)) != cudaSuccess) throw std::runtime_error("gpuCreate: cudaMalloc failed");
    cudaMemset(b.data, 0, numel * sizeof(float));
    return b;
}

KvCache initKvCache(const ModelShape &m) {                           // src/model.nim:729-739
    KvCache kv;
    for (int li = 0; li < m.nLayer; li++) {
        kv.k.push_back(gpuCreate((size_t)m.nKvHead * m.blockSize * m.headDim));
        kv.v.push_back(gpuCreate((size_t)m.nKvHead * m.blockSize * m.headDim));
    }
    kv.pos = 0;
    return kv;
}

void resetKvCache(KvCache &kv) {                                     // src/model.nim:741-746
    for (auto &b : kv.k) cudaMemset(b.data, 0, b.numel * sizeof(float));
    for (auto &b : kv.v) cudaMemset(b.data, 0, b.numel * sizeof(float));
    kv.pos = 0;
}

void freeKvCache(KvCache &kv) {
    for (auto &b : kv.k) cudaFree(b.data);
    for (auto &b : kv.v) cudaFree(b.data);
    kv.k.clear();
    kv.v.clear();
}

void initRope(const ModelShape &m, float ropeTheta, GpuBuf &ropeCos, GpuBuf &ropeSin) {
    size_t n = (size_t)m.blockSize * (m.headDim / 2);
    std::vector<float> c(n), s(n);
    nimllm_rope_tables_host(c.data(), s.data(), m.blockSize, m.headDim, ropeTheta);
    ropeCos = gpuCreate(n);
    ropeSin = gpuCreate(n);
    cudaMemcpy(ropeCos.data, c.data(), n * sizeof(float), cudaMemcpyHostToDevice);
    cudaMemcpy(ropeSin.data, s.data(), n * sizeof(float), cudaMemcpyHostToDevice);
}

int attnForward(const ModelShape &m, GpuBuf q, GpuBuf k, GpuBuf v, GpuBuf ropeCos, GpuBuf ropeSin,
                GpuBuf attnOut, int S, bool saveCache) {
    const float scale = 1.0f / std::sqrt((float)m.headDim);          // src/model.nim:469
    return nimllm_attn_prefill(q.data, k.data, v.data, NIMLLM_F32, (const float *)ropeCos.data,
                               (const float *)ropeSin.data, 0, attnOut.data, 1, S, m.nHead, m.nKvHead, m.headDim,
                               scale, saveCache ? 1 : 0, nullptr, nullptr, NIMLLM_F32, nullptr, 0, 0, 0, nullptr,
                               nullptr, 0, nullptr);
}

int attnForwardCached(const ModelShape &m, KvCache &kv, int li, GpuBuf q, GpuBuf kNew, GpuBuf vNew,
                      GpuBuf ropeCos, GpuBuf ropeSin, GpuBuf attnOut, Arena &arena) {
    if (kv.pos + 1 > m.blockSize) return NIMLLM_ERR_ARG;             // src/chat.nim:96,103 guard
    const float scale = 1.0f / std::sqrt((float)m.headDim);          // src/model.nim:762
    const int64_t seqStride = (int64_t)m.nKvHead * m.blockSize * m.headDim;
    const int64_t headStride = (int64_t)m.blockSize * m.headDim;
    int rc = nimllm_rope_append(q.data, m.nHead, kNew.data, vNew.data, NIMLLM_F32, 1, (const float *)ropeCos.data,
                                (const float *)ropeSin.data, nullptr, kv.pos, kv.k[li].data, kv.v[li].data, NIMLLM_F32,
                                nullptr, seqStride, headStride, 0, m.blockSize, 1, 1, m.nKvHead, m.headDim, nullptr);
    if (rc) return rc;
    const int S = kv.pos + 1;                                        // src/model.nim:754
    size_t wsBytes = nimllm_attn_decode_workspace_bytes(1, m.nHead, m.nKvHead, m.headDim, S, 0);
    void *ws = wsBytes ? arena.bytes(wsBytes) : nullptr;
    return nimllm_attn_decode(q.data, NIMLLM_F32, kv.k[li].data, kv.v[li].data, NIMLLM_F32, nullptr, seqStride,
                              headStride, nullptr, S, attnOut.data, NIMLLM_F32, nullptr, 1, m.nHead, m.nKvHead,
                              m.headDim, scale, 0, ws, wsBytes, nullptr);
}

int attnStepCached(const ModelShape &m, KvCache &kv, int li, const AttnWeights &w, GpuBuf xNorm, GpuBuf xResid,
                   GpuBuf xOut, GpuBuf ropeCos, GpuBuf ropeSin, Arena &arena) {
    if (kv.pos + 1 > m.blockSize) return NIMLLM_ERR_ARG;             // src/chat.nim:96,103 guard
    const float scale = 1.0f / std::sqrt((float)m.headDim);          // src/model.nim:762
    const int64_t seqStride = (int64_t)m.nKvHead * m.blockSize * m.headDim;
    const int64_t headStride = (int64_t)m.blockSize * m.headDim;
    GpuBuf q = arena.trackedCreate((size_t)m.nEmbd()), attn = arena.trackedCreate((size_t)m.nEmbd());
    // src/model.nim:775-815: three mat-vecs, two ropeFwd, 2 * nKvHead copies -> one launch
    int rc = nimllm_qkv_rope_append((const float *)xNorm.data, w.wq, w.wk, w.wv, w.wType, (float *)q.data, nullptr, nullptr,
                                    (const float *)ropeCos.data, (const float *)ropeSin.data, nullptr, kv.pos, kv.k[li].data,
                                    kv.v[li].data, NIMLLM_F32, nullptr, seqStride, headStride, 0, m.blockSize, 1, m.nEmbd(),
                                    m.nHead, m.nKvHead, m.headDim, nullptr);
    if (rc) return rc;
    const int S = kv.pos + 1;                                        // src/model.nim:754
    size_t wsBytes = nimllm_attn_decode_workspace_bytes(1, m.nHead, m.nKvHead, m.headDim, S, 0);
    void *ws = wsBytes ? arena.bytes(wsBytes) : nullptr;
    rc = nimllm_attn_decode(q.data, NIMLLM_F32, kv.k[li].data, kv.v[li].data, NIMLLM_F32, nullptr, seqStride, headStride,
                            nullptr, S, attn.data, NIMLLM_F32, nullptr, 1, m.nHead, m.nKvHead, m.headDim, scale, 0, ws,
                            wsBytes, nullptr);
    if (rc) return rc;
    // src/model.nim:843-849: wo mat-vec + gpu_add -> one launch
    return nimllm_wo_residual((const float *)attn.data, w.wo, w.wType, (const float *)xResid.data, (float *)xOut.data, 1,
                              m.nEmbd(), m.nEmbd(), nullptr);
}

int prefillStatus(bool reset) { return nimllm_attn_prefill_status(reset ? 1 : 0); }

std::string lastError() { return nimllm_attn_last_error(); }

}  // namespace nimllm

// ---------------------------------------------------------------- ctypes shim (tests only)
using namespace nimllm;

struct HostSession {
    ModelShape shape;
    KvCache kv;
    Arena *arena;
    GpuBuf ropeCos, ropeSin;
};

extern "C" {

void *nimllm_host_session_create(int nLayer, int nHead, int nKvHead, int headDim, int blockSize, float ropeTheta,
                                 size_t arenaBytes) {
    try {
        HostSession *s = new HostSession();
        s->shape = ModelShape{nLayer, nHead, nKvHead, headDim, blockSize};
        s->kv = initKvCache(s->shape);
        s->arena = new Arena(arenaBytes);
        initRope(s->shape, ropeTheta, s->ropeCos, s->ropeSin);
        return s;
    } catch (...) {
        return nullptr;
    }
}

void nimllm_host_session_destroy(void *h) {
    HostSession *s = (HostSession *)h;
    freeKvCache(s->kv);
    cudaFree(s->ropeCos.data);
    cudaFree(s->ropeSin.data);
    delete s->arena;
    delete s;
}

int nimllm_host_kv_pos(void *h) { return ((HostSession *)h)->kv.pos; }
void nimllm_host_kv_set_pos(void *h, int pos) { ((HostSession *)h)->kv.pos = pos; }
void nimllm_host_kv_reset(void *h) { resetKvCache(((HostSession *)h)->kv); }
void *nimllm_host_kv_k(void *h, int li) { return ((HostSession *)h)->kv.k[li].data; }
void *nimllm_host_kv_v(void *h, int li) { return ((HostSession *)h)->kv.v[li].data; }

// forward()'s block on device buffers, then the multi-token cache fill (src/model.nim:810-815)
int nimllm_host_attn_forward(void *h, void *q, void *k, void *v, void *attnOut, int S, int saveCache, int fillLayer) {
    HostSession *s = (HostSession *)h;
    const ModelShape &m = s->shape;
    int rc = attnForward(m, GpuBuf{q, (size_t)S * m.nEmbd()}, GpuBuf{k, (size_t)S * m.nKvDim()},
                         GpuBuf{v, (size_t)S * m.nKvDim()}, s->ropeCos, s->ropeSin, GpuBuf{attnOut, (size_t)S * m.nEmbd()},
                         S, saveCache != 0);
    if (rc || fillLayer < 0) return rc;
    // k is rotated now: copy rows 0..S-1 into the cache (no second rotation: tables NULL)
    rc = nimllm_rope_append(nullptr, 0, k, v, NIMLLM_F32, 0, nullptr, nullptr, nullptr, 0, s->kv.k[fillLayer].data,
                            s->kv.v[fillLayer].data, NIMLLM_F32, nullptr, (int64_t)m.nKvHead * m.blockSize * m.headDim,
                            (int64_t)m.blockSize * m.headDim, 0, m.blockSize, 1, S, m.nKvHead, m.headDim, nullptr);
    if (!rc) s->kv.pos = S;
    return rc;
}

int nimllm_host_attn_forward_cached(void *h, int li, void *q, void *kNew, void *vNew, void *attnOut) {
    HostSession *s = (HostSession *)h;
    const ModelShape &m = s->shape;
    try {
        return attnForwardCached(m, s->kv, li, GpuBuf{q, (size_t)m.nEmbd()}, GpuBuf{kNew, (size_t)m.nKvDim()},
                                 GpuBuf{vNew, (size_t)m.nKvDim()}, s->ropeCos, s->ropeSin,
                                 GpuBuf{attnOut, (size_t)m.nEmbd()}, *s->arena);
    } catch (...) {
        return NIMLLM_ERR_WORKSPACE;
    }
}

int nimllm_host_attn_step_cached(void *h, int li, const void *wq, const void *wk, const void *wv, const void *wo, int wType,
                                 void *xNorm, void *xResid, void *xOut) {
    HostSession *s = (HostSession *)h;
    const ModelShape &m = s->shape;
    try {
        return attnStepCached(m, s->kv, li, AttnWeights{wq, wk, wv, wo, wType}, GpuBuf{xNorm, (size_t)m.nEmbd()},
                              GpuBuf{xResid, (size_t)m.nEmbd()}, GpuBuf{xOut, (size_t)m.nEmbd()}, s->ropeCos, s->ropeSin,
                              *s->arena);
    } catch (...) {
        return NIMLLM_ERR_WORKSPACE;
    }
}

void nimllm_host_free_step(void *h) { ((HostSession *)h)->arena->freeStepAllocations(); }

}  // extern "C"
