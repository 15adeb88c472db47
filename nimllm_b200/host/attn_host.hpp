// attn_host.hpp -- C++ host layer over the C ABI, named after the reference's Nim procedures.
//
// nimllm's host code is Nim (compiled to C); no Nim compiler exists on the build image, so the
// host-side mirror a compiled caller would use is given in C++:
//
//   reference (src/model.nim, src/gpu.nim, src/autograd.nim)      here
//   GpuBuf {data, numel}            (src/gpu.nim:114-117)         nimllm::GpuBuf
//   trackedCreate / freeStepAllocations (src/autograd.nim:37-65)  nimllm::Arena (bump allocator)
//   KvCache, initKvCache, resetKvCache  (src/model.nim:70-73,729-746)   nimllm::KvCache
//   forward()'s attention block         (src/model.nim:494-508)   nimllm::attnForward
//   forwardCached()'s attention block   (src/model.nim:788-840)   nimllm::attnForwardCached
//
// Everything computes through include/nimllm_attn.h; nothing here runs on the CPU.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/nimllm_attn.h"

namespace nimllm {

struct GpuBuf {          // src/gpu.nim:114-117
    void *data = nullptr;
    size_t numel = 0;    // float32 elements
};

struct ModelShape {      // the compile-time consts of src/model.nim:12-23, at run time
    int nLayer, nHead, nKvHead, headDim, blockSize;
    int nEmbd() const { return nHead * headDim; }
    int nKvDim() const { return nKvHead * headDim; }
    int kvRepeat() const { return nHead / nKvHead; }
};

// Bump allocator over one device allocation (src/autograd.nim:16-65): 128-byte aligned
// slices, reset once per step; no cudaMalloc between init and destruction.
class Arena {
  public:
    explicit Arena(size_t bytes);
    ~Arena();
    GpuBuf trackedCreate(size_t numel);     // float32 elements, zero-filled by freeStepAllocations
    void *bytes(size_t n);                  // raw slice
    void freeStepAllocations();             // memset of the high-water mark, offset back to 0
    size_t used() const { return off_; }

  private:
    char *base_ = nullptr;
    size_t cap_ = 0, off_ = 0;
};

// One K and one V buffer per layer, [nKvHead, blockSize, headDim] fp32, zero-filled; host pos.
struct KvCache {
    std::vector<GpuBuf> k, v;
    int pos = 0;
};

KvCache initKvCache(const ModelShape &m);
void resetKvCache(KvCache &kv);
void freeKvCache(KvCache &kv);

// RoPE tables as initModel builds them (src/model.nim:153-163), uploaded to the device.
void initRope(const ModelShape &m, float ropeTheta, GpuBuf &ropeCos, GpuBuf &ropeSin);

// forward()'s attention block: q [S,nEmbd], k, v [S,nKvDim] (rotated in place), attnOut [S,nEmbd].
// Returns the ABI status; lastError() explains a non-zero one.
int attnForward(const ModelShape &m, GpuBuf q, GpuBuf k, GpuBuf v, GpuBuf ropeCos, GpuBuf ropeSin,
                GpuBuf attnOut, int S, bool saveCache);

// forwardCached()'s attention block for ONE new token (newTokens == 1) of layer li: RoPE at row
// kv.pos, append, attend rows 0..kv.pos.  The caller advances kv.pos after the last layer.
int attnForwardCached(const ModelShape &m, KvCache &kv, int li, GpuBuf q, GpuBuf kNew, GpuBuf vNew,
                      GpuBuf ropeCos, GpuBuf ropeSin, GpuBuf attnOut, Arena &arena);

// The attention weights of one layer as the reference holds them (src/model.nim:36-47): row-major
// [out, in] matrices, fp32 or -- the GGUF path, src/model.nim:445-450 -- Q8_0 / Q4_0 blocks.
struct AttnWeights {
    const void *wq, *wk, *wv, *wo;
    int wType;               // NIMLLM_W_F32, _BF16, _Q8_0, _Q4_0
};

// forwardCached()'s whole attention part for ONE new token of layer li (src/model.nim:775-849) in three
// launches + one merge: q/k/v projection of xNorm with RoPE and the cache append fused in, attention over
// rows 0..kv.pos, output projection with the residual added: xOut = xResid + wo * attn.  Scratch for q and
// the attention output comes from the arena.  The caller advances kv.pos after the last layer.
int attnStepCached(const ModelShape &m, KvCache &kv, int li, const AttnWeights &w, GpuBuf xNorm, GpuBuf xResid,
                   GpuBuf xOut, GpuBuf ropeCos, GpuBuf ropeSin, Arena &arena);

// Sticky status of the bf16 tensor-core prefill on the current device (0 ok, 1 a launch gave up on a
// bounded wait and left incomplete results); synchronises the device.  Call it where the host waits
// for results anyway -- after a forward pass, before sampling (src/chat.nim:97-101).
int prefillStatus(bool reset = true);

std::string lastError();

}  // namespace nimllm
