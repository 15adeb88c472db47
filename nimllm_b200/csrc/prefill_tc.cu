// prefill_tc.cu -- placeholder until the tcgen05 kernel lands.
#include "common.cuh"
namespace nimllm {
size_t prefill_tc_workspace_bytes(int, int, int, int, int) { return 0; }
int launch_prefill_tc(void *, const void *, const void *, void *, float *, const float *, const float *, int, int,
                      int, int, int, int, int, float, void *, size_t, cudaStream_t) {
    return fail(NIMLLM_ERR_UNSUPPORTED, "attn_prefill: bf16 tensor-core kernel not built");
}
}
