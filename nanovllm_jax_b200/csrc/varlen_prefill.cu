#include "common.cuh"
extern "C" size_t nvllm_b200_varlen_prefill_workspace_bytes(int64_t, int, int, int, int) { return 0; }
extern "C" int nvllm_b200_varlen_prefill(const void*, const void*, const void*, const int32_t*, const int32_t*,
                                         const int32_t*, void*, void*, size_t, int64_t, int, int, int, int, int, float,
                                         void*) {
    return nvllm::fail(NVLLM_B200_EUNSUPPORTED, "varlen_prefill: kernel not built");
}
