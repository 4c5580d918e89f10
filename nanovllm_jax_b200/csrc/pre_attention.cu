// qk_norm_rope_store: the stand-alone launch of the fused pre-attention step (see pre_attention.cuh); the decode
// step that folds it into its first kernel lives in paged_decode.cu.
#include "pre_attention.cuh"

namespace nvllm {
namespace preattn {

__global__ void __launch_bounds__(kThreads) pre_attention_kernel(const Params p) {
    griddep_wait();  // q, k, v may come from the kernel just before this one (the QKV projection)
    griddep_launch_dependents();
    pre_attention_block(blockIdx.x, p);
}

int check_args(const char* who, const void* q, const void* k, const void* v, const float* q_weight, const float* k_weight,
               const float* cos_sin_cache, const int32_t* positions, const void* k_cache, const void* v_cache,
               const int32_t* slot_mapping, int64_t T, int H, int KVH, int D, int64_t num_slots, int64_t max_pos) {
    if (T < 0 || H <= 0 || KVH <= 0 || num_slots < 0 || max_pos <= 0)
        return fail(NVLLM_B200_EINVAL, "%s: bad size (T=%lld H=%d KVH=%d num_slots=%lld max_pos=%lld)", who, (long long)T,
                    H, KVH, (long long)num_slots, (long long)max_pos);
    if (D != kD) return fail(NVLLM_B200_EUNSUPPORTED, "%s: head_dim %d (only 128)", who, D);
    if (T == 0) return NVLLM_B200_OK;
    if (!q || !k || !v || !q_weight || !k_weight || !cos_sin_cache || !positions || !k_cache || !v_cache || !slot_mapping)
        return fail(NVLLM_B200_EINVAL, "%s: null pointer", who);
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q_weight |
         (uintptr_t)k_weight | (uintptr_t)cos_sin_cache) & 15)
        return fail(NVLLM_B200_EINVAL, "%s: buffers must be 16-byte aligned", who);
    if (blocks_for(T, H, KVH) > 0x3fffffffLL) return fail(NVLLM_B200_EUNSUPPORTED, "%s: too many rows", who);
    return NVLLM_B200_OK;
}

}  // namespace preattn
}  // namespace nvllm

extern "C" int nvllm_b200_qk_norm_rope_store(void* q, void* k, const void* v, const float* q_weight, const float* k_weight,
                                             const float* cos_sin_cache, const int32_t* positions, void* k_cache,
                                             void* v_cache, const int32_t* slot_mapping, int64_t T, int H, int KVH, int D,
                                             int64_t num_slots, int64_t max_pos, float eps, void* stream) {
    using namespace nvllm;
    int rc = preattn::check_args("qk_norm_rope_store", q, k, v, q_weight, k_weight, cos_sin_cache, positions, k_cache,
                                 v_cache, slot_mapping, T, H, KVH, D, num_slots, max_pos);
    if (rc || T == 0) return rc;
    preattn::Params p{(__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, q_weight, k_weight, cos_sin_cache,
                      positions, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slot_mapping, T, H, KVH, num_slots,
                      max_pos, eps};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)preattn::blocks_for(T, H, KVH));
    cfg.blockDim = dim3(preattn::kThreads);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, preattn::pre_attention_kernel, p));
    return NVLLM_B200_OK;
}
