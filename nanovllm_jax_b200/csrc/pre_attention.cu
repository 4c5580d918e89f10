// qk_norm_rope_store: the stand-alone launch of the fused pre-attention step (see pre_attention.cuh); the decode
// step that folds it into its first kernel lives in paged_decode.cu.
#include "pre_attention.cuh"

namespace nvllm {
namespace preattn {

// Persistent: the row blocks are dealt round-robin to a grid of a few CTAs per SM, and every thread has the loads of
// kRowsInFlight rows in flight before it starts on the first one.
__global__ void __launch_bounds__(kThreads, 2) pre_attention_kernel(const Params p, const int64_t blocks) {
    griddep_wait();  // q, k, v may come from the kernel just before this one (the QKV projection)
    griddep_launch_dependents();
    const int q = threadIdx.x & 3;
    const int rb = threadIdx.x >> 2;
    for (int64_t b0 = (int64_t)blockIdx.x * kRowsInFlight; b0 < blocks; b0 += (int64_t)gridDim.x * kRowsInFlight) {
        Part c[kRowsInFlight];
#pragma unroll
        for (int u = 0; u < kRowsInFlight; ++u) c[u] = load_part((b0 + u) * kRowsPerBlock + rb, q, p);  // dead past the end
#pragma unroll
        for (int u = 0; u < kRowsInFlight; ++u) finish_part(c[u], q, p);
    }
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
    const int64_t blocks = preattn::blocks_for(T, H, KVH);
    const int64_t groups = (blocks + preattn::kRowsInFlight - 1) / preattn::kRowsInFlight;
    const int64_t resident = (int64_t)sm_count() * 2;  // the launch bounds keep two CTAs of 256 threads on an SM
    cfg.gridDim = dim3((unsigned)(groups < resident ? groups : resident));
    cfg.blockDim = dim3(preattn::kThreads);
    cfg.stream = reinterpret_cast<cudaStream_t>(stream);
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, preattn::pre_attention_kernel, p, blocks));
    return NVLLM_B200_OK;
}
