// store_kvcache: scatter the step's new K/V rows into the paged cache by slot.
//
// Replaces store_kv_to_cache (reference layers/attention.py:42-77).  Pure data
// movement, HBM-bound: per token it reads KVH*D elements of K and of V and
// writes the same number of bf16 elements to each cache, plus one int32 slot.
// The per-block work lives in store_kvcache.cuh (shared with the fused decode step).
#include "store_kvcache.cuh"

namespace nvllm {

template <typename SrcT>
__global__ void __launch_bounds__(kStoreThreads)
store_kvcache_kernel(const SrcT* __restrict__ k, const SrcT* __restrict__ v, __nv_bfloat16* __restrict__ k_cache,
                     __nv_bfloat16* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping, int64_t total_chunks,
                     int row_chunks, int64_t num_slots) {
    griddep_wait();  // k, v and slot_mapping may come from the kernel just before this one
    griddep_launch_dependents();
    store_block<SrcT>(blockIdx.x, k, v, k_cache, v_cache, slot_mapping, total_chunks, row_chunks, num_slots);
}

}  // namespace nvllm

extern "C" int nvllm_b200_store_kvcache(const void* k, const void* v, void* k_cache, void* v_cache,
                                        const int32_t* slot_mapping, int64_t T, int KVH, int D, int64_t num_slots,
                                        int src_dtype, void* stream) {
    using namespace nvllm;
    if (T < 0 || KVH <= 0 || D <= 0 || num_slots < 0)
        return fail(NVLLM_B200_EINVAL, "store_kvcache: negative size (T=%lld KVH=%d D=%d num_slots=%lld)", (long long)T,
                    KVH, D, (long long)num_slots);
    if (T == 0 || num_slots == 0) return NVLLM_B200_OK;
    if (!k || !v || !k_cache || !v_cache || !slot_mapping) return fail(NVLLM_B200_EINVAL, "store_kvcache: null pointer");
    if (((int64_t)KVH * D) % 8 != 0)
        return fail(NVLLM_B200_EUNSUPPORTED, "store_kvcache: KVH*D=%d must be a multiple of 8", KVH * D);
    if (src_dtype != NVLLM_B200_DTYPE_BF16 && src_dtype != NVLLM_B200_DTYPE_F32)
        return fail(NVLLM_B200_EUNSUPPORTED, "store_kvcache: src_dtype %d", src_dtype);
    const uintptr_t align = (uintptr_t)k | (uintptr_t)v | (uintptr_t)k_cache | (uintptr_t)v_cache;
    if (align & 15) return fail(NVLLM_B200_EINVAL, "store_kvcache: pointers must be 16-byte aligned");
    const int row_chunks = KVH * D / 8;
    const int64_t total = T * row_chunks;
    const int64_t blocks = store_blocks_for(total);
    if (blocks > 0x7fffffffLL) return fail(NVLLM_B200_EUNSUPPORTED, "store_kvcache: T too large");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)blocks);
    cfg.blockDim = dim3(kStoreThreads);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    if (src_dtype == NVLLM_B200_DTYPE_BF16) {
        NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, store_kvcache_kernel<__nv_bfloat16>, (const __nv_bfloat16*)k,
                                         (const __nv_bfloat16*)v, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache,
                                         slot_mapping, total, row_chunks, num_slots));
    } else {
        NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, store_kvcache_kernel<float>, (const float*)k, (const float*)v,
                                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slot_mapping, total,
                                         row_chunks, num_slots));
    }
    return NVLLM_B200_OK;
}
