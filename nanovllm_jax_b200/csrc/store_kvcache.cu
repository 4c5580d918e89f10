// store_kvcache: scatter the step's new K/V rows into the paged cache by slot.
//
// Replaces store_kv_to_cache (reference layers/attention.py:42-77).  Pure data
// movement, HBM-bound: per token it reads KVH*D elements of K and of V and
// writes the same number of bf16 elements to each cache, plus one int32 slot.
//
// Layout: a cache row (one token, all KV heads) is KVH*D*2 contiguous bytes;
// the kernel moves it as 16-byte chunks.  Work is flattened over
// (token, chunk) so consecutive threads touch consecutive 16-byte chunks of
// one row (fully coalesced on both sides); every thread issues UNROLL
// independent K and V loads before its first store to keep many requests in
// flight.
#include "common.cuh"

namespace nvllm {

constexpr int kStoreThreads = 256;
constexpr int kStoreUnroll = 4;

__device__ __forceinline__ uint4 load_chunk_as_bf16(const __nv_bfloat16* src, int64_t chunk) {
    return __ldg(reinterpret_cast<const uint4*>(src) + chunk);
}

__device__ __forceinline__ uint4 load_chunk_as_bf16(const float* src, int64_t chunk) {
    const float4* p = reinterpret_cast<const float4*>(src) + 2 * chunk;
    float4 a = __ldg(p), b = __ldg(p + 1);
    uint4 r;
    r.x = pack_bf16(a.x, a.y);
    r.y = pack_bf16(a.z, a.w);
    r.z = pack_bf16(b.x, b.y);
    r.w = pack_bf16(b.z, b.w);
    return r;
}

template <typename SrcT>
__global__ void __launch_bounds__(kStoreThreads)
store_kvcache_kernel(const SrcT* __restrict__ k, const SrcT* __restrict__ v, __nv_bfloat16* __restrict__ k_cache,
                     __nv_bfloat16* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping, int64_t total_chunks,
                     int row_chunks, int64_t num_slots) {
    griddep_wait();  // k, v and slot_mapping may come from the kernel just before this one
    griddep_launch_dependents();
    const int64_t base = (int64_t)blockIdx.x * (kStoreThreads * kStoreUnroll) + threadIdx.x;
    uint4 kv[kStoreUnroll], vv[kStoreUnroll];
    int64_t dst[kStoreUnroll];
#pragma unroll
    for (int u = 0; u < kStoreUnroll; ++u) {
        const int64_t i = base + (int64_t)u * kStoreThreads;
        dst[u] = -1;
        if (i < total_chunks) {
            const int64_t t = i / row_chunks;
            const int c = (int)(i - t * row_chunks);
            const int64_t slot = __ldg(slot_mapping + t);
            if (slot >= 0 && slot < num_slots) {
                dst[u] = slot * row_chunks + c;
                kv[u] = load_chunk_as_bf16(k, i);
                vv[u] = load_chunk_as_bf16(v, i);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kStoreUnroll; ++u) {
        if (dst[u] >= 0) {
            reinterpret_cast<uint4*>(k_cache)[dst[u]] = kv[u];
            reinterpret_cast<uint4*>(v_cache)[dst[u]] = vv[u];
        }
    }
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
    const int64_t per_block = (int64_t)kStoreThreads * kStoreUnroll;
    const int64_t blocks = (total + per_block - 1) / per_block;
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
