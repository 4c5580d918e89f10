// store_kvcache device code shared by the stand-alone scatter kernel (store_kvcache.cu) and by the kernels that
// fold the scatter into a larger step (paged_decode.cu: decode_prepare_kernel).
//
// Layout: a cache row (one token, all KV heads) is KVH*D*2 contiguous bytes; it moves as 16-byte chunks.  Work
// is flattened over (token, chunk) so consecutive threads touch consecutive 16-byte chunks of one row (fully
// coalesced on both sides); every thread issues kStoreUnroll independent K and V loads before its first store
// to keep many requests in flight.
#pragma once

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

// The share of store block `block` (of kStoreThreads threads): chunks [block*kStoreThreads*kStoreUnroll, +that).
// A slot < 0 is skipped, a slot >= num_slots dropped.
template <typename SrcT>
__device__ __forceinline__ void store_block(int64_t block, const SrcT* __restrict__ k, const SrcT* __restrict__ v,
                                            __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                            const int32_t* __restrict__ slot_mapping, int64_t total_chunks,
                                            int row_chunks, int64_t num_slots) {
    const int64_t base = block * (kStoreThreads * kStoreUnroll) + threadIdx.x;
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

inline int64_t store_blocks_for(int64_t total_chunks) {
    const int64_t per_block = (int64_t)kStoreThreads * kStoreUnroll;
    return (total_chunks + per_block - 1) / per_block;
}

}  // namespace nvllm
