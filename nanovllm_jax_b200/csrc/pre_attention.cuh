// Fused pre-attention step, device code: per-head RMSNorm of q and k, rotary embedding, and the scatter of the
// step's K/V rows into the paged cache, in one pass over q, k, v.
//
// Replaces, for one layer (reference models/qwen3.py:157-166):
//     q = q_norm(q); k = k_norm(k)           layers/layernorm.py:31-48  (fp32 math, result cast back to bf16)
//     q, k = rotary_emb(positions, q, k)     layers/rotary_embedding.py:13-37, 97-104  (x1 cos - x2 sin | x2 cos + x1 sin
//                                            in fp32 with the fp32 cos/sin table, halves split at head_dim / 2)
//     store_kv_to_cache(k, v, ...)           layers/attention.py:42-77 (cast to the cache dtype, scatter by slot)
// q and k are updated in place (prefill reads the packed k); k and v rows also go to their cache slots.
//
// HBM-bound: per token (H + 2 KVH) rows of 256 B are read once, the q and k rows written back, the k and v rows
// written to the cache.  One half-warp per row, 16 bytes per lane; the rotation partner of lane l is lane l ^ 8.
//
// Arithmetic is pinned so that a host restatement reproduces the bf16 results bit for bit: every fp32 operation
// is a separate IEEE round-to-nearest multiply / add / divide / square root (no fused multiply-add, no approximate
// reciprocal square root), and the sum of squares runs in one fixed order: eight elements left to right inside a
// lane, then a butterfly over the sixteen lanes of the row (xor 8, 4, 2, 1).
#pragma once

#include "common.cuh"

namespace nvllm {
namespace preattn {

constexpr int kD = 128;
constexpr int kThreads = 256;
constexpr int kRowsPerBlock = kThreads / 16;

struct Params {
    __nv_bfloat16* q;
    __nv_bfloat16* k;
    const __nv_bfloat16* v;
    const float* q_weight;
    const float* k_weight;
    const float* cos_sin;      // [max_pos, 128]: cos(64) | sin(64)
    const int32_t* positions;  // [T]
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    const int32_t* slot_mapping;
    int64_t T;
    int H, KVH;
    int64_t num_slots, max_pos;
    float eps;
};

__device__ __forceinline__ void unpack8(const uint4& w, float (&f)[8]) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 w;
    w.x = pack_bf16(f[0], f[1]);
    w.y = pack_bf16(f[2], f[3]);
    w.z = pack_bf16(f[4], f[5]);
    w.w = pack_bf16(f[6], f[7]);
    return w;
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

inline int64_t blocks_for(int64_t T, int H, int KVH) {
    const int64_t rows = T * (H + 2 * KVH);
    return (rows + kRowsPerBlock - 1) / kRowsPerBlock;
}

// The share of block `block` (kThreads threads): rows [block * 16, block * 16 + 16) of the T * (H + 2 KVH) rows.
__device__ __forceinline__ void pre_attention_block(int64_t block, const Params& p) {
    const int rows_per_token = p.H + 2 * p.KVH;
    const int64_t row = block * kRowsPerBlock + (threadIdx.x >> 4);  // one half-warp per row
    const int l = threadIdx.x & 15;                                   // 16-byte chunk of the row
    const bool live = row < p.T * rows_per_token;
    const int64_t t = live ? row / rows_per_token : 0;
    const int r = live ? (int)(row - t * rows_per_token) : 0;
    // r in [0, H): q head; [H, H+KVH): k head; [H+KVH, H+2KVH): v head
    const int kind = r < p.H ? 0 : (r < p.H + p.KVH ? 1 : 2);
    const int head = kind == 0 ? r : (kind == 1 ? r - p.H : r - p.H - p.KVH);
    const __nv_bfloat16* src = kind == 0 ? p.q + (t * p.H + head) * kD
                                          : (kind == 1 ? p.k : p.v) + (t * p.KVH + head) * kD;
    uint4 w = make_uint4(0, 0, 0, 0);
    if (live) w = *reinterpret_cast<const uint4*>(src + l * 8);
    const int64_t slot = live && kind != 0 ? (int64_t)__ldg(p.slot_mapping + t) : -1;
    {   // every lane runs the math (full-warp shuffles; the two rows of a warp may be of different kinds);
        // v rows and dead rows simply do not use the result
        const uint4 w_in = w;
        float x[8];
        unpack8(w, x);
        float ss = __fmul_rn(x[0], x[0]);
#pragma unroll
        for (int i = 1; i < 8; ++i) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
        // butterfly over the 16 lanes of the row (xor offsets below 16 stay inside the half-warp); both partners
        // compute the same sum, so every lane ends with the same value
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, 1.0f / kD), p.eps)));
        const float* wgt = (kind == 1 ? p.k_weight : p.q_weight) + l * 8;
        const float4 w0 = __ldg(reinterpret_cast<const float4*>(wgt)), w1 = __ldg(reinterpret_cast<const float4*>(wgt) + 1);
        const float ws[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float y[8], z[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = round_bf16(__fmul_rn(__fmul_rn(x[i], inv), ws[i]));  // the norm returns bf16
        // rotation partner: dims d and d + 64 -> lanes l and l ^ 8
#pragma unroll
        for (int i = 0; i < 8; ++i) z[i] = __shfl_xor_sync(0xffffffffu, y[i], 8);
        int64_t pos = live ? (int64_t)__ldg(p.positions + t) : 0;
        if (pos < 0) pos = 0;
        if (pos >= p.max_pos) pos = p.max_pos - 1;
        const float* cs = p.cos_sin + pos * kD + (l & 7) * 8;
        const float4 c0 = __ldg(reinterpret_cast<const float4*>(cs)), c1 = __ldg(reinterpret_cast<const float4*>(cs) + 1);
        const float4 s0 = __ldg(reinterpret_cast<const float4*>(cs + 64)), s1 = __ldg(reinterpret_cast<const float4*>(cs + 64) + 1);
        const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        const float s[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
        float o[8];
        if (l < 8) {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = __fsub_rn(__fmul_rn(y[i], c[i]), __fmul_rn(z[i], s[i]));  // x1 cos - x2 sin
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = __fadd_rn(__fmul_rn(y[i], c[i]), __fmul_rn(z[i], s[i]));  // x2 cos + x1 sin
        }
        w = kind == 2 ? w_in : pack8(o);
        if (live && kind != 2) {
            __nv_bfloat16* dst = kind == 0 ? p.q + (t * p.H + head) * kD : p.k + (t * p.KVH + head) * kD;
            *reinterpret_cast<uint4*>(dst + l * 8) = w;
        }
    }
    if (live && kind != 0 && slot >= 0 && slot < p.num_slots) {
        __nv_bfloat16* cache = kind == 1 ? p.k_cache : p.v_cache;
        *reinterpret_cast<uint4*>(cache + (slot * p.KVH + head) * kD + l * 8) = w;
    }
}

}  // namespace preattn
}  // namespace nvllm
