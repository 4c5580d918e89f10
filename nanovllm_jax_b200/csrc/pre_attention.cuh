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
// written to the cache.  Four lanes per row, four 16-byte chunks per lane (chunks q, q+4, q+8, q+12 of the row's sixteen:
// a dim and its rotation partner 64 dims further sit in the same lane, and three quarters of the per-row scalar work --
// the divide and the square root -- that sixteen lanes per row repeated is gone).
//
// Arithmetic is pinned so that a host restatement reproduces the bf16 results bit for bit: every fp32 operation
// is a separate IEEE round-to-nearest multiply / add / divide / square root (no fused multiply-add, no approximate
// reciprocal square root), and the sum of squares runs in one fixed order: sixteen partial sums of eight elements
// each, left to right, then a butterfly over the sixteen partial sums (index xor 8, 4, 2, 1).
#pragma once

#include "common.cuh"

namespace nvllm {
namespace preattn {

constexpr int kD = 128;
constexpr int kThreads = 256;
constexpr int kRowsPerBlock = kThreads / 4;  // four lanes per 256-byte row

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

constexpr int kRowsInFlight = 2;  // rows a thread of the stand-alone kernel has loads in flight for

inline int64_t blocks_for(int64_t T, int H, int KVH) {
    const int64_t rows = T * (H + 2 * KVH);
    return (rows + kRowsPerBlock - 1) / kRowsPerBlock;
}

// A quarter of one row as a thread holds it between its loads and its math: lane q (0..3) of the row's four lanes owns
// the 16-byte chunks q, q + 4, q + 8 and q + 12 (chunk c = dims 8c .. 8c+7).
struct Part {
    uint4 w[4];    // the four chunks (zeros for a dead row)
    int64_t t;     // token
    int64_t slot;  // cache slot (k and v rows), -1: none
    int pos;       // position of the token
    int r;         // row of the token: [0, H) q heads, [H, H+KVH) k heads, [H+KVH, H+2KVH) v heads
    bool live;
};

// Issues the loads of lane q's part of row `row` (of the T * (H + 2 KVH) rows); nothing here waits for them.
__device__ __forceinline__ Part load_part(int64_t row, const int q, const Params& p) {
    Part c;
    const int rows_per_token = p.H + 2 * p.KVH;
    c.live = row < p.T * rows_per_token;
    c.t = c.live ? row / rows_per_token : 0;
    c.r = c.live ? (int)(row - c.t * rows_per_token) : 0;
    const int kind = c.r < p.H ? 0 : (c.r < p.H + p.KVH ? 1 : 2);
    const int head = kind == 0 ? c.r : (kind == 1 ? c.r - p.H : c.r - p.H - p.KVH);
    const __nv_bfloat16* src = kind == 0 ? p.q + (c.t * p.H + head) * kD
                                          : (kind == 1 ? p.k : p.v) + (c.t * p.KVH + head) * kD;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        c.w[i] = make_uint4(0, 0, 0, 0);
        if (c.live) c.w[i] = *reinterpret_cast<const uint4*>(src + (q + 4 * i) * 8);
    }
    c.slot = c.live && kind != 0 ? (int64_t)__ldg(p.slot_mapping + c.t) : -1;
    c.pos = c.live ? __ldg(p.positions + c.t) : 0;
    return c;
}

__device__ __forceinline__ void load8(const float* src, float (&f)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(src)), b = __ldg(reinterpret_cast<const float4*>(src) + 1);
    f[0] = a.x, f[1] = a.y, f[2] = a.z, f[3] = a.w, f[4] = b.x, f[5] = b.y, f[6] = b.z, f[7] = b.w;
}

// Norm, rotation and stores of one part.  Every lane of the warp must call this together (full-warp shuffles; the
// eight rows of a warp may be of different kinds): v rows and dead rows simply do not use the result of the math.
//
// The sum of squares keeps one fixed order whatever the lane layout: sixteen partial sums, one per chunk, each taken
// front to back, then the butterfly p[c] + p[c ^ 8], + [c ^ 4], + [c ^ 2], + [c ^ 1].  With chunks q, q+4, q+8, q+12
// in one lane the first two levels are local and the last two are shuffles over the row's four lanes.
__device__ __forceinline__ void finish_part(const Part& ch, const int q, const Params& p) {
    const int kind = ch.r < p.H ? 0 : (ch.r < p.H + p.KVH ? 1 : 2);
    const int head = kind == 0 ? ch.r : (kind == 1 ? ch.r - p.H : ch.r - p.H - p.KVH);
    uint4 out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) out[i] = ch.w[i];
    // a warp whose eight rows are all v rows (or past the end) has nothing to compute: the rows are copied
    if (!__all_sync(0xffffffffu, kind == 2 || !ch.live)) {
        float x[4][8], pp[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            unpack8(ch.w[i], x[i]);
            float ss = __fmul_rn(x[i][0], x[i][0]);
#pragma unroll
            for (int e = 1; e < 8; ++e) ss = __fadd_rn(ss, __fmul_rn(x[i][e], x[i][e]));
            pp[i] = ss;
        }
        float ss = __fadd_rn(__fadd_rn(pp[0], pp[2]), __fadd_rn(pp[1], pp[3]));  // levels c ^ 8 and c ^ 4
        ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, 2));                  // level c ^ 2
        ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, 1));                  // level c ^ 1
        const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fmul_rn(ss, 1.0f / kD), p.eps)));
        const float* wgt = kind == 1 ? p.k_weight : p.q_weight;
        float y[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float ws[8];
            load8(wgt + (q + 4 * i) * 8, ws);
#pragma unroll
            for (int e = 0; e < 8; ++e) y[i][e] = round_bf16(__fmul_rn(__fmul_rn(x[i][e], inv), ws[e]));  // the norm returns bf16
        }
        int64_t pos = ch.pos;
        if (pos < 0) pos = 0;
        if (pos >= p.max_pos) pos = p.max_pos - 1;
#pragma unroll
        for (int i = 0; i < 2; ++i) {  // chunk q + 4i holds dims d < 64, its rotation partner d + 64 is chunk q + 4i + 8
            float c[8], sn[8], lo[8], hi[8];
            const float* cs = p.cos_sin + pos * kD + (q + 4 * i) * 8;
            load8(cs, c);
            load8(cs + 64, sn);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                lo[e] = __fsub_rn(__fmul_rn(y[i][e], c[e]), __fmul_rn(y[i + 2][e], sn[e]));  // x1 cos - x2 sin
                hi[e] = __fadd_rn(__fmul_rn(y[i + 2][e], c[e]), __fmul_rn(y[i][e], sn[e]));  // x2 cos + x1 sin
            }
            out[i] = pack8(lo);
            out[i + 2] = pack8(hi);
        }
        if (kind == 2) {
#pragma unroll
            for (int i = 0; i < 4; ++i) out[i] = ch.w[i];
        }
    }
    if (ch.live && kind != 2) {
        __nv_bfloat16* dst = kind == 0 ? p.q + (ch.t * p.H + head) * kD : p.k + (ch.t * p.KVH + head) * kD;
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(dst + (q + 4 * i) * 8) = out[i];
    }
    if (ch.live && kind != 0 && ch.slot >= 0 && ch.slot < p.num_slots) {
        __nv_bfloat16* cache = (kind == 1 ? p.k_cache : p.v_cache) + (ch.slot * p.KVH + head) * kD;
#pragma unroll
        for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(cache + (q + 4 * i) * 8) = out[i];
    }
}

// The share of block `block` (kThreads threads): rows [block * 64, block * 64 + 64) of the T * (H + 2 KVH) rows, four
// lanes per row, 64 bytes per lane.
__device__ __forceinline__ void pre_attention_block(int64_t block, const Params& p) {
    const int q = threadIdx.x & 3;
    const Part c = load_part(block * kRowsPerBlock + (threadIdx.x >> 2), q, p);
    finish_part(c, q, p);
}

}  // namespace preattn
}  // namespace nvllm
