// paged_decode: flash-decoding over the block-table KV cache for sm_100a.
//
// Replaces paged_attention / paged_decode_attention_vectorized of the
// reference (layers/pallas_attention.py:465-507, :146-238).
//
// The op is HBM-bound: every live K and V row is read exactly once.  Design:
//
//  * Work unit = one 64-token tile of one (sequence, kv head).  All tiles of
//    one kv head are laid end to end (sequence after sequence) and cut into
//    `num_groups` contiguous ranges of equal COST ("stream-K" partition): a tile
//    costs one unit and every sequence four more in front of its tiles (the
//    time a CTA loses at a sequence boundary -- q load, page lookup, the
//    cross-warp combine, and the partial results at the ends of a range).  So every CTA
//    finishes at the same time no matter how skewed the context lengths are or
//    how many short sequences fall into its range.  CTA c serves kv head c % KVH of group c / KVH; the KVH CTAs of a
//    group walk the same tokens at the same pace, so the 256-byte per-head rows
//    they fetch are neighbours in DRAM.
//  * Persistent CTAs, 2 per SM: one producer warp issues TMA tile loads
//    (cp.async.bulk.tensor, 128-byte swizzle, no multicast) into a 3-stage
//    mbarrier ring and runs ahead across sequence boundaries; four consumer
//    warps each own 16 tokens of a tile.
//  * The G = H/KVH query heads that share a kv head are packed into the 16-row
//    M dimension of mma.sync.m16n8k16 (bf16 in, fp32 accumulate) for both
//    q.K^T and P.V; the online softmax (exp2 domain) lives in registers with
//    warp-shuffle row reductions.
//  * A range that ends inside a sequence leaves an fp32 partial (m, l, O) in
//    the caller's workspace and takes a ticket for that (sequence, kv head); the
//    CTA that draws the last ticket combines all partials of the sequence, in
//    group order (bitwise reproducible whichever CTA arrives last), and writes
//    the rows -- all G rows at once, every load of a batch of four partials in
//    flight together, so the combine costs about one round trip to L2 per four
//    partials.  Nobody waits for another CTA.  Sequences wholly inside one range are
//    written directly.  The tickets are cleared by the small kernel that runs
//    before this one (decode_prepare_kernel, which in the fused decode step
//    also scatters the step's new K/V rows into the cache).
//
// No spin-wait is unbounded: every mbarrier wait gives up after a poll limit,
// raises a device error flag (readable through nvllm_b200_device_status) and
// the CTA drains and returns.
#include "pre_attention.cuh"
#include "store_kvcache.cuh"

#include <mutex>
#include <stdlib.h>
#include <string.h>

namespace nvllm {
namespace decode {

constexpr int kTile = 64;                      // tokens per tile
constexpr int kD = 128;                        // head_dim
constexpr int kConsumerWarps = 4;
constexpr int kWarps = kConsumerWarps + 1;     // consumers, TMA producer
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;
constexpr int kMaxG = 8;                       // query heads per kv head packed in one CTA
constexpr int kItemCostDefault = 4;            // cost of a sequence boundary in tile units (stream-K weights)
constexpr int kPanelBytes = kTile * 128;       // 64 tokens x 64 dims bf16, 128B-swizzled
constexpr int kTileBytes = 2 * kPanelBytes;    // one K or V tile
constexpr int kQBytes = kMaxG * kD * 2;        // 2 KiB
constexpr int kStageBytes = 2 * kTileBytes + kQBytes;  // 34816
constexpr int kOsStride = kD + 8;              // padded row of the cross-warp merge buffers (bank spread)
constexpr int kOsBytes = 2 * kMaxG * kOsStride * 4;  // two buffers [8][136] fp32
constexpr int kMiscBytes = 1024;
constexpr int kSmemBytes = kStages * kStageBytes + kOsBytes + kMiscBytes + 1024;  // + alignment slack
constexpr int kCtasPerSm = 2;

// Per-partial record in the workspace: O[G][128] fp32, then m[8], l[8].
__host__ __device__ inline size_t partial_floats(int G) { return (size_t)G * kD + 2 * kMaxG; }

__device__ int g_error_flag = 0;

struct Params {
    const __nv_bfloat16* q;
    const int32_t* block_tables;
    const int32_t* context_lens;
    __nv_bfloat16* out;
    float* partials;        // [grid][2][partial_floats]
    unsigned int* tickets;  // [B*KVH] partials delivered so far per (sequence, kv head); zero when the kernel starts
    int B, H, KVH, G, NB, block_size, MB;
    int num_groups;
    int item_cost;  // units a sequence boundary costs on the cost line (see units_of)
    float scale_log2;
};

__device__ __forceinline__ int clamp_ctx(int c, int max_ctx) { return c < 0 ? 0 : (c > max_ctx ? max_ctx : c); }
__device__ __forceinline__ int tiles_of(int ctx) { return (ctx + kTile - 1) / kTile; }

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col); rows 8..15 of A are zero here.
__device__ __forceinline__ void mma_lo(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    const uint32_t z = 0u;
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}

// The cost line: sequence b with tb > 0 tiles occupies tb + item_cost units, the first item_cost of them standing
// for its boundary overhead, the rest for its tiles 0 .. tb-1; empty sequences occupy nothing.
__device__ __forceinline__ int units_of(int tb, int item_cost) { return tb > 0 ? tb + item_cost : 0; }

struct Walk {
    int b;             // next sequence to look at
    long long fv;      // unit at which sequence b starts
    long long x0, x1;  // this CTA's range of units
};
struct Item {
    int b, t0, n;      // sequence, first tile and number of tiles this CTA serves of it
    int ctx, tb;       // its context length and total tiles
    long long fv;      // unit at which the sequence starts (its tile 0 sits at fv + item_cost)
};

// Advance to the next sequence of which this CTA serves at least one tile; false when the range is exhausted.
// (hint_b, hint_ctx): a context length the caller has fetched ahead of time (hint_b < 0: none).
__device__ __forceinline__ bool next_item(Walk& w, const Params& p, int max_ctx, Item& it, int hint_b = -1,
                                          int hint_ctx = 0) {
    while (w.b < p.B && w.fv < w.x1) {
        const int ctx = clamp_ctx(w.b == hint_b ? hint_ctx : __ldg(p.context_lens + w.b), max_ctx);
        const int tb = tiles_of(ctx);
        const long long t_base = w.fv + p.item_cost;  // unit of tile 0
        it.b = w.b;
        it.fv = w.fv;
        ++w.b;
        w.fv += units_of(tb, p.item_cost);
        if (tb == 0) continue;
        const long long lo = w.x0 - t_base, hi = w.x1 - t_base;
        const int t0 = (int)(lo < 0 ? 0 : (lo > tb ? tb : lo));
        const int t1 = (int)(hi < 0 ? 0 : (hi > tb ? tb : hi));
        if (t0 >= t1) continue;  // only boundary units of this sequence fall into the range
        it.t0 = t0;
        it.n = t1 - t0;
        it.ctx = ctx;
        it.tb = tb;
        return true;
    }
    return false;
}

// Combine the partials of sequence b (its tiles occupy units [first, first + tb) of the cost line) for kv head kvh and
// write its G output rows.  Called by the 128 consumer threads: thread t owns row t / 16 and dims 8 (t % 16) ..
// 8 (t % 16) + 7.  Partials are taken in group order, four at a time (all loads of a batch are independent), so the
// result does not depend on which CTA runs this.
__device__ __forceinline__ void merge_sequence(const Params& p, int b, int kvh, long long first, int tb,
                                               long long total, int ctid) {
    const int r = ctid >> 4, c8 = (ctid & 15) * 8;
    if (r >= p.G) return;
    const int ng = p.num_groups;
    long long gf = ((first + 1) * ng - 1) / total;
    long long gl = ((first + tb) * ng - 1) / total;
    if (gf > ng - 1) gf = ng - 1;
    if (gl > ng - 1) gl = ng - 1;
    const size_t pf = partial_floats(p.G);
    float mt = -INFINITY, lt = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (long long g0 = gf; g0 <= gl; g0 += 4) {
        float mv[4], lv[4];
        float4 oa[4], ob[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long g = g0 + u;
            const bool live = g <= gl && (g * total / ng < (g + 1) * total / ng);  // empty groups wrote nothing
            const float* part = p.partials + ((size_t)(g * p.KVH + kvh) * 2 + (g == gf ? 1 : 0)) * pf;
            mv[u] = live ? __ldcg(part + p.G * kD + r) : -INFINITY;
            lv[u] = live ? __ldcg(part + p.G * kD + kMaxG + r) : 0.f;
            oa[u] = live ? __ldcg(reinterpret_cast<const float4*>(part + r * kD + c8)) : make_float4(0.f, 0.f, 0.f, 0.f);
            ob[u] = live ? __ldcg(reinterpret_cast<const float4*>(part + r * kD + c8) + 1) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        const float mnew = fmaxf(fmaxf(mt, fmaxf(mv[0], mv[1])), fmaxf(mv[2], mv[3]));
        if (mnew == -INFINITY) continue;
        const float sc = (mt == -INFINITY) ? 0.f : fast_exp2(mt - mnew);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= sc;
        lt *= sc;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float f = (mv[u] == -INFINITY) ? 0.f : fast_exp2(mv[u] - mnew);
            acc[0] += oa[u].x * f;
            acc[1] += oa[u].y * f;
            acc[2] += oa[u].z * f;
            acc[3] += oa[u].w * f;
            acc[4] += ob[u].x * f;
            acc[5] += ob[u].y * f;
            acc[6] += ob[u].z * f;
            acc[7] += ob[u].w * f;
            lt += lv[u] * f;
        }
        mt = mnew;
    }
    const float inv = 1.0f / (lt + 1e-9f);
    uint4 w;
    w.x = pack_bf16(acc[0] * inv, acc[1] * inv);
    w.y = pack_bf16(acc[2] * inv, acc[3] * inv);
    w.z = pack_bf16(acc[4] * inv, acc[5] * inv);
    w.w = pack_bf16(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(p.out + ((size_t)b * p.H + (size_t)kvh * p.G + r) * kD + c8) = w;
}

__global__ void __launch_bounds__(kThreads, kCtasPerSm)
paged_decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* Os = reinterpret_cast<float*>(smem + kStages * kStageBytes);
    uint8_t* misc = smem + kStages * kStageBytes + kOsBytes;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(misc);            // [kStages]
    uint64_t* empty_bar = full_bar + kStages;                          // [kStages]
    int* sm_i = reinterpret_cast<int*>(misc + 64);                     // scan scratch [8] + start [2] + abort [1]
    volatile int* sm_abort = sm_i + 12;
    long long* sm_fv = reinterpret_cast<long long*>(sm_i + 14);       // unit at which the CTA's first sequence starts
    float* sm_ml = reinterpret_cast<float*>(misc + 128);               // [2 parities][m|l][4 warps][8 rows]

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x % p.KVH;
    const int group = blockIdx.x / p.KVH;
    const int max_ctx = p.MB * p.block_size;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, kConsumerWarps);
        }
        fence_mbar_init();
        sm_i[10] = -1;
        sm_i[11] = 0;
        *sm_abort = 0;
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }

    griddep_launch_dependents();  // lets the next kernel of the stream run its own prologue while this grid streams

    // Programmatic dependent launch: this grid starts while the kernel launched just before it on the stream
    // (decode_prepare_kernel: ticket clear, and in the fused step the scatter / rotation of the step's rows) is
    // still running.  That kernel writes tickets, cache rows and (fused step) q -- never context_lens or
    // block_tables -- and everything launched before IT has completed by the time this grid starts (its own
    // blocks passed their griddepcontrol.wait before they let this grid go).  So the scan below and the first
    // page lookup read only settled memory and run ahead of the wait; the wait sits right before the first
    // access to anything the preparing kernel writes.

    // ---- prologue: total cost units per head and the sequence this CTA's range starts in ----
    // Every CTA scans context_lens itself (B / 160 values per thread and one warp scan): that is one global
    // load latency, paid in parallel by all CTAs, and cheaper than fetching the result of a serial plan.
    const int per = (p.B + kThreads - 1) / kThreads;
    const int b_lo = min(p.B, tid * per), b_hi = min(p.B, b_lo + per);
    int mine = 0;
    for (int b = b_lo; b < b_hi; ++b) {
        const int tb = tiles_of(clamp_ctx(__ldg(p.context_lens + b), max_ctx));
        mine += units_of(tb, p.item_cost);
        if (tb == 0 && b % p.num_groups == group) {
            // an empty sequence attends to nothing: its rows are zeros (one CTA per kv head writes them)
            uint4* orow = reinterpret_cast<uint4*>(p.out + ((size_t)b * p.H + (size_t)kvh * p.G) * kD);
            for (int i = 0; i < p.G * (kD * 2 / 16); ++i) orow[i] = make_uint4(0, 0, 0, 0);
        }
    }
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) sm_i[warp] = incl;
    __syncthreads();
    long long total = 0;
    int warp_off = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
        const int v = sm_i[w];
        if (w < warp) warp_off += v;
        total += v;
    }
    const long long x0 = (long long)group * total / p.num_groups;
    const long long x1 = (long long)(group + 1) * total / p.num_groups;
    {
        long long run = warp_off + incl - mine;
        for (int b = b_lo; b < b_hi; ++b) {
            const int ub = units_of(tiles_of(clamp_ctx(__ldg(p.context_lens + b), max_ctx)), p.item_cost);
            if (ub > 0 && run <= x0 && x0 < run + ub) {
                sm_i[10] = b;
                *sm_fv = run;
            }
            run += ub;
        }
    }
    __syncthreads();
    if (x0 >= x1 || sm_i[10] < 0) return;  // nothing to do (uniform across the CTA)

    Walk walk;
    walk.b = sm_i[10];
    walk.fv = *sm_fv;
    walk.x0 = x0;
    walk.x1 = x1;
    // page of the first tile, fetched ahead of the wait (block_tables is settled memory, see above)
    int first_phys = 0;
    if (warp == kConsumerWarps && lane == 0) {
        Walk peek = walk;
        Item first;
        if (next_item(peek, p, max_ctx, first))
            first_phys = __ldg(p.block_tables + (size_t)first.b * p.MB + (first.t0 * kTile) / p.block_size);
    }
    griddep_wait();

    if (warp == kConsumerWarps) {
        // =========================== producer warp ===========================
        if (lane == 0) {
            const uint64_t pol = policy_evict_first();
            uint32_t it = 0;
            Item item;
            bool ok = true;
            // Metadata of the sequence after the current one is fetched one item ahead (its length and its first
            // page: every item but a CTA's first starts at tile 0), so that a sequence boundary does not put two
            // dependent global-load latencies between two tile requests.
            int pf_b = -1, pf_ctx = 0, pf_phys = 0;
            while (ok && next_item(walk, p, max_ctx, item, pf_b, pf_ctx)) {
                const int32_t* bt = p.block_tables + (size_t)item.b * p.MB;
                for (int i = 0; i < item.n; ++i, ++it) {
                    const int stage = it % kStages;
                    const uint32_t parity = ((it / kStages) & 1u) ^ 1u;
                    if (*sm_abort || !mbar_wait(empty_bar + stage, parity)) {
                        ok = false;
                        break;
                    }
                    const int tok0 = (item.t0 + i) * kTile;
                    const int bi = tok0 / p.block_size;
                    int phys = it == 0 ? first_phys : ((i == 0 && item.b == pf_b && bi == 0) ? pf_phys : __ldg(bt + bi));
                    phys = phys < 0 ? 0 : (phys >= p.NB ? p.NB - 1 : phys);
                    const int slot = phys * p.block_size + (tok0 - bi * p.block_size);
                    uint8_t* st = smem + stage * kStageBytes;
                    uint64_t* bar = full_bar + stage;
                    const uint32_t qbytes = (i == 0) ? (uint32_t)p.G * kD * 2 : 0u;
                    mbar_expect_tx(bar, 2 * kTileBytes + qbytes);
                    tma_load_3d_hint(st, &tm_k, bar, 0, kvh, slot, pol);
                    tma_load_3d_hint(st + kPanelBytes, &tm_k, bar, 64, kvh, slot, pol);
                    tma_load_3d_hint(st + kTileBytes, &tm_v, bar, 0, kvh, slot, pol);
                    tma_load_3d_hint(st + kTileBytes + kPanelBytes, &tm_v, bar, 64, kvh, slot, pol);
                    if (i == 0) {
                        bulk_load(st + 2 * kTileBytes, p.q + ((size_t)item.b * p.H + (size_t)kvh * p.G) * kD, qbytes,
                                  bar);
                        if (walk.b < p.B) {  // the loads are issued now and first used at the next boundary
                            pf_b = walk.b;
                            pf_ctx = __ldg(p.context_lens + walk.b);
                            pf_phys = __ldg(p.block_tables + (size_t)walk.b * p.MB);
                        }
                    }
                }
            }
            if (!ok) {
                *sm_abort = 1;
                atomicOr(&g_error_flag, 1);
                // Let loads already issued land before the CTA's shared memory is released.
                for (uint32_t j = (it >= kStages ? it - kStages : 0); j < it; ++j)
                    (void)mbar_wait(full_bar + (j % kStages), (j / kStages) & 1u, 1u << 16);
            }
        }
        return;
    }

    // ============================= consumer warps =============================
    const int row = lane >> 2;       // query head within the group (valid if < G)
    const int quad = lane & 3;
    const int mi = lane >> 3;        // which 8x8 matrix this lane addresses in ldmatrix.x4
    const int r8 = lane & 7;
    const int tok_base = warp * 16;
    const int ctid = tid;            // 0..127 among consumers
    uint32_t it = 0, item = 0;
    Item cur;
    bool ok = true;

    for (; ok && next_item(walk, p, max_ctx, cur); ++item) {
        const int n = cur.n, ctx = cur.ctx, tb = cur.tb;
        const bool full_item = (cur.t0 == 0 && n == tb);
        // (m, l) exchange buffers alternate between consecutive items so that a warp that races ahead
        // into the next item cannot overwrite values a slower warp is still reading.
        float* sm_m = sm_ml + (item & 1u) * (2 * kConsumerWarps * kMaxG);
        float* sm_l = sm_m + kConsumerWarps * kMaxG;
        uint32_t qa[8][2];
        float o[16][4];
        float m = -INFINITY, l = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

        for (int i = 0; i < n; ++i, ++it) {
            const int stage = it % kStages;
            if (*sm_abort || !mbar_wait(full_bar + stage, (it / kStages) & 1u)) {
                ok = false;
                break;
            }
            uint8_t* st = smem + stage * kStageBytes;
            if (i == 0) {
                const uint32_t* qs = reinterpret_cast<const uint32_t*>(st + 2 * kTileBytes);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    qa[ks][0] = row < p.G ? qs[row * 64 + ks * 8 + quad] : 0u;
                    qa[ks][1] = row < p.G ? qs[row * 64 + ks * 8 + 4 + quad] : 0u;
                }
            }
            const int valid = ctx - ((cur.t0 + i) * kTile + tok_base);  // live tokens in this warp's 16-token slice
            if (valid > 0) {
                const uint32_t kbase = smem_u32(st);
                const uint32_t vbase = kbase + kTileBytes;
                if (valid < 16) {
                    // Rows past the context end may hold anything (even NaN bit patterns): zero the V rows so
                    // that 0 * garbage cannot reach the accumulators.  Each row is 2 panels x 8 chunks of 16 B.
                    for (int idx = lane; idx < (16 - valid) * 16; idx += 32) {
                        const int r = tok_base + valid + (idx >> 4);
                        const int c = idx & 15;
                        uint8_t* dst = st + kTileBytes + (c >> 3) * kPanelBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4);
                        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();  // order these generic writes before the stage's next TMA refill
                    __syncwarp();
                }
                // ---- S = Q K^T for 16 tokens: two n-tiles of 8 tokens ----
                float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
                {
                    const int tok = tok_base + (mi >> 1) * 8 + r8;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks) {
                        const int chunk = ks * 2 + (mi & 1);
                        const uint32_t addr =
                            kbase + (chunk >> 3) * kPanelBytes + tok * 128 + (((chunk & 7) ^ r8) << 4);
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4(addr, b0, b1, b2, b3);
                        mma_lo(s0, qa[ks][0], qa[ks][1], b0, b1);
                        mma_lo(s1, qa[ks][0], qa[ks][1], b2, b3);
                    }
                }
                // ---- online softmax (log2 domain) ----
                const int c0 = 2 * quad;
                float v00 = (c0 < valid) ? s0[0] * p.scale_log2 : -INFINITY;
                float v01 = (c0 + 1 < valid) ? s0[1] * p.scale_log2 : -INFINITY;
                float v10 = (c0 + 8 < valid) ? s1[0] * p.scale_log2 : -INFINITY;
                float v11 = (c0 + 9 < valid) ? s1[1] * p.scale_log2 : -INFINITY;
                float rmax = fmaxf(fmaxf(v00, v01), fmaxf(v10, v11));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 1));
                rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, 2));
                const float m_new = fmaxf(m, rmax);
                const float alpha = fast_exp2(m - m_new);
                v00 = fast_exp2(v00 - m_new);
                v01 = fast_exp2(v01 - m_new);
                v10 = fast_exp2(v10 - m_new);
                v11 = fast_exp2(v11 - m_new);
                l = l * alpha + ((v00 + v01) + (v10 + v11));
                m = m_new;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    o[j][0] *= alpha;
                    o[j][1] *= alpha;
                }
                const uint32_t pa0 = pack_bf16(v00, v01), pa2 = pack_bf16(v10, v11);
                // ---- O += P V: 16 n-tiles of 8 dims, two per ldmatrix.x4.trans ----
                {
                    const int tok = tok_base + (mi & 1) * 8 + r8;
#pragma unroll
                    for (int np = 0; np < 8; ++np) {
                        const int chunk = np * 2 + (mi >> 1);
                        const uint32_t addr =
                            vbase + (chunk >> 3) * kPanelBytes + tok * 128 + (((chunk & 7) ^ r8) << 4);
                        uint32_t b0, b1, b2, b3;
                        ldsm_x4_t(addr, b0, b1, b2, b3);
                        mma_lo(o[2 * np], pa0, pa2, b0, b1);
                        mma_lo(o[2 * np + 1], pa0, pa2, b2, b3);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty_bar + stage);
        }
        if (!ok) break;

        // ---- merge the four warps' (m, l, O) and emit the item ----
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (quad == 0) {
            sm_m[warp * kMaxG + row] = m;
            sm_l[warp * kMaxG + row] = l;
        }
        named_barrier_sync(1, kConsumerWarps * 32);
        {
            // Fixed-order reduction (bitwise reproducible): warps 0,1 store, warps 2,3 add, readers sum the two.
            float mt = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) mt = fmaxf(mt, sm_m[w * kMaxG + row]);
            const float f = (m == -INFINITY) ? 0.f : fast_exp2(m - mt);
            float* dst = Os + (warp & 1) * (kMaxG * kOsStride) + row * kOsStride + 2 * quad;
            if (warp < 2) {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    *reinterpret_cast<float2*>(dst + j * 8) = make_float2(o[j][0] * f, o[j][1] * f);
            }
            named_barrier_sync(1, kConsumerWarps * 32);
            if (warp >= 2) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float2 cur = *reinterpret_cast<float2*>(dst + j * 8);
                    cur.x += o[j][0] * f;
                    cur.y += o[j][1] * f;
                    *reinterpret_cast<float2*>(dst + j * 8) = cur;
                }
            }
        }
        named_barrier_sync(1, kConsumerWarps * 32);
        {
            float* part = nullptr;
            if (!full_item)
                part = p.partials + ((size_t)blockIdx.x * 2 + (cur.t0 == 0 ? 1 : 0)) * partial_floats(p.G);
            for (int r = 0; r < p.G; ++r) {
                float mt = -INFINITY;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) mt = fmaxf(mt, sm_m[w * kMaxG + r]);
                float lt = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w) {
                    const float mw = sm_m[w * kMaxG + r];
                    if (mw != -INFINITY) lt += sm_l[w * kMaxG + r] * fast_exp2(mw - mt);
                }
                const float acc = Os[r * kOsStride + ctid] + Os[(kMaxG + r) * kOsStride + ctid];
                if (full_item) {
                    p.out[((size_t)cur.b * p.H + (size_t)kvh * p.G + r) * kD + ctid] =
                        __float2bfloat16_rn(acc / (lt + 1e-9f));
                } else {
                    part[r * kD + ctid] = acc;
                    if (ctid == 0) {
                        part[p.G * kD + r] = mt;
                        part[p.G * kD + kMaxG + r] = lt;
                    }
                }
            }
            if (!full_item) {
                // Publish the partial, then take a ticket for this (sequence, kv head).  Whoever draws the last
                // ticket finds every partial of the sequence visible and combines them; nobody waits.
                __threadfence();
                named_barrier_sync(1, kConsumerWarps * 32);
                if (ctid == 0) sm_i[9] = (int)atomicAdd(p.tickets + (size_t)cur.b * p.KVH + kvh, 1u);
                named_barrier_sync(1, kConsumerWarps * 32);
                const long long first = cur.fv + p.item_cost;  // unit of the sequence's tile 0 on the cost line
                long long parts = tb;  // fewer units than groups: every non-empty group holds exactly one unit
                if (total >= p.num_groups)
                    parts = ((first + tb) * p.num_groups - 1) / total - ((first + 1) * p.num_groups - 1) / total + 1;
                if ((long long)sm_i[9] == parts - 1) {
                    __threadfence();
                    merge_sequence(p, cur.b, kvh, first, tb, total, ctid);
                }
            }
        }
    }
    if (!ok) {
        *sm_abort = 1;
        atomicOr(&g_error_flag, 2);
    }
}

// Clears the tickets of one decode call and, in the fused decode step, scatters the step's new K/V rows into
// the cache (blocks [0, store_blocks) do the scatter, the rest clear).  Runs right before paged_decode_kernel
// on the same stream.
template <typename SrcT>
__global__ void __launch_bounds__(kStoreThreads)
decode_prepare_kernel(unsigned int* __restrict__ tickets, int num_tickets, int store_blocks,
                      const SrcT* __restrict__ k, const SrcT* __restrict__ v, __nv_bfloat16* __restrict__ k_cache,
                      __nv_bfloat16* __restrict__ v_cache, const int32_t* __restrict__ slot_mapping,
                      int64_t total_chunks, int row_chunks, int64_t num_slots) {
    griddep_wait();  // the previous kernel may still be reading these tickets or the cache rows written below
    griddep_launch_dependents();
    if ((int)blockIdx.x < store_blocks) {
        store_block<SrcT>(blockIdx.x, k, v, k_cache, v_cache, slot_mapping, total_chunks, row_chunks, num_slots);
    } else {
        const int i = ((int)blockIdx.x - store_blocks) * kStoreThreads + threadIdx.x;
        if (i < num_tickets) tickets[i] = 0u;
    }
}

// The same with the whole pre-attention step in front: blocks [0, pre_blocks) normalise and rotate the step's q and
// k rows and scatter the k and v rows (pre_attention.cuh), the rest clear the tickets.
__global__ void __launch_bounds__(preattn::kThreads)
decode_prepare_fused_kernel(unsigned int* __restrict__ tickets, int num_tickets, int pre_blocks, const preattn::Params pp) {
    griddep_wait();
    griddep_launch_dependents();
    if ((int)blockIdx.x < pre_blocks) {
        preattn::pre_attention_block(blockIdx.x, pp);
    } else {
        const int i = ((int)blockIdx.x - pre_blocks) * preattn::kThreads + threadIdx.x;
        if (i < num_tickets) tickets[i] = 0u;
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
static int main_grid() { return kCtasPerSm * sm_count(); }

// NVLLM_B200_ITEM_COST overrides the boundary weight of the stream-K partition (an experiment knob; 0 = by tiles only).
static int item_cost() {
    static const int v = [] {
        const char* e = getenv("NVLLM_B200_ITEM_COST");
        const int x = e ? atoi(e) : kItemCostDefault;
        return x < 0 ? 0 : (x > 64 ? 64 : x);
    }();
    return v;
}

static size_t round256(size_t x) { return (x + 255) & ~size_t(255); }

static size_t ticket_bytes(int B, int KVH) { return round256((size_t)B * KVH * 4); }
static size_t partial_bytes(int ctas, int G) { return round256((size_t)ctas * 2 * partial_floats(G) * 4); }

// Tensor maps of the caches seen so far, keyed by what they encode (base address, slots, kv heads).  Encoding
// one costs the host a microsecond or two per call; a serving loop hands over the same few caches for ever.
// A map holds no reference to the memory: an entry stays valid for any later buffer with the same key.
static int cached_cache_map(CUtensorMap* map, const void* base, int64_t num_slots, int KVH) {
    struct Entry {
        const void* base;
        int64_t num_slots;
        int kvh, dev;
        CUtensorMap map;
    };
    constexpr int kEntries = 256;  // two per layer of a 128-layer model
    static std::mutex mu;
    static Entry table[kEntries];
    static int used = 0, next = 0;
    int dev = 0;
    NVLLM_CUDA_OK(cudaGetDevice(&dev));
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < used; ++i) {
            const Entry& e = table[i];
            if (e.base == base && e.num_slots == num_slots && e.kvh == KVH && e.dev == dev) {
                memcpy(map, &e.map, sizeof(CUtensorMap));
                return NVLLM_B200_OK;
            }
        }
    }
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(NVLLM_B200_EDRIVER, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)KVH, (cuuint64_t)num_slots};
    cuuint64_t strides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)KVH * kD * 2};
    cuuint32_t box[3] = {64, 1, (cuuint32_t)kTile};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NVLLM_B200_EDRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    std::lock_guard<std::mutex> lock(mu);
    Entry& e = table[used < kEntries ? used++ : (next = (next + 1) % kEntries)];
    e.base = base;
    e.num_slots = num_slots;
    e.kvh = KVH;
    e.dev = dev;
    memcpy(&e.map, map, sizeof(CUtensorMap));
    return NVLLM_B200_OK;
}

static int ensure_smem_attr() {
    static std::mutex mu;
    static bool done[64];
    int dev = 0;
    NVLLM_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !done[dev]) {
        NVLLM_CUDA_OK(cudaFuncSetAttribute(paged_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        done[dev] = true;
    }
    return NVLLM_B200_OK;
}

// What every decode entry point shares: the argument checks and the two launches.  `tickets` / `partials` point
// into whatever scratch the entry point owns; `step` (may be null) adds the scatter of the step's new K/V rows
// to the first launch.
struct DecodeArgs {
    const void *q, *k_cache, *v_cache;
    const int32_t *block_tables, *context_lens;
    void* out;
    int B, H, KVH, D, NB, block_size, MB;
    float scale;
    void* stream;
};
struct StepArgs {
    const void *k, *v;
    const int32_t* slot_mapping;
    int src_dtype;
};

static int check_decode_args(const char* who, const DecodeArgs& a) {
    if (a.B < 0 || a.H <= 0 || a.KVH <= 0 || a.NB <= 0 || a.block_size <= 0 || a.MB <= 0)
        return fail(NVLLM_B200_EINVAL, "%s: non-positive size (B=%d H=%d KVH=%d NB=%d block=%d MB=%d)", who, a.B, a.H,
                    a.KVH, a.NB, a.block_size, a.MB);
    if (a.D != kD) return fail(NVLLM_B200_EUNSUPPORTED, "%s: head_dim %d (only 128)", who, a.D);
    if (a.block_size % kTile != 0)
        return fail(NVLLM_B200_EUNSUPPORTED, "%s: block_size %d must be a multiple of %d", who, a.block_size, kTile);
    if (a.H % a.KVH != 0 || a.H / a.KVH > kMaxG)
        return fail(NVLLM_B200_EUNSUPPORTED, "%s: H/KVH = %d/%d must be an integer <= %d", who, a.H, a.KVH, kMaxG);
    if ((long long)a.MB * a.block_size > 0x3fffffffLL || (long long)a.NB * a.block_size > 0x7fffffffLL)
        return fail(NVLLM_B200_EUNSUPPORTED, "%s: cache or context too large for 32-bit token indices", who);
    if ((long long)a.B * a.KVH > 0x3fffffffLL) return fail(NVLLM_B200_EUNSUPPORTED, "%s: batch too large", who);
    return NVLLM_B200_OK;
}

static int check_decode_pointers(const char* who, const DecodeArgs& a) {
    if (!a.q || !a.k_cache || !a.v_cache || !a.block_tables || !a.context_lens || !a.out)
        return fail(NVLLM_B200_EINVAL, "%s: null pointer", who);
    if (((uintptr_t)a.q | (uintptr_t)a.k_cache | (uintptr_t)a.v_cache | (uintptr_t)a.out) & 15)
        return fail(NVLLM_B200_EINVAL, "%s: q/k_cache/v_cache/out must be 16-byte aligned", who);
    if (a.KVH > main_grid())
        return fail(NVLLM_B200_EUNSUPPORTED, "%s: KVH %d exceeds the CTA count %d", who, a.KVH, main_grid());
    return NVLLM_B200_OK;
}

static int launch_decode(const char* who, const DecodeArgs& a, const StepArgs* step, unsigned int* tickets,
                         float* partials, const preattn::Params* pre = nullptr) {
    int rc = ensure_smem_attr();
    if (rc) return rc;
    CUtensorMap tm_k, tm_v;
    const int64_t num_slots = (int64_t)a.NB * a.block_size;
    if ((rc = cached_cache_map(&tm_k, a.k_cache, num_slots, a.KVH))) return rc;
    if ((rc = cached_cache_map(&tm_v, a.v_cache, num_slots, a.KVH))) return rc;

    Params p;
    p.q = (const __nv_bfloat16*)a.q;
    p.block_tables = a.block_tables;
    p.context_lens = a.context_lens;
    p.out = (__nv_bfloat16*)a.out;
    p.tickets = tickets;
    p.partials = partials;
    p.B = a.B;
    p.H = a.H;
    p.KVH = a.KVH;
    p.G = a.H / a.KVH;
    p.NB = a.NB;
    p.block_size = a.block_size;
    p.MB = a.MB;
    p.num_groups = main_grid() / a.KVH;
    p.item_cost = item_cost();
    p.scale_log2 = a.scale * 1.4426950408889634f;

    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.stream = reinterpret_cast<cudaStream_t>(a.stream);
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;

    const int num_tickets = a.B * a.KVH;
    const int clear_blocks = (num_tickets + kStoreThreads - 1) / kStoreThreads;
    const int row_chunks = a.KVH * kD / 8;
    const int64_t total_chunks = step ? (int64_t)a.B * row_chunks : 0;
    const int64_t store_blocks = step ? store_blocks_for(total_chunks) : 0;
    if (store_blocks + clear_blocks > 0x7fffffffLL) return fail(NVLLM_B200_EUNSUPPORTED, "%s: batch too large", who);
    cfg.gridDim = dim3((unsigned)(store_blocks + clear_blocks));
    cfg.blockDim = dim3(kStoreThreads);
    cfg.dynamicSmemBytes = 0;
    if (pre) {
        const int64_t pre_blocks = preattn::blocks_for(pre->T, pre->H, pre->KVH);
        cfg.gridDim = dim3((unsigned)(pre_blocks + clear_blocks));
        cfg.blockDim = dim3(preattn::kThreads);
        NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_prepare_fused_kernel, tickets, num_tickets, (int)pre_blocks, *pre));
    } else if (step && step->src_dtype == NVLLM_B200_DTYPE_F32) {
        NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_prepare_kernel<float>, tickets, num_tickets, (int)store_blocks,
                                         (const float*)step->k, (const float*)step->v, (__nv_bfloat16*)a.k_cache,
                                         (__nv_bfloat16*)a.v_cache, step->slot_mapping, total_chunks, row_chunks,
                                         num_slots));
    } else {
        NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, decode_prepare_kernel<__nv_bfloat16>, tickets, num_tickets,
                                         (int)store_blocks, (const __nv_bfloat16*)(step ? step->k : nullptr),
                                         (const __nv_bfloat16*)(step ? step->v : nullptr), (__nv_bfloat16*)a.k_cache,
                                         (__nv_bfloat16*)a.v_cache, step ? step->slot_mapping : nullptr, total_chunks,
                                         row_chunks, num_slots));
    }
    cfg.gridDim = dim3((unsigned)(p.num_groups * a.KVH));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, paged_decode_kernel, tm_k, tm_v, p));
    return NVLLM_B200_OK;
}

static int decode_with_workspace(const char* who, const DecodeArgs& a, const StepArgs* step, void* workspace,
                                 size_t workspace_bytes, const preattn::Params* pre = nullptr) {
    int rc = check_decode_args(who, a);
    if (rc) return rc;
    if (step) {
        if (step->src_dtype != NVLLM_B200_DTYPE_BF16 && step->src_dtype != NVLLM_B200_DTYPE_F32)
            return fail(NVLLM_B200_EUNSUPPORTED, "%s: src_dtype %d", who, step->src_dtype);
    }
    if (a.B == 0) return NVLLM_B200_OK;
    if ((rc = check_decode_pointers(who, a))) return rc;
    if (step) {
        if (!step->k || !step->v || !step->slot_mapping) return fail(NVLLM_B200_EINVAL, "%s: null pointer", who);
        if (((uintptr_t)step->k | (uintptr_t)step->v) & 15)
            return fail(NVLLM_B200_EINVAL, "%s: k/v must be 16-byte aligned", who);
    }
    const size_t need = nvllm_b200_paged_decode_workspace_bytes(a.B, a.H, a.KVH, a.D, a.MB, a.block_size);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 255))
        return fail(NVLLM_B200_EWORKSPACE, "%s: workspace of %zu bytes (256-byte aligned) required, got %zu", who, need,
                    workspace ? workspace_bytes : (size_t)0);
    return launch_decode(who, a, step, (unsigned int*)workspace,
                         (float*)((uint8_t*)workspace + ticket_bytes(a.B, a.KVH)), pre);
}

}  // namespace decode
}  // namespace nvllm

extern "C" size_t nvllm_b200_paged_decode_workspace_bytes(int B, int H, int KVH, int D, int MB, int block_size) {
    using namespace nvllm::decode;
    (void)D;
    (void)MB;
    (void)block_size;
    if (B < 0 || H <= 0 || KVH <= 0 || H % KVH != 0) return 256;
    return ticket_bytes(B, KVH) + partial_bytes(main_grid(), H / KVH) + 256;
}

extern "C" int nvllm_b200_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                                       const int32_t* block_tables, const int32_t* context_lens, void* out,
                                       void* workspace, size_t workspace_bytes, int B, int H, int KVH, int D, int NB,
                                       int block_size, int MB, float scale, void* stream) {
    using namespace nvllm::decode;
    const DecodeArgs a = {q, k_cache, v_cache, block_tables, context_lens, out, B, H, KVH, D, NB, block_size, MB, scale,
                          stream};
    return decode_with_workspace("paged_decode", a, nullptr, workspace, workspace_bytes);
}

extern "C" int nvllm_b200_decode_step(const void* q, const void* k, const void* v, void* k_cache, void* v_cache,
                                      const int32_t* slot_mapping, const int32_t* block_tables,
                                      const int32_t* context_lens, void* out, void* workspace, size_t workspace_bytes,
                                      int B, int H, int KVH, int D, int NB, int block_size, int MB, float scale,
                                      int src_dtype, void* stream) {
    using namespace nvllm::decode;
    const DecodeArgs a = {q, k_cache, v_cache, block_tables, context_lens, out, B, H, KVH, D, NB, block_size, MB, scale,
                          stream};
    const StepArgs s = {k, v, slot_mapping, src_dtype};
    return decode_with_workspace("decode_step", a, &s, workspace, workspace_bytes);
}

namespace nvllm {
namespace preattn {
int check_args(const char* who, const void* q, const void* k, const void* v, const float* q_weight, const float* k_weight,
               const float* cos_sin_cache, const int32_t* positions, const void* k_cache, const void* v_cache,
               const int32_t* slot_mapping, int64_t T, int H, int KVH, int D, int64_t num_slots, int64_t max_pos);
}
}  // namespace nvllm

extern "C" int nvllm_b200_fused_decode_step(void* q, void* k, const void* v, const float* q_weight, const float* k_weight,
                                            const float* cos_sin_cache, const int32_t* positions, int64_t max_pos,
                                            float eps, void* k_cache, void* v_cache, const int32_t* slot_mapping,
                                            const int32_t* block_tables, const int32_t* context_lens, void* out,
                                            void* workspace, size_t workspace_bytes, int B, int H, int KVH, int D, int NB,
                                            int block_size, int MB, float scale, void* stream) {
    using namespace nvllm;
    using namespace nvllm::decode;
    const int64_t num_slots = (int64_t)NB * block_size;
    int rc = preattn::check_args("fused_decode_step", q, k, v, q_weight, k_weight, cos_sin_cache, positions, k_cache, v_cache,
                                 slot_mapping, B, H, KVH, D, num_slots, max_pos);
    if (rc) return rc;
    const DecodeArgs a = {q, k_cache, v_cache, block_tables, context_lens, out, B, H, KVH, D, NB, block_size, MB, scale,
                          stream};
    const preattn::Params pp{(__nv_bfloat16*)q, (__nv_bfloat16*)k, (const __nv_bfloat16*)v, q_weight, k_weight,
                             cos_sin_cache, positions, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, slot_mapping,
                             (int64_t)B, H, KVH, num_slots, max_pos, eps};
    return decode_with_workspace("fused_decode_step", a, nullptr, workspace, workspace_bytes, &pp);
}

namespace nvllm {
int read_decode_flags(int* out) {
    NVLLM_CUDA_OK(cudaMemcpyFromSymbol(out, decode::g_error_flag, sizeof(int)));
    return NVLLM_B200_OK;
}
int clear_decode_flags() {
    const int zero = 0;
    NVLLM_CUDA_OK(cudaMemcpyToSymbol(decode::g_error_flag, &zero, sizeof(int)));
    return NVLLM_B200_OK;
}
}  // namespace nvllm

// ---------------------------------------------------------------------------
// paged decode without a caller-provided workspace
// ---------------------------------------------------------------------------
// Some hosts of this library cannot hand it scratch memory and cannot obtain any at call time: a custom-call
// handler whose operand list is fixed by the framework, running in a process where the framework's own pool
// has already reserved nearly all of HBM (so a cudaMalloc there fails or starves the pool), or a serving
// loop that must not take the device-wide synchronisation that cudaMalloc / cudaFree imply.  For them the
// split-K scratch of the decode kernels lives in this fixed array, which every device that loads the
// library carries until the process exits.
//
// Sizes are capped so the array stays small: B * KVH <= kStaticMaxTickets and a main grid of at most
// kStaticMaxCtas CTAs (2 per SM, i.e. devices with up to 160 SMs).
namespace nvllm {
namespace decode {

constexpr int kStaticMaxBatch = 4096;
constexpr int kStaticMaxTickets = kStaticMaxBatch * 8;
constexpr int kStaticMaxCtas = 320;
constexpr size_t kStaticTicketBytes = (size_t)kStaticMaxTickets * 4;
constexpr size_t kStaticPartialBytes = (size_t)kStaticMaxCtas * 2 * ((size_t)kMaxG * kD + 2 * kMaxG) * 4;
constexpr size_t kStaticScratchBytes = kStaticTicketBytes + kStaticPartialBytes;  // about 2.8 MB

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device.  In host code the array's name is only a handle
// for the runtime, never a pointer a kernel may use, so the address is looked up once per device (with that
// device current) and cached.
static int static_scratch_address(void** out) {
    static std::mutex mu;
    static void* cached[64];
    int dev = 0;
    NVLLM_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(NVLLM_B200_EUNSUPPORTED, "paged_decode_static: device ordinal %d", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(NVLLM_B200_ECUDA, "paged_decode_static: cudaGetSymbolAddress failed: %s",
                        cudaGetErrorString(e));
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return NVLLM_B200_OK;
}

}  // namespace decode
}  // namespace nvllm

extern "C" int nvllm_b200_paged_decode_static(const void* q, const void* k_cache, const void* v_cache,
                                              const int32_t* block_tables, const int32_t* context_lens, void* out,
                                              int B, int H, int KVH, int D, int NB, int block_size, int MB,
                                              float scale, void* stream) {
    using namespace nvllm;
    using namespace nvllm::decode;
    const char* who = "paged_decode_static";
    const DecodeArgs a = {q, k_cache, v_cache, block_tables, context_lens, out, B, H, KVH, D, NB, block_size, MB, scale,
                          stream};
    int rc = check_decode_args(who, a);
    if (rc) return rc;
    if (B > kStaticMaxBatch || (long long)B * KVH > kStaticMaxTickets)
        return fail(NVLLM_B200_EWORKSPACE,
                    "paged_decode_static: batch %d x %d kv heads exceeds the built-in scratch (max %d sequences and "
                    "%d sequence-heads); use nvllm_b200_paged_decode with a caller workspace",
                    B, KVH, kStaticMaxBatch, kStaticMaxTickets);
    if (main_grid() > kStaticMaxCtas)
        return fail(NVLLM_B200_EWORKSPACE,
                    "paged_decode_static: this device needs %d CTAs, the built-in scratch holds %d; use "
                    "nvllm_b200_paged_decode with a caller workspace",
                    main_grid(), kStaticMaxCtas);
    if (B == 0) return NVLLM_B200_OK;
    if ((rc = check_decode_pointers(who, a))) return rc;
    void* scratch = nullptr;
    if ((rc = static_scratch_address(&scratch))) return rc;
    return launch_decode(who, a, nullptr, (unsigned int*)scratch, (float*)((uint8_t*)scratch + kStaticTicketBytes));
}
