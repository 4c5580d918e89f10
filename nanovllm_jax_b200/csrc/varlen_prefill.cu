// varlen_prefill: causal attention over packed variable-length sequences on the
// sm_100a tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Replaces variable_length_attention_prefill (reference layers/attention.py:135-279)
// and paged_prefill_attention (layers/pallas_attention.py:557-608).  Keys and values
// are either packed like the queries ([T, KVH, 128], cu_seqlens_k == cu_seqlens_q) or
// read from the paged cache through block tables (prefix-cached prefill,
// cu_seqlens_k >= cu_seqlens_q: query i of a sequence sits at position prefix + i,
// prefix = len_k - len_q; the model runner attaches the tables on a prefix hit,
// engine/model_runner.py:311-314).
//
// Work item = two 128-row Q tiles (A and B) that share every K/V tile they read.  When
// the GQA group size is even the two tiles are the same 128 query rows of two q heads of
// one kv head: both see the same keys, run the same number of K/V tiles and finish
// together.  Otherwise they are two consecutive row blocks of one head (B then sees one
// K/V tile more than A).  A tiny plan kernel turns cu_seqlens into the list of
// (sequence, row block) pairs, longest causal span first; one persistent CTA per SM
// takes items round-robin from that list (heavy ones first, so the CTAs finish
// together), and the heads of one (sequence, row block) are neighbours in the list so
// that the G heads of a kv head find each other's K/V tiles in L2.  Tensor memory and
// barriers are set up once per CTA; the loads of the next item are already in flight
// while the current one drains.
//
// Per CTA (12 warps = 3 warpgroups; the first gives registers away with setmaxnreg, the softmax
// warpgroups take them):
//   warp 0      TMA producer: Q tiles once per item, then K and V tiles [128 tokens x
//               128 dims] through one five-slot mbarrier ring filled K0 V0 K1 V1 ...
//               (cp.async.bulk.tensor, 128-byte swizzle, no multicast): K(j+2) takes the
//               slot V(j-1) leaves and V(j+2) the slot K(j) leaves, so every tile is
//               requested about two tiles before it is needed.
//   warps 1, 2  MMA issuers, one thread each for Q tile A and Q tile B: S = Q K^T
//               (operands in shared memory) and O += P V (P read from tensor memory, V
//               from shared memory, MN-major), M = N = 128, K = 16 per instruction;
//               tcgen05.commit signals the mbarriers.  K(j+1) is awaited before P.V(j) is
//               issued and all commits of the pair follow the Q.K^T(j+1) MMAs, so nothing
//               is polled between the two groups of MMAs.  Warp 1 also owns the tensor-
//               memory allocation (512 columns: S_A S_B O_A O_B).
//   warps 4-7   softmax of tile A, warps 8-11 of tile B: one thread per query row holds
//               its S row (128 scores) in registers, keeps the running max / sum (packed
//               f32x2 math, 3-input max), writes bf16 P back over S in two halves (each
//               releases four P.V k-steps) and rescales O only when the max grew by more
//               than 2^8 (exact: the stale max is carried into the final normalisation).
//               Tiles strictly above the diagonal are skipped, the diagonal tile is
//               masked element-wise.  The exponentials of the two tiles take turns
//               (A(0) B(0) A(1) ...): they share the four MUFU pipes, which bound the
//               kernel, and alternating keeps one tile's MMAs, score loads and row max
//               running under the other tile's exponentials.
// Measures that only pay off together (each alone hits the next bottleneck at the same level): two
// MMA issuers, the five-slot ring, the turn-taking, and -- later -- turn-taking for the exponentials
// alone together with the poll-free MMA issue order.
// Every mbarrier wait is bounded; on timeout the CTA raises a device error flag,
// stops issuing work, and still releases its tensor memory before it exits.
#include "common.cuh"

#include <mutex>
#include <type_traits>

namespace nvllm {
namespace prefill {

// bit 2 (4): pipeline wait timed out; bit 4 (16): sequence too long for the plan kernel; bit 5 (32): a sequence has
// fewer keys than queries, or (packed keys) a different number -- nothing is computed for that call
__device__ int g_error_flag = 0;

constexpr int kD = 128;
constexpr int kTileQ = 128;            // rows per Q tile
constexpr int kBlockQ = 2 * kTileQ;    // rows per work item when its two Q tiles are row blocks of one head
constexpr int kTileKV = 128;
constexpr int kThreads = 384;            // 3 warpgroups: {TMA, MMA, 2 idle warps} | softmax A | softmax B
constexpr int kPanelBytes = 128 * 128;  // 128 rows x 64 dims bf16, 128B-swizzled
constexpr int kTileBytes = 2 * kPanelBytes;
constexpr int kSlots = 5;                // one ring for K and V tiles, filled in the order K0 V0 K1 V1 ...
constexpr int kSmemTiles = (2 + kSlots) * kTileBytes;  // Q_A Q_B | K/V ring  (224 KB)
constexpr int kSmemBytes = kSmemTiles + 512 + 1024;
constexpr int kMaxLevels = 2048;       // row blocks per sequence the plan kernel can rank
constexpr uint32_t kTmemCols = 512;
constexpr float kRescaleThreshold = 8.0f;  // log2 units

struct Params {
    const int4* items;  // record 0: {number of (sequence, row block) pairs, 0, 0, 0}; then two records per pair, longest
                        // causal span first: {first query token of the sequence, its query length, first row of the
                        // block, sequence index} and {first key token (packed keys), key length, 0, 0}
    const int32_t* block_tables;  // [B, MB] page ids, or nullptr for packed keys/values
    int MB, block_size;
    __nv_bfloat16* out;
    int H, G;
    int pair_heads;  // 1: an item is 128 rows of heads (2h, 2h+1); 0: 256 rows of one head
    float scale_log2;
};

// ------------------------------------------------------------------------------------------
// tcgen05 wrappers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
                 "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc)
        : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base + i), columns c..c+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
        "%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
        "%31,%32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 32 lanes x 16 columns, from the first 16 words of r.
template <int N>
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[N]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
            taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// Packed fp32 pairs (one instruction, two lanes of math) and the three-input max of sm_100.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;  // descriptor version
    d |= (uint64_t)2 << 61;  // SWIZZLE_128B
    return d;
}
// K-major operand tile [128 rows][128 dims] stored as two 64-dim panels; k-step = 16 dims.
__device__ __forceinline__ uint64_t kmajor_desc(uint32_t tile_addr, int ks) {
    return make_desc(tile_addr + (ks >> 2) * kPanelBytes + (ks & 3) * 32, 16, 1024);
}
// MN-major operand: V tile [128 tokens][128 dims] as two 64-dim panels; N = dims, K = tokens; k-step = 16 tokens.
__device__ __forceinline__ uint64_t mnmajor_desc(uint32_t tile_addr, int ks) {
    return make_desc(tile_addr + ks * 16 * 128, kPanelBytes, 1024);
}

constexpr uint32_t kIdescQK = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescPV = kIdescQK | (1u << 16);  // B operand MN-major

// ------------------------------------------------------------------------------------------
// plan kernel: (sequence, row block) pairs sorted by causal span, largest first
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) prefill_plan_kernel(const int32_t* __restrict__ cu_seqlens,
                                                            const int32_t* __restrict__ cu_k, int paged, int B,
                                                            int4* __restrict__ items, int capacity, int bq) {
    // bq = query rows per block (256, or 128 when an item is two heads).  A row block's weight is its causal span in
    // bq-key units: level = prefix / bq + block index.
    __shared__ int hist[kMaxLevels];
    __shared__ int base[kMaxLevels];
    __shared__ int max_level, bad;
    griddep_wait();
    griddep_launch_dependents();
    for (int i = threadIdx.x; i < kMaxLevels; i += blockDim.x) hist[i] = 0;
    if (threadIdx.x == 0) max_level = 0, bad = 0;
    __syncthreads();
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const int len = cu_seqlens[b + 1] - cu_seqlens[b];
        const int len_k = cu_k[b + 1] - cu_k[b];
        // keys can never be fewer than queries; packed keys sit beside the queries, so the counts must be equal
        if (len > 0 && (len_k < len || (!paged && (len_k != len || cu_k[b] != cu_seqlens[b])))) bad = 1;
        const int lvl0 = len_k > len ? (len_k - len) / bq : 0;
        const int n = len > 0 ? (len + bq - 1) / bq : 0;
        for (int l = 0; l < n; ++l) {
            int lvl = lvl0 + l;
            if (lvl >= kMaxLevels) {
                lvl = kMaxLevels - 1;
                atomicOr(&g_error_flag, 16);
            }
            atomicAdd(&hist[lvl], 1);
            atomicMax(&max_level, lvl + 1);
        }
    }
    __syncthreads();
    if (bad) {  // uniform: publish an empty list so that the main kernel computes nothing
        if (threadIdx.x == 0) {
            items[0] = make_int4(0, 0, 0, 0);
            atomicOr(&g_error_flag, 32);
        }
        return;
    }
    if (threadIdx.x == 0) {
        int run = 0;
        for (int l = max_level - 1; l >= 0; --l) {
            base[l] = run;
            run += hist[l];
        }
        items[0] = make_int4(run < capacity ? run : capacity, 0, 0, 0);
    }
    __syncthreads();
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const int start = cu_seqlens[b];
        const int len = cu_seqlens[b + 1] - start;
        const int len_k = cu_k[b + 1] - cu_k[b];
        const int lvl0 = len_k > len ? (len_k - len) / bq : 0;
        const int n = len > 0 ? (len + bq - 1) / bq : 0;
        for (int l = 0; l < n; ++l) {
            const int lvl = min(lvl0 + l, kMaxLevels - 1);
            const int slot = atomicAdd(&base[lvl], 1);
            if (slot < capacity) {
                items[1 + 2 * slot] = make_int4(start, len, l * bq, b);
                items[2 + 2 * slot] = make_int4(cu_k[b], len_k, 0, 0);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------
// main kernel
// ------------------------------------------------------------------------------------------
struct Shared {
    uint64_t q_full, q_empty;
    uint64_t kv_full[kSlots], kv_empty[kSlots];
    uint64_t s_full[2], p_full[2][2], o_full[2], o_empty[2];
    uint64_t turn[2];  // softmax ping-pong: turn[0] = "tile A finished a softmax", turn[1] = "tile B finished one"
    uint32_t tmem_base;
    volatile int abort_flag;
};

__device__ __forceinline__ bool wait_or_abort(Shared* sh, uint64_t* bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    if (sh->abort_flag) return false;
    if (mbar_wait(bar, parity)) return true;
    sh->abort_flag = 1;
    atomicOr(&g_error_flag, 4);
    return false;
}

struct Item {
    int seq_start, len, q0, head, b;  // first query token of the sequence, query length, first row of the block
    int k_start, len_k, prefix;       // first key token (packed keys), key length, len_k - len
    int dq, dh;          // Q tile B = rows + dq of head + dh
    int n_a, n_b, n_kv;  // KV tiles seen by Q tile A, by Q tile B (0: no such rows; else n_a or n_a + 1), and the larger
    bool ragged;         // the last KV tile reaches past the sequence's last key
};

__device__ __forceinline__ Item load_item(const Params& p, int idx) {
    Item it;
    const int per_pair = p.pair_heads ? p.H >> 1 : p.H;
    const int pair = idx / per_pair;
    it.head = (idx - pair * per_pair) << p.pair_heads;
    it.dq = p.pair_heads ? 0 : kTileQ;
    it.dh = p.pair_heads;
    const int4 r = __ldg(p.items + 1 + 2 * pair), rk = __ldg(p.items + 2 + 2 * pair);
    it.seq_start = r.x;
    it.len = r.y;
    it.q0 = r.z;
    it.b = r.w;
    it.k_start = rk.x;
    it.len_k = rk.y;
    it.prefix = it.len_k - it.len;  // >= 0: the plan kernel publishes no items otherwise
    const int rows = min(p.pair_heads ? kTileQ : kBlockQ, it.len - it.q0);
    const int nk_total = (it.len_k + kTileKV - 1) / kTileKV;
    // the last row of Q tile x sees keys 0 .. prefix + q0 + 128 x + 127
    it.n_a = min(nk_total, (it.prefix + it.q0 + kTileQ - 1) / kTileKV + 1);
    it.n_b = p.pair_heads ? it.n_a
                          : (rows > kTileQ ? min(nk_total, (it.prefix + it.q0 + 2 * kTileQ - 1) / kTileKV + 1) : 0);
    it.n_kv = max(it.n_a, it.n_b);
    it.ragged = it.n_kv * kTileKV > it.len_k;
    return it;
}

// First token (row of the k / v tensor map) of KV tile j of the item's sequence.
__device__ __forceinline__ int kv_tile_token(const Params& p, const Item& it, int j) {
    const int off = j * kTileKV;
    if (p.block_tables == nullptr) return it.k_start + off;
    int page = __ldg(p.block_tables + (size_t)it.b * p.MB + off / p.block_size);
    if (page < 0) page = 0;  // a padding entry: never reached for keys below len_k
    return page * p.block_size + off % p.block_size;  // block_size is a multiple of the tile: a tile never straddles pages
}

// One 128-column S row -> running max, optional O rescale, bf16 P in two halves.  DIAG: key column c of this tile is
// visible iff c <= lim (lim may be negative -- nothing visible in this tile -- or >= 127).  turn_bar (or null): the
// other tile's hand-over this tile's exponentials wait for; turn_out (or null): where this tile hands over.
// The whole row is held in registers (the softmax warpgroups raise their register budget with setmaxnreg), so
// tensor memory is read once and its latency is paid once per tile.
template <bool DIAG>
__device__ __forceinline__ bool softmax_tile(Shared* sh, const int x, const uint32_t t_s, const uint32_t t_o,
                                             const int lim, const bool first, const uint32_t o_parity_prev,
                                             const float scale_log2, float& m_run, float& m_used, float& l,
                                             uint64_t* turn_bar, const uint32_t turn_parity, uint64_t* turn_out) {
    uint32_t v[4][32];
    tmem_ld32(t_s, v[0]);
    tmem_ld32(t_s + 32, v[1]);
    tmem_ld32(t_s + 64, v[2]);
    tmem_ld32(t_s + 96, v[3]);
    tmem_wait_ld();
    float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
            if (DIAG) {  // mask in place so that the second pass needs no select
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (c * 32 + i + u > lim) v[c][i + u] = 0xFF800000u;
            }
            mx0 = max3(mx0, __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
            mx1 = max3(mx1, __uint_as_float(v[c][i + 2]), __uint_as_float(v[c][i + 3]));
            mx2 = max3(mx2, __uint_as_float(v[c][i + 4]), __uint_as_float(v[c][i + 5]));
            mx3 = max3(mx3, __uint_as_float(v[c][i + 6]), __uint_as_float(v[c][i + 7]));
        }
    }
    m_run = fmaxf(m_run, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)));
    if (turn_bar != nullptr && !wait_or_abort(sh, turn_bar, turn_parity)) return false;
    if (first) {
        m_used = m_run;  // finite: key 0 of the sequence is visible to every row and sits in the first tile
    } else {
        const bool grow = (m_run - m_used) * scale_log2 > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
            // O holds sums relative to m_used: bring it to m_run before this tile's P.V is added.
            if (!wait_or_abort(sh, &sh->o_full[x], o_parity_prev)) return false;
            tc_fence_after();
            const float f = fast_exp2((m_used - m_run) * scale_log2);
#pragma unroll 1
            for (int c = 0; c < 8; ++c) {
                uint32_t ov[16];
                tmem_ld16(t_o + c * 16, ov);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * f);
                tmem_st16(t_o + c * 16, ov);
            }
            tmem_wait_st();
            l *= f;
            m_used = m_run;
        }
    }
    // p = 2^(s*scale - m) as bf16 pairs, written over the S columns (all of them are in registers by now):
    // chunk c (scores 32c..32c+31) becomes packed columns 16c..16c+15.
    const float neg = -m_used * scale_log2;
    const uint64_t scale2 = pack2(scale_log2, scale_log2), neg2 = pack2(neg, neg);
    uint64_t acc_a = pack2(0.f, 0.f), acc_b = pack2(0.f, 0.f);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            float x0, x1, x2, x3;
            unpack2(fma2(pack2(__uint_as_float(v[c][2 * i]), __uint_as_float(v[c][2 * i + 1])), scale2, neg2), x0, x1);
            unpack2(fma2(pack2(__uint_as_float(v[c][2 * i + 2]), __uint_as_float(v[c][2 * i + 3])), scale2, neg2), x2,
                    x3);
            const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);  // 2^-inf = 0 for masked keys
            const float e2 = fast_exp2(x2), e3 = fast_exp2(x3);
            acc_a = add2(acc_a, pack2(e0, e1));
            acc_b = add2(acc_b, pack2(e2, e3));
            v[c][i] = pack_bf16(e0, e1);  // in place: word i <= 2i has been consumed
            v[c][i + 1] = pack_bf16(e2, e3);
        }
        tmem_st16(t_s + c * 16, v[c]);
        if (c == 3 && turn_out != nullptr) {
            __syncwarp();
            if ((threadIdx.x & 31) == 0) mbar_arrive(turn_out);
        }
        if (c & 1) {  // a half of P (64 keys) is complete: release its four P.V k-steps
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if ((threadIdx.x & 31) == 0) mbar_arrive(&sh->p_full[x][c >> 1]);
        }
    }
    float s0, s1, s2, s3;
    unpack2(acc_a, s0, s1);
    unpack2(acc_b, s2, s3);
    l += (s0 + s1) + (s2 + s3);
    return true;
}

__global__ void __launch_bounds__(kThreads, 1)
varlen_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                      const __grid_constant__ CUtensorMap tm_v, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                                   // [2][tile]
    uint8_t* sKV = smem + 2 * kTileBytes;                 // [kSlots][tile]: ring position 2j holds K(j), 2j+1 holds V(j)
    Shared* sh = reinterpret_cast<Shared*>(smem + kSmemTiles);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        mbar_init(&sh->q_full, 1);
        mbar_init(&sh->q_empty, 2);   // both MMA issuers
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(&sh->kv_full[s], 1);
            mbar_init(&sh->kv_empty[s], 2);  // both MMA issuers
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(&sh->s_full[x], 1);
            mbar_init(&sh->p_full[x][0], kTileQ / 32);  // one arrival per softmax warp
            mbar_init(&sh->p_full[x][1], kTileQ / 32);
            mbar_init(&sh->o_full[x], 1);
            mbar_init(&sh->o_empty[x], kTileQ / 32);
            mbar_init(&sh->turn[x], kTileQ / 32);
        }
        sh->abort_flag = 0;
        sh->tmem_base = 0xFFFFFFFFu;
        fence_mbar_init();
        prefetch_tensormap(&tm_q);
        prefetch_tensormap(&tm_k);
        prefetch_tensormap(&tm_v);
    }
    __syncthreads();
    if (warp == 1) {
        tmem_alloc(&sh->tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sh->tmem_base;

    griddep_wait();  // the plan kernel's item list (and the caller's q/k/v) must be visible from here on

    // Register budget: the TMA / MMA warpgroup keeps 96 registers per thread, the two softmax warpgroups take 200
    // (96*128 + 200*256 <= 64K), enough to hold a whole 128-column score row.
    const int total = (tmem != 0xFFFFFFFFu) ? p.items[0].x * (p.pair_heads ? p.H >> 1 : p.H) : 0;
    const int first_idx = blockIdx.x, stride = gridDim.x;

    if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 96;");
    if (warp == 0) {
        // =============================== TMA producer ===============================
        if (lane == 0) {
            uint32_t kt = 0;
            int i = 0;
            bool ok = true;
            for (int idx = first_idx; ok && idx < total; idx += stride, ++i) {
                const Item it = load_item(p, idx);
                const int kvh = it.head / p.G;
                const int tok_q = it.seq_start + it.q0;
                if (i > 0 && !(ok = wait_or_abort(sh, &sh->q_empty, (i - 1) & 1u))) break;
                mbar_expect_tx(&sh->q_full, (it.n_b > 0 ? 2 : 1) * kTileBytes);
                tma_load_3d(sQ, &tm_q, &sh->q_full, 0, it.head, tok_q);
                tma_load_3d(sQ + kPanelBytes, &tm_q, &sh->q_full, 64, it.head, tok_q);
                if (it.n_b > 0) {
                    tma_load_3d(sQ + kTileBytes, &tm_q, &sh->q_full, 0, it.head + it.dh, tok_q + it.dq);
                    tma_load_3d(sQ + kTileBytes + kPanelBytes, &tm_q, &sh->q_full, 64, it.head + it.dh, tok_q + it.dq);
                }
                for (int j = 0; j < it.n_kv; ++j, ++kt) {
                    const int tok = kv_tile_token(p, it, j);
#pragma unroll
                    for (int kv = 0; kv < 2; ++kv) {  // K(j) then V(j): with five slots both are requested ~2 tiles ahead
                        const uint32_t pos = 2 * kt + kv;
                        const int slot = pos % kSlots;
                        if (!(ok = wait_or_abort(sh, &sh->kv_empty[slot], ((pos / kSlots) & 1u) ^ 1u))) break;
                        const CUtensorMap* tm = kv == 0 ? &tm_k : &tm_v;
                        mbar_expect_tx(&sh->kv_full[slot], kTileBytes);
                        tma_load_3d(sKV + slot * kTileBytes, tm, &sh->kv_full[slot], 0, kvh, tok);
                        tma_load_3d(sKV + slot * kTileBytes + kPanelBytes, tm, &sh->kv_full[slot], 64, kvh, tok);
                    }
                    if (!ok) break;
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ============================== MMA issuers ===============================
        // One issuing thread per Q tile (warp 1: tile A, warp 2: tile B).  An issuing thread blocks on every
        // tcgen05.mma until the tensor pipe accepts it and pays a couple of hundred cycles for every barrier it
        // polls; with two independent issuers one tile's bookkeeping hides behind the other tile's MMAs.  Each
        // thread owns its tile's S / P / O barriers; the shared K/V ring slots and the Q buffer are released by
        // both (their "empty" barriers count two arrivals: a tcgen05.commit from a thread that read the slot, a
        // plain arrive from a thread whose tile does not need it).
        if (lane == 0) {
            const int x = warp - 1;
            const uint32_t s_t = tmem + x * 128, o_t = tmem + 256 + x * 128;
            // Descriptors are built once: per k-step and per ring slot only the 14-bit start-address field
            // (bytes >> 4) moves, so issuing an MMA costs one 32-bit add instead of a descriptor rebuild.
            const uint64_t q_desc = kmajor_desc(smem_u32(sQ + x * kTileBytes), 0);
            const uint64_t k_desc0 = kmajor_desc(smem_u32(sKV), 0), v_desc0 = mnmajor_desc(smem_u32(sKV), 0);
            constexpr uint32_t kSlotStep = (uint32_t)(kTileBytes >> 4);  // next ring slot, in descriptor address units
            uint32_t kt = 0;     // K/V tiles consumed before this item
            uint32_t tiles = 0;  // tiles finished by this Q tile, over all items (barrier phases)
            uint32_t used = 0;   // items in which this Q tile was active (o_empty phases)
            int i = 0;
            bool ok = true;

            auto issue_qk = [&](uint64_t kd) {
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    const uint32_t step = (uint32_t)(((ks >> 2) * kPanelBytes + (ks & 3) * 32) >> 4);
                    mma_ss(s_t, q_desc + step, kd + step, kIdescQK, ks > 0);
                }
                tc_commit(&sh->s_full[x]);
            };
            auto issue_pv = [&](int j, uint64_t vd) -> bool {
                if (j == 0 && used > 0 && !wait_or_abort(sh, &sh->o_empty[x], (used - 1) & 1u)) return false;
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (!wait_or_abort(sh, &sh->p_full[x][half], tiles & 1u)) return false;
                    tc_fence_after();
#pragma unroll
                    for (int ks = half * 4; ks < half * 4 + 4; ++ks)
                        mma_ts(o_t, s_t + ks * 8, vd + (uint32_t)((ks * 16 * 128) >> 4), kIdescPV, (j > 0 || ks > 0));
                }
                ++tiles;
                return true;
            };
            // the slot holding ring position pos: K(j) sits at 2j, V(j) at 2j+1
            auto slot_full = [&](uint32_t pos) { return wait_or_abort(sh, &sh->kv_full[pos % kSlots], (pos / kSlots) & 1u); };

            for (int idx = first_idx; ok && idx < total; idx += stride, ++i) {
                const Item it = load_item(p, idx);
                const int n_x = x == 0 ? it.n_a : it.n_b;
                if (!(ok = wait_or_abort(sh, &sh->q_full, i & 1u))) break;
                if (n_x == 0) mbar_arrive(&sh->q_empty);  // this tile never reads the Q buffer of this item
                {
                    const uint32_t kpos = 2 * kt;
                    if (!(ok = slot_full(kpos))) break;
                    if (n_x > 0) {
                        tc_fence_after();
                        issue_qk(k_desc0 + (kpos % kSlots) * kSlotStep);
                        tc_commit(&sh->kv_empty[kpos % kSlots]);
                        if (n_x == 1) tc_commit(&sh->q_empty);
                    } else {
                        mbar_arrive(&sh->kv_empty[kpos % kSlots]);
                    }
                }
                for (int j = 0; ok && j < it.n_kv; ++j) {
                    const uint32_t vpos = 2 * (kt + j) + 1, kpos = vpos + 1;  // ring positions of V(j) and K(j+1)
                    if (!(ok = slot_full(vpos))) break;
                    if (j + 1 < it.n_kv && !(ok = slot_full(kpos))) break;
                    if (j < n_x) {
                        if (!(ok = issue_pv(j, v_desc0 + (vpos % kSlots) * kSlotStep))) break;
                        if (!(j + 1 < n_x)) {
                            tc_commit(&sh->o_full[x]);
                            tc_commit(&sh->kv_empty[vpos % kSlots]);
                        }
                    } else {
                        mbar_arrive(&sh->kv_empty[vpos % kSlots]);
                    }
                    if (j + 1 < it.n_kv) {
                        if (j + 1 < n_x) {
                            issue_qk(k_desc0 + (kpos % kSlots) * kSlotStep);
                            tc_commit(&sh->kv_empty[kpos % kSlots]);
                            tc_commit(&sh->o_full[x]);
                            tc_commit(&sh->kv_empty[vpos % kSlots]);
                            if (j + 2 == n_x) tc_commit(&sh->q_empty);  // this tile's last Q.K^T has been issued
                        } else {
                            mbar_arrive(&sh->kv_empty[kpos % kSlots]);
                        }
                    }
                }
                used += n_x > 0 ? 1 : 0;
                kt += it.n_kv;
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 200;");
        // ============================ softmax warpgroups ============================
        const int x = (warp - 4) >> 2;              // 0: tile A, 1: tile B
        const int quarter = warp & 3;               // tensor-memory lane quarter this warp may touch
        const int row = quarter * 32 + lane;        // row within the Q tile
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const uint32_t t_s = tmem + x * 128 + lane_base;
        const uint32_t t_o = tmem + 256 + x * 128 + lane_base;
        uint32_t tiles = 0;  // tiles finished by this Q tile over all items (barrier phases)
        // Ping-pong between the two softmax warpgroups.  Both tiles' exponentials go through the same four MUFU
        // pipes; if both warpgroups exponentiate at once each takes twice as long and afterwards both tiles' MMAs
        // queue up behind one another.  Inside an item with both tiles active the exponentials therefore alternate
        // A(0) B(0) A(1) B(1) ...: a warpgroup loads its scores and finds the row max while the other one still
        // exponentiates, takes the turn, and hands it over once its last chunk of P is on its way to tensor memory.
        uint32_t turns_seen = 0;  // completions of the other tile's turn barrier this warp has consumed
        uint32_t kt = 0;          // K/V tiles of the items before this one (ring positions)
        bool ok = true;
        for (int idx = first_idx; ok && idx < total; idx += stride) {
            const Item it = load_item(p, idx);
            const int n_x = x == 0 ? it.n_a : it.n_b;
            const uint32_t kt0 = kt;
            kt += it.n_kv;
            if (n_x == 0) continue;
            const bool both = it.n_b > 0;
            const int q_pos = it.q0 + x * it.dq + row;             // row of the sequence's query block
            const int first_lim = it.prefix + it.q0 + x * it.dq;  // last key visible to the first row of this Q tile
            float m_run = -INFINITY, m_used = -INFINITY, l = 0.f;
            // One KV tile of this Q tile.  Tiles whose last key the tile's first row may still see need no mask; the
            // one or two after them (one when the prefix is a multiple of the tile) are masked per element.  The two
            // kinds run in two separate loops so that each loop body is straight-line code.
            auto tile_step = [&](const int j, auto diag) -> bool {
                constexpr bool kDiag = decltype(diag)::value;
                if (!wait_or_abort(sh, &sh->s_full[x], tiles & 1u)) return false;
                // A(j) starts after B(j-1); B(j) starts after A(j) while A still has tiles.
                uint64_t* turn_bar = nullptr;
                const uint32_t turn_parity = turns_seen & 1u;
                if (both && (x == 0 ? j >= 1 : j < it.n_a)) {
                    turn_bar = &sh->turn[x ^ 1];
                    ++turns_seen;
                }
                tc_fence_after();
                if (kDiag && it.ragged && j == it.n_kv - 1) {
                    // The last KV tile of the sequence reaches past its last key: those rows of the V tile hold
                    // whatever follows in memory (the next sequence, padding, recycled cache rows).  Their
                    // probabilities are exactly zero, but 0 * NaN or 0 * Inf in the P.V product would still poison the
                    // row, so each thread zeroes "its" row of the V tile before this tile's P is handed over (the
                    // hand-over orders these stores before the MMA that reads them).  Garbage in the K rows is
                    // harmless: those scores are overwritten with -inf by the mask.  This warpgroup trails the MMA
                    // issuer, and the slot cannot be refilled before P.V of this very tile, so the parity wait sees
                    // either "still loading" or "landed", never another tile.  When both Q tiles use the tile both
                    // warpgroups zero it (same bytes, same value).  (Such a tile is always a masked one.)
                    const uint32_t vpos = 2 * (kt0 + it.n_kv - 1) + 1;
                    if (!wait_or_abort(sh, &sh->kv_full[vpos % kSlots], (vpos / kSlots) & 1u)) return false;
                    if (row >= it.len_k - (it.n_kv - 1) * kTileKV) {
                        // a row is 128 contiguous bytes in each 64-dim panel (the swizzle permutes inside a row)
                        uint8_t* vrow = sKV + (vpos % kSlots) * kTileBytes + row * 128;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            *reinterpret_cast<uint4*>(vrow + c * 16) = make_uint4(0, 0, 0, 0);
                            *reinterpret_cast<uint4*>(vrow + kPanelBytes + c * 16) = make_uint4(0, 0, 0, 0);
                        }
                        fence_proxy_async_smem();  // generic-proxy stores must be visible to the tensor core's reads
                    }
                }
                if (!softmax_tile<kDiag>(sh, x, t_s, t_o, kDiag ? first_lim - j * kTileKV + row : 0, j == 0,
                                         (tiles - 1) & 1u, p.scale_log2, m_run, m_used, l, turn_bar, turn_parity,
                                         (both && (x == 0 || j + 1 < it.n_a)) ? &sh->turn[x] : nullptr))
                    return false;
                // hand the turn over: A after each of its tiles, B while A still has a tile that will wait for it
                ++tiles;
                return true;
            };
            const int n_plain = min(n_x, (first_lim + 1) / kTileKV);  // tiles j with j * 128 + 127 <= first_lim
            int j = 0;
            for (; ok && j < n_plain; ++j) ok = tile_step(j, std::false_type{});
            for (; ok && j < n_x; ++j) ok = tile_step(j, std::true_type{});
            if (!ok) break;
            // ---- epilogue: O / l -> bf16 -> global, then hand O back to the MMA thread ----
            if (!(ok = wait_or_abort(sh, &sh->o_full[x], (tiles - 1) & 1u))) break;
            tc_fence_after();
            const float inv = 1.0f / l;
            __nv_bfloat16* orow = p.out + ((size_t)(it.seq_start + q_pos) * p.H + it.head + x * it.dh) * kD;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t ov[32];
                tmem_ld32(t_o + c * 32, ov);
                tmem_wait_ld();
                if (q_pos < it.len) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(ov[8 * i + 0]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = w;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh->o_empty[x]);
        }
    }

    // ---- teardown: everyone meets here, then the allocating warp frees tensor memory ----
    tc_fence_before();
    __syncthreads();
    if (warp == 1 && tmem != 0xFFFFFFFFu) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------
// host
// ------------------------------------------------------------------------------------------
static int make_map(CUtensorMap* map, const void* base, int heads, int64_t tokens) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return fail(NVLLM_B200_EDRIVER, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)heads, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)kD * 2, (cuuint64_t)heads * kD * 2};
    cuuint32_t box[3] = {64, 1, 128};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(NVLLM_B200_EDRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return NVLLM_B200_OK;
}

static int ensure_attr() {
    static std::mutex mu;
    static bool done[64];
    int dev = 0;
    NVLLM_CUDA_OK(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64 && !done[dev]) {
        NVLLM_CUDA_OK(
            cudaFuncSetAttribute(varlen_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        done[dev] = true;
    }
    return NVLLM_B200_OK;
}

static int64_t item_capacity(int64_t T, int B) { return T / kTileQ + B + 1; }  // covers 128-row blocks

// Common launcher.  kv_tokens: extent of the token axis of k / v (T for packed tensors, the slot count of the cache).
static int launch(const char* who, const void* q, const void* k, const void* v, int64_t kv_tokens,
                  const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* block_tables, int MB,
                  int block_size, const int32_t* cu_seqlens_host, void* out, void* workspace, size_t workspace_bytes,
                  int64_t T, int B, int max_seqlen, int H, int KVH, int D, float scale, void* stream) {
    if (T < 0 || B < 0 || H <= 0 || KVH <= 0)
        return fail(NVLLM_B200_EINVAL, "%s: bad size (T=%lld B=%d H=%d KVH=%d)", who, (long long)T, B, H, KVH);
    if (D != kD) return fail(NVLLM_B200_EUNSUPPORTED, "%s: head_dim %d (only 128)", who, D);
    if (H % KVH != 0) return fail(NVLLM_B200_EUNSUPPORTED, "%s: H %d not a multiple of KVH %d", who, H, KVH);
    if (B > 65535) return fail(NVLLM_B200_EUNSUPPORTED, "%s: more than 65535 sequences", who);
    if (T > 0x7fffffffLL || kv_tokens > 0x7fffffffLL)
        return fail(NVLLM_B200_EUNSUPPORTED, "%s: more than 2^31-1 tokens", who);
    if (!(scale > 0.f)) return fail(NVLLM_B200_EINVAL, "%s: scale must be positive", who);
    if (T == 0 || B == 0) return NVLLM_B200_OK;
    if (!q || !k || !v || !cu_seqlens_q || !cu_seqlens_k || !out) return fail(NVLLM_B200_EINVAL, "%s: null pointer", who);
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out) & 15)
        return fail(NVLLM_B200_EINVAL, "%s: q/k/v/out must be 16-byte aligned", who);
    const size_t need = nvllm_b200_varlen_prefill_workspace_bytes(T, B, H, KVH, D);
    if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15))
        return fail(NVLLM_B200_EWORKSPACE, "%s: workspace of %zu bytes required, got %zu", who, need,
                    workspace ? workspace_bytes : (size_t)0);

    // Two q heads of one kv head make an item when there are such pairs: both Q tiles then see the same number of K/V
    // tiles and finish together.  Otherwise an item is 256 rows of one head.
    const int pair_heads = ((H / KVH) % 2 == 0) ? 1 : 0;
    const int bq = pair_heads ? kTileQ : kBlockQ;
    const int per_pair = pair_heads ? H / 2 : H;
    // Upper bound of (sequence, row block) pairs: exact from the host copy of cu_seqlens, else from max_seqlen.
    int64_t pairs = 0;
    const int64_t cap = item_capacity(T, B);
    if (cu_seqlens_host) {
        for (int b = 0; b < B; ++b) {
            const int64_t len = (int64_t)cu_seqlens_host[b + 1] - cu_seqlens_host[b];
            if (len < 0 || cu_seqlens_host[b + 1] > T)
                return fail(NVLLM_B200_EINVAL, "%s: cu_seqlens_host is not a non-decreasing prefix of T", who);
            if (len > (int64_t)kMaxLevels * bq)
                return fail(NVLLM_B200_EUNSUPPORTED, "%s: sequence of %lld tokens (max %d)", who, (long long)len,
                            kMaxLevels * bq);
            pairs += (len + bq - 1) / bq;
        }
    } else {
        if (max_seqlen <= 0) return fail(NVLLM_B200_EINVAL, "%s: max_seqlen must be positive", who);
        if (max_seqlen > kMaxLevels * bq)
            return fail(NVLLM_B200_EUNSUPPORTED, "%s: max_seqlen %d (max %d)", who, max_seqlen, kMaxLevels * bq);
        pairs = (int64_t)B * ((max_seqlen + bq - 1) / bq);
    }
    if (pairs > cap) pairs = cap;
    if (pairs == 0) return NVLLM_B200_OK;
    if (pairs * per_pair > 0x7fffffffLL) return fail(NVLLM_B200_EUNSUPPORTED, "%s: grid too large", who);

    int rc = ensure_attr();
    if (rc) return rc;
    CUtensorMap tm_q, tm_k, tm_v;
    if ((rc = make_map(&tm_q, q, H, T))) return rc;
    if ((rc = make_map(&tm_k, k, KVH, kv_tokens))) return rc;
    if ((rc = make_map(&tm_v, v, KVH, kv_tokens))) return rc;

    Params p;
    p.items = (const int4*)workspace;
    p.block_tables = block_tables;
    p.MB = MB;
    p.block_size = block_size;
    p.out = (__nv_bfloat16*)out;
    p.H = H;
    p.G = H / KVH;
    p.pair_heads = pair_heads;
    p.scale_log2 = scale * 1.4426950408889634f;

    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, prefill_plan_kernel, cu_seqlens_q, cu_seqlens_k, block_tables ? 1 : 0, B,
                                     (int4*)workspace, (int)cap, bq));
    const int64_t ctas = pairs * per_pair < (int64_t)sm_count() ? pairs * per_pair : (int64_t)sm_count();
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, varlen_prefill_kernel, tm_q, tm_k, tm_v, p));
    return NVLLM_B200_OK;
}

}  // namespace prefill

int read_prefill_flags(int* out) {
    NVLLM_CUDA_OK(cudaMemcpyFromSymbol(out, prefill::g_error_flag, sizeof(int)));
    return NVLLM_B200_OK;
}
int clear_prefill_flags() {
    const int zero = 0;
    NVLLM_CUDA_OK(cudaMemcpyToSymbol(prefill::g_error_flag, &zero, sizeof(int)));
    return NVLLM_B200_OK;
}
}  // namespace nvllm

extern "C" size_t nvllm_b200_varlen_prefill_workspace_bytes(int64_t T, int B, int H, int KVH, int D) {
    (void)H;
    (void)KVH;
    (void)D;
    if (T < 0 || B < 0) return 256;
    const size_t n = (size_t)(2 * nvllm::prefill::item_capacity(T, B) + 1) * 16;
    return (n + 255) & ~size_t(255);
}

extern "C" int nvllm_b200_varlen_prefill(const void* q, const void* k, const void* v, const int32_t* cu_seqlens_q,
                                         const int32_t* cu_seqlens_k, const int32_t* cu_seqlens_host, void* out,
                                         void* workspace, size_t workspace_bytes, int64_t T, int B, int max_seqlen,
                                         int H, int KVH, int D, float scale, void* stream) {
    // packed keys/values lie beside the queries (k, v are [T, KVH, 128] like q): cu_seqlens_k must equal
    // cu_seqlens_q, which the plan kernel checks on the device
    return nvllm::prefill::launch("varlen_prefill", q, k, v, T, cu_seqlens_q, cu_seqlens_k, nullptr, 0, 0,
                                  cu_seqlens_host, out, workspace, workspace_bytes, T, B, max_seqlen, H, KVH, D, scale,
                                  stream);
}

extern "C" int nvllm_b200_paged_prefill(const void* q, const void* k_cache, const void* v_cache,
                                        const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                        const int32_t* block_tables, const int32_t* cu_seqlens_q_host, void* out,
                                        void* workspace, size_t workspace_bytes, int64_t T, int B, int max_seqlen_q,
                                        int H, int KVH, int D, int NB, int block_size, int MB, float scale,
                                        void* stream) {
    using namespace nvllm;
    if (!block_tables || MB <= 0) return fail(NVLLM_B200_EINVAL, "paged_prefill: block_tables required");
    if (block_size <= 0 || block_size % prefill::kTileKV != 0)
        return fail(NVLLM_B200_EUNSUPPORTED, "paged_prefill: block_size %d (must be a multiple of %d)", block_size,
                    prefill::kTileKV);
    if (NB <= 0) return fail(NVLLM_B200_EINVAL, "paged_prefill: NB must be positive");
    return prefill::launch("paged_prefill", q, k_cache, v_cache, (int64_t)NB * block_size, cu_seqlens_q, cu_seqlens_k,
                           block_tables, MB, block_size, cu_seqlens_q_host, out, workspace, workspace_bytes, T, B,
                           max_seqlen_q, H, KVH, D, scale, stream);
}
