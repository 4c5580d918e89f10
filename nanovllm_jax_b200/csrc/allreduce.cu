// One-shot sum over the tensor-parallel ranks of one node for decode-size messages, over NVLink peer memory.
//
// Replaces the collective behind the row-parallel projections of the reference (RowParallelLinear.__call__,
// layers/linear.py:486-510: the sum over ranks after o_proj and down_proj, models/qwen3.py:170, 230) for messages of up
// to a megabyte or so -- 72 of them per decode step of a 36-layer model, each far too small for a ring to pay off.
// Optionally adds the residual stream in the same pass (x = x + sum, models/qwen3.py:225-231).
//
// Every rank owns one "symmetric" buffer (same layout on every rank, mapped into every other rank's address space
// through CUDA IPC):  flags[world][kCtas] u32, a control block (calls completed, CTAs finished), then two staging
// slots of max_bytes each.  One call with epoch e (given by the caller, or -- epoch 0 -- taken from the control
// block as "calls completed + 1", which every rank counts alike; only the latter survives CUDA-graph replay, where
// kernel parameters are frozen):
//   1. CTA c copies its chunks of the input into the rank's own staging slot e & 1;
//   2. it publishes them: system-scope fence, then flags[rank][c] = e written into EVERY peer's buffer;
//   3. it waits until its own flags[p][c] >= e for every peer p (a bounded spin on LOCAL memory);
//   4. it adds up the same chunks of all ranks' staging slots in rank order 0 .. world-1 (fp32 accumulation, so every
//      rank computes bit-identical sums), adds the residual if given, and writes bf16.
// Chunks are a fixed 8 KB and chunk i always belongs to CTA i % kCtas, on every rank and in every call, so "CTA c of
// every peer has signalled epoch e + 1" implies "they have finished reading my chunks of epoch e": two slots suffice.
//
// Plain peer loads and stores only: no multimem, no TMA from peer memory.  No wait is unbounded: when a peer's flag
// does not arrive within `max_spins` polls the CTA raises a device error flag (bit 6 of nvllm_b200_device_status),
// skips its reduction and returns; the context stays usable.
#include "common.cuh"

#include <string.h>

namespace nvllm {
namespace comm {

constexpr int kCtas = 64;          // CTAs per rank, fixed: the chunk -> CTA map must never change
constexpr int kThreads = 512;
// a chunk = kThreads 16-byte vectors = 8 KB
constexpr int kMaxWorld = 8;

__device__ int g_error_flag = 0;  // bit 6 (64): a peer's flag did not arrive in time

__host__ __device__ inline size_t flag_bytes() { return (size_t)kMaxWorld * kCtas * 4 + 256; }  // flags + control block
__host__ __device__ inline size_t ctrl_offset() { return (size_t)kMaxWorld * kCtas * 4; }

struct Params {
    // one entry per emulated rank (blockIdx.y); a real multi-GPU launch uses entry 0 only
    const uint4* in[kMaxWorld];
    uint4* out[kMaxWorld];
    const uint4* residual[kMaxWorld];
    uint8_t* bufs[kMaxWorld][kMaxWorld];  // bufs[y][p]: rank p's symmetric buffer as mapped for the rank in entry y
    int rank0;                            // rank of entry 0 (entry y is rank rank0 + y)
    int world;
    long long chunks;                     // ceil(bytes / kChunkBytes)
    long long vecs;                       // bytes / 16
    size_t max_bytes;
    unsigned int epoch;  // 0: use the device-side call counter of the rank's control block
    long long max_spins;
};

__device__ __forceinline__ void st_flag_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_flag_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ld_vec_sys(const uint4* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void add_bf16x8(float (&acc)[8], const uint4& w) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        acc[2 * i] += __uint_as_float(u[i] << 16);
        acc[2 * i + 1] += __uint_as_float(u[i] & 0xFFFF0000u);
    }
}

__global__ void __launch_bounds__(kThreads) allreduce_sum_kernel(const Params p) {
    __shared__ int s_ok;
    const int y = blockIdx.y, rank = p.rank0 + y, c = blockIdx.x, tid = threadIdx.x;
    uint8_t* mine = p.bufs[y][rank];
    unsigned int* ctrl = reinterpret_cast<unsigned int*>(mine + ctrl_offset());  // [0] calls completed, [1] CTAs finished
    griddep_wait();  // the input comes from the kernel just before this one (the row-parallel GEMM); so does ctrl[0]
    griddep_launch_dependents();
    // every CTA of the launch reads the same value: ctrl[0] only moves when the last CTA of a launch has finished
    const unsigned int epoch = p.epoch ? p.epoch : *reinterpret_cast<volatile unsigned int*>(ctrl) + 1u;
    const size_t slot_off = flag_bytes() + (size_t)(epoch & 1u) * p.max_bytes;
    if (tid == 0) s_ok = 1;
    // 1. my chunks -> my staging slot
    uint4* stage = reinterpret_cast<uint4*>(mine + slot_off);
    for (long long ch = c; ch < p.chunks; ch += kCtas) {
        const long long i = ch * kThreads + tid;
        if (i < p.vecs) stage[i] = p.in[y][i];
    }
    // 2. publish: every thread's stores are ordered before the flag stores by the barrier + system-scope fence
    __syncthreads();
    if (tid < p.world && tid != rank) {
        __threadfence_system();
        st_flag_sys(reinterpret_cast<unsigned int*>(p.bufs[y][tid]) + rank * kCtas + c, epoch);
    }
    // 3. wait for every peer's CTA c (bounded; the flags I poll live in my own memory)
    if (tid < p.world && tid != rank) {
        const unsigned int* f = reinterpret_cast<const unsigned int*>(mine) + tid * kCtas + c;
        long long spins = 0;
        while ((int)(ld_flag_sys(f) - epoch) < 0) {
            if (++spins > p.max_spins) {
                s_ok = 0;
                atomicOr(&g_error_flag, 64);
                break;
            }
        }
    }
    __syncthreads();
    // 4. sum in rank order (skipped when a peer never delivered)
    for (long long ch = c; s_ok && ch < p.chunks; ch += kCtas) {
        const long long i = ch * kThreads + tid;
        if (i >= p.vecs) continue;
        uint4 v[kMaxWorld];
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)
            if (r < p.world) v[r] = ld_vec_sys(reinterpret_cast<const uint4*>(p.bufs[y][r] + slot_off) + i);
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)
            if (r < p.world) add_bf16x8(acc, v[r]);
        if (p.residual[y]) add_bf16x8(acc, p.residual[y][i]);
        uint4 w;
        w.x = pack_bf16(acc[0], acc[1]);
        w.y = pack_bf16(acc[2], acc[3]);
        w.z = pack_bf16(acc[4], acc[5]);
        w.w = pack_bf16(acc[6], acc[7]);
        p.out[y][i] = w;
    }
    // 5. the last CTA of this rank's launch to get here advances the rank's call counter
    __syncthreads();
    if (tid == 0) {
        if (atomicAdd(ctrl + 1, 1u) == (unsigned int)kCtas - 1u) {
            ctrl[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned int*>(ctrl) = epoch;
        }
    }
}

}  // namespace comm

int read_comm_flags(int* out) {
    NVLLM_CUDA_OK(cudaMemcpyFromSymbol(out, comm::g_error_flag, sizeof(int)));
    return NVLLM_B200_OK;
}
int clear_comm_flags() {
    const int zero = 0;
    NVLLM_CUDA_OK(cudaMemcpyToSymbol(comm::g_error_flag, &zero, sizeof(int)));
    return NVLLM_B200_OK;
}
}  // namespace nvllm

extern "C" size_t nvllm_b200_comm_buffer_bytes(size_t max_bytes) {
    const size_t m = (max_bytes + 255) & ~size_t(255);
    return nvllm::comm::flag_bytes() + 2 * m;
}

extern "C" int nvllm_b200_comm_alloc(size_t max_bytes, void** buffer, void* ipc_handle_64) {
    using namespace nvllm;
    if (!buffer || !ipc_handle_64 || max_bytes == 0) return fail(NVLLM_B200_EINVAL, "comm_alloc: bad argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    void* p = nullptr;
    const size_t bytes = nvllm_b200_comm_buffer_bytes(max_bytes);
    NVLLM_CUDA_OK(cudaMalloc(&p, bytes));
    cudaError_t e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(ipc_handle_64), p);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(NVLLM_B200_ECUDA, "comm_alloc: %s", cudaGetErrorString(e));
    }
    *buffer = p;
    return NVLLM_B200_OK;
}

extern "C" int nvllm_b200_comm_open(const void* ipc_handle_64, void** buffer) {
    using namespace nvllm;
    if (!buffer || !ipc_handle_64) return fail(NVLLM_B200_EINVAL, "comm_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle_64, sizeof(h));
    NVLLM_CUDA_OK(cudaIpcOpenMemHandle(buffer, h, cudaIpcMemLazyEnablePeerAccess));
    return NVLLM_B200_OK;
}

extern "C" int nvllm_b200_comm_close(void* buffer) {
    using namespace nvllm;
    if (buffer) NVLLM_CUDA_OK(cudaIpcCloseMemHandle(buffer));
    return NVLLM_B200_OK;
}

extern "C" int nvllm_b200_comm_free(void* buffer) {
    using namespace nvllm;
    if (buffer) NVLLM_CUDA_OK(cudaFree(buffer));
    return NVLLM_B200_OK;
}

namespace nvllm {
namespace comm {
static int launch(const Params& p, int ranks_in_launch, bool cooperative, void* stream) {
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (cooperative) {
        // several ranks emulated on one device: their CTAs wait on one another, so all of them must be resident
        void* args[] = {const_cast<Params*>(&p)};
        NVLLM_CUDA_OK(cudaLaunchCooperativeKernel((const void*)allreduce_sum_kernel, dim3(kCtas, ranks_in_launch),
                                                  dim3(kThreads), args, 0, st));
        return NVLLM_B200_OK;
    }
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kCtas, ranks_in_launch);
    cfg.blockDim = dim3(kThreads);
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    NVLLM_CUDA_OK(cudaLaunchKernelEx(&cfg, allreduce_sum_kernel, p));
    return NVLLM_B200_OK;
}

static int check(const char* who, int world, int64_t count, size_t max_bytes, long long max_spins) {
    if (world < 1 || world > kMaxWorld) return fail(NVLLM_B200_EUNSUPPORTED, "%s: world size %d (1..%d)", who, world, kMaxWorld);
    if (count < 0 || count % 8 != 0) return fail(NVLLM_B200_EUNSUPPORTED, "%s: count %lld must be a multiple of 8", who, (long long)count);
    if ((size_t)count * 2 > max_bytes)
        return fail(NVLLM_B200_EWORKSPACE, "%s: %lld bytes exceed the buffers' %zu", who, (long long)count * 2, max_bytes);
    if (max_spins <= 0) return fail(NVLLM_B200_EINVAL, "%s: max_spins must be positive", who);
    return NVLLM_B200_OK;
}
}  // namespace comm
}  // namespace nvllm

extern "C" int nvllm_b200_allreduce_sum(const void* in, void* out, const void* residual, void* const* buffers_host,
                                        int rank, int world, int64_t count, size_t max_bytes, unsigned int epoch,
                                        int64_t max_spins, void* stream) {
    using namespace nvllm;
    using namespace nvllm::comm;
    int rc = check("allreduce_sum", world, count, max_bytes, max_spins);
    if (rc) return rc;
    if (rank < 0 || rank >= world) return fail(NVLLM_B200_EINVAL, "allreduce_sum: rank %d of %d", rank, world);
    if (count == 0) return NVLLM_B200_OK;
    if (!in || !out || !buffers_host) return fail(NVLLM_B200_EINVAL, "allreduce_sum: null pointer");
    if (((uintptr_t)in | (uintptr_t)out | (uintptr_t)residual) & 15)
        return fail(NVLLM_B200_EINVAL, "allreduce_sum: in/out/residual must be 16-byte aligned");
    Params p = {};
    p.in[0] = (const uint4*)in;
    p.out[0] = (uint4*)out;
    p.residual[0] = (const uint4*)residual;
    for (int r = 0; r < world; ++r) {
        if (!buffers_host[r]) return fail(NVLLM_B200_EINVAL, "allreduce_sum: buffer of rank %d missing", r);
        p.bufs[0][r] = (uint8_t*)buffers_host[r];
    }
    p.rank0 = rank;
    p.world = world;
    p.vecs = count / 8;
    p.chunks = (p.vecs + kThreads - 1) / kThreads;
    p.max_bytes = (max_bytes + 255) & ~size_t(255);
    p.epoch = epoch;
    p.max_spins = max_spins;
    return launch(p, 1, false, stream);
}

// All ranks of a world emulated on ONE device by one cooperative launch (grid.y = world): for tests on a single GPU.
// in / out / residual / buffers_host hold one pointer per rank; every "rank" sees the same mapping of the buffers.
extern "C" int nvllm_b200_allreduce_sum_emulated(void* const* in, void* const* out, void* const* residual,
                                                 void* const* buffers_host, int world, int64_t count, size_t max_bytes,
                                                 unsigned int epoch, int64_t max_spins, void* stream) {
    using namespace nvllm;
    using namespace nvllm::comm;
    int rc = check("allreduce_sum_emulated", world, count, max_bytes, max_spins);
    if (rc) return rc;
    if (count == 0) return NVLLM_B200_OK;
    if (!in || !out || !buffers_host) return fail(NVLLM_B200_EINVAL, "allreduce_sum_emulated: null pointer");
    Params p = {};
    for (int y = 0; y < world; ++y) {
        p.in[y] = (const uint4*)in[y];
        p.out[y] = (uint4*)out[y];
        p.residual[y] = residual ? (const uint4*)residual[y] : nullptr;
        for (int r = 0; r < world; ++r) p.bufs[y][r] = (uint8_t*)buffers_host[r];
    }
    p.rank0 = 0;
    p.world = world;
    p.vecs = count / 8;
    p.chunks = (p.vecs + kThreads - 1) / kThreads;
    p.max_bytes = (max_bytes + 255) & ~size_t(255);
    p.epoch = epoch;
    p.max_spins = max_spins;
    return launch(p, world, true, stream);
}
