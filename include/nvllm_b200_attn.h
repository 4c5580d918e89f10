/*
 * nvllm_b200_attn.h -- C ABI of the B200 (sm_100a) attention hot path.
 *
 * One shared library, libnvllm_b200_attn.so, replaces the device work behind
 * three call sites of nanovllm_jax (paths relative to the reference project):
 *
 *   store_kv_to_cache                    layers/attention.py:42-77
 *   paged_attention (decode)             layers/pallas_attention.py:465-507
 *                                        -> paged_decode_attention_vectorized :146-238
 *   variable_length_attention_prefill    layers/attention.py:135-279
 *   (also reached as paged_prefill_attention, layers/pallas_attention.py:557-608)
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer on the current CUDA device unless the
 *     parameter name ends in _host.  The caller owns every buffer.  Unless a
 *     function's comment says otherwise the library never allocates or frees
 *     device memory and never synchronises: each call only enqueues work on
 *     `stream` (a cudaStream_t passed as void*; NULL = the legacy default stream).
 *   - Tensors are dense row-major.  K/V caches, q, k, v and outputs are bf16
 *     (2 bytes); index tensors are int32.
 *   - Return value: 0 on success, a negative NVLLM_B200_E* code otherwise.
 *     Nothing throws or aborts.  nvllm_b200_last_error_string() returns a
 *     thread-local description of the most recent failure on this thread.
 *   - Supported set: head_dim == 128; block_size a multiple of 64 (the
 *     reference asserts a multiple of 256, config.py:38); num_heads a multiple
 *     of num_kv_heads with ratio <= 8 (decode) / any ratio (prefill); bf16.
 *     Anything else returns NVLLM_B200_EUNSUPPORTED -- there is no fallback path.
 *   - Thread safety: re-entrant; calls may come from any host thread; work is
 *     ordered by the stream it is enqueued on.
 */
#ifndef NVLLM_B200_ATTN_H_
#define NVLLM_B200_ATTN_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NVLLM_B200_OK            0
#define NVLLM_B200_EINVAL       -1  /* null pointer, negative size, misaligned pointer */
#define NVLLM_B200_EUNSUPPORTED -2  /* shape outside the supported set */
#define NVLLM_B200_EWORKSPACE   -3  /* workspace missing or too small */
#define NVLLM_B200_ECUDA        -4  /* a CUDA runtime call or kernel launch failed */
#define NVLLM_B200_EDRIVER      -5  /* cuTensorMapEncodeTiled unavailable / failed */

/* Element type of the k/v rows handed to nvllm_b200_store_kvcache. */
#define NVLLM_B200_DTYPE_BF16 0
#define NVLLM_B200_DTYPE_F32  1

/* Library version, major*10000 + minor*100 + patch. */
int nvllm_b200_version(void);

/* Thread-local text for the last non-zero return on this thread ("" if none). */
const char* nvllm_b200_last_error_string(void);

/*
 * store_kvcache: k_cache[slot_mapping[t]] = bf16(k[t]), v_cache[...] = bf16(v[t]).
 * Replaces store_kv_to_cache, layers/attention.py:42-77 (called at :465-467).
 *
 *   k, v          [T, KVH, D]            bf16 or f32 (src_dtype); f32 is rounded
 *                                        to nearest-even, as the reference's
 *                                        astype(cache dtype) at :70-71
 *   k_cache, v_cache [num_slots, KVH, D] bf16, updated in place (the reference
 *                                        donates them, :42)
 *   slot_mapping  [T] int32              flat slot = block * block_size + offset
 *
 * A slot < 0 is SKIPPED, which is what the reference documents (:57-58); the
 * reference code as written instead overwrites slot 0 (:64-67) -- its model
 * runner never emits a negative slot (engine/model_runner.py:300-309,361), so
 * the two never differ in practice.  A slot >= num_slots is dropped (:74-75).
 * Slots must be unique within a call (the block manager guarantees it).
 */
int nvllm_b200_store_kvcache(const void* k, const void* v, void* k_cache, void* v_cache,
                             const int32_t* slot_mapping, int64_t T, int KVH, int D,
                             int64_t num_slots, int src_dtype, void* stream);

/*
 * Bytes of scratch nvllm_b200_paged_decode / nvllm_b200_decode_step need for
 * these sizes (always > 0, a multiple of 256).  Depends on B, KVH, H/KVH and the
 * current device's SM count.
 */
size_t nvllm_b200_paged_decode_workspace_bytes(int B, int H, int KVH, int D, int MB, int block_size);

/*
 * paged_decode: out[b,h,:] = softmax(scale * q[b,h,:] . K_b^T) V_b over the
 * first context_lens[b] tokens of the pages block_tables[b,:], kv head = h / (H/KVH).
 * Replaces paged_attention, layers/pallas_attention.py:465-507 and its live body
 * paged_decode_attention_vectorized :146-238 (called from layers/attention.py:389-397).
 *
 *   q             [B, H, D] bf16
 *   k_cache, v_cache [NB, block_size, KVH, D] bf16
 *   block_tables  [B, MB] int32, -1 padded; ids are clamped to [0, NB-1] (:185)
 *                 and only the first ceil(ctx/block_size) entries of a row are read
 *   context_lens  [B] int32; clamped to [0, MB*block_size]; 0 gives a zero row
 *   out           [B, H, D] bf16
 *   workspace     >= nvllm_b200_paged_decode_workspace_bytes(...) bytes, 256-byte
 *                 aligned; contents need not be initialised and are not preserved
 *
 * Math: fp32 scores and softmax, bf16 probabilities into the P.V product with
 * fp32 accumulation; 1e-9 is added to the softmax denominator as in :227.
 * Tokens at positions >= context_lens[b] are never used, whatever bytes their
 * cache rows hold.
 */
int nvllm_b200_paged_decode(const void* q, const void* k_cache, const void* v_cache,
                            const int32_t* block_tables, const int32_t* context_lens, void* out,
                            void* workspace, size_t workspace_bytes,
                            int B, int H, int KVH, int D, int NB, int block_size, int MB,
                            float scale, void* stream);

/*
 * decode_step: what Attention.__call__ does for one layer in the decode phase
 * (layers/attention.py:436-480, decode branch): scatter the step's new K/V rows
 * into the cache by slot (store_kv_to_cache, :465-467), then attend over the
 * pages (_decode_attention, :366-397) -- one C call, two kernel launches.
 * Equivalent to nvllm_b200_store_kvcache(k, v, ..., T = B) followed by
 * nvllm_b200_paged_decode(...) on the same stream, with the same argument
 * meanings, limits and workspace size; k and v are [B, KVH, D] in src_dtype.
 */
int nvllm_b200_decode_step(const void* q, const void* k, const void* v, void* k_cache, void* v_cache,
                           const int32_t* slot_mapping, const int32_t* block_tables,
                           const int32_t* context_lens, void* out,
                           void* workspace, size_t workspace_bytes,
                           int B, int H, int KVH, int D, int NB, int block_size, int MB,
                           float scale, int src_dtype, void* stream);

/*
 * paged_decode_static: the same computation as nvllm_b200_paged_decode, for callers that can give the
 * library no scratch buffer and cannot allocate one themselves.  It has no counterpart in the reference.
 *
 * Who needs it: a host whose operand list is fixed (it can pass inputs and outputs, nothing else) and that
 * runs where device allocation is off limits at call time -- typically a framework custom-call handler
 * in a process whose memory pool already owns almost all of HBM, so that a cudaMalloc may fail or take
 * memory the pool counts on, or a latency-critical loop that must avoid the device-wide synchronisation
 * cudaMalloc and cudaFree cause.  This entry point calls no allocating routine: its split-K scratch is a
 * fixed array of about 2.8 MB inside the library image, present on every device that loads the library
 * for as long as the process lives.
 *
 * Limits (beyond those of nvllm_b200_paged_decode): B <= 4096 sequences and B * KVH <= 32768, and a
 * device with at most 160 SMs (the main kernel runs 2 CTAs per SM and the array holds the partial results of 320).  Larger
 * sizes return NVLLM_B200_EWORKSPACE and the error text names the limit; nothing is launched.
 *
 * The first call on each device looks up the array's device address (one cudaGetSymbolAddress with that
 * device current, which may also make the runtime load the library's device code); make that first call
 * outside any stream capture.  Later calls only enqueue kernels on `stream`.
 *
 * All calls on a device share the one array, and it keeps whatever the previous call left in it.  The
 * words that must start at zero (one arrival counter per sequence and kv head) are cleared by the call's
 * own first kernel, so there is nothing for the caller to clear between calls; but two calls whose
 * kernels may overlap on the GPU -- different streams, or different host threads without ordering -- race
 * on it and corrupt each other's results.  Issue them on one stream, or order them with events.
 */
int nvllm_b200_paged_decode_static(const void* q, const void* k_cache, const void* v_cache,
                                   const int32_t* block_tables, const int32_t* context_lens, void* out,
                                   int B, int H, int KVH, int D, int NB, int block_size, int MB,
                                   float scale, void* stream);

/*
 * Reads (and leaves set) the device-side error flags of the current device into
 * *flags_host.  0 = no kernel of this library ever gave up a bounded wait.
 * Bit 0 / 1: paged_decode producer / consumer timed out on a pipeline barrier.
 * Bit 2 (4): a prefill pipeline wait timed out.  Bit 4 (16): a sequence too long
 * for the prefill plan.  Bit 5 (32): prefill called with inconsistent
 * cu_seqlens_q / cu_seqlens_k (see nvllm_b200_varlen_prefill / _paged_prefill).
 * Bit 6 (64): an all-reduce gave up waiting for a peer's flag.
 * This call synchronises with the device (it copies one int back).
 */
int nvllm_b200_device_status(int* flags_host);

/* Bytes of scratch nvllm_b200_varlen_prefill needs (may be 0). */
size_t nvllm_b200_varlen_prefill_workspace_bytes(int64_t T, int B, int H, int KVH, int D);

/*
 * varlen_prefill: causal attention over B packed sequences,
 * out[t,h,:] = softmax_{s <= pos(t)}(scale * q[t,h,:] . k[s,h/(H/KVH),:]) v[s,...].
 * Replaces variable_length_attention_prefill, layers/attention.py:135-279
 * (via Attention._prefill_attention :331-364) and paged_prefill_attention,
 * layers/pallas_attention.py:557-608.
 *
 *   q             [T, H, D] bf16;  k, v [T, KVH, D] bf16;  out [T, H, D] bf16
 *   cu_seqlens_q, cu_seqlens_k  [B+1] int32 DEVICE arrays; they must be equal
 *                 element-wise (prompt without cached prefix -- the only case in
 *                 which the reference function is correct).  The device checks
 *                 it: if they differ nothing is computed and bit 5 (32) of the
 *                 device status is raised -- a prompt with a cached prefix goes
 *                 to nvllm_b200_paged_prefill.  cu_seqlens_host, if
 *                 not NULL, is a host copy of cu_seqlens_q that lets the library
 *                 size its grid without reading device memory
 *   max_seqlen    upper bound of any sequence length (used for grid sizing when
 *                 cu_seqlens_host is NULL)
 *
 * Unlike the reference, rows beyond the 8192-token bucket (utils/context.py:18-32)
 * are computed rather than returned as zeros.  Rows of `out` at token indices
 * >= cu_seqlens_q[B] belong to no sequence and are left untouched.
 */
int nvllm_b200_varlen_prefill(const void* q, const void* k, const void* v,
                              const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                              const int32_t* cu_seqlens_host, void* out,
                              void* workspace, size_t workspace_bytes,
                              int64_t T, int B, int max_seqlen, int H, int KVH, int D,
                              float scale, void* stream);

/*
 * paged_prefill: causal attention of the new tokens of B sequences over ALL their
 * tokens, cached prefix included, with keys/values read from the paged cache:
 * query i of sequence b sits at position prefix_b + i, prefix_b = len_k - len_q,
 * and attends positions 0 .. prefix_b + i of the pages block_tables[b, :].
 *
 * This is the prefill the reference's metadata asks for on a prefix-cache hit and
 * its attention code does not deliver: engine/model_runner.py:286-292 emits
 * cu_seqlens_k > cu_seqlens_q and :311-314 attaches block_tables, but
 * Attention._prefill_attention (layers/attention.py:351-364) drops the tables and
 * attends the new tokens only.  It replaces that branch, and it is what makes the
 * block manager's prefix cache (engine/block_manager.py:137-182) usable.  With
 * cu_seqlens_k == cu_seqlens_q it computes what nvllm_b200_varlen_prefill does.
 *
 *   q, out        [T, H, D] bf16, new tokens packed by cu_seqlens_q
 *   k_cache, v_cache [NB, block_size, KVH, D] bf16; the step's new K/V rows must
 *                 already be stored (Attention.__call__ stores before it attends,
 *                 layers/attention.py:465-467); block_size a multiple of 128
 *   cu_seqlens_q, cu_seqlens_k [B+1] int32 device arrays (only the differences of
 *                 cu_seqlens_k are used: the key count of each sequence);
 *                 len_k >= len_q for every sequence, else nothing is computed and
 *                 bit 5 (32) of the device status is raised
 *   block_tables  [B, MB] int32, -1 padded
 *   cu_seqlens_q_host  optional host copy of cu_seqlens_q (exact grid sizing)
 *   workspace     >= nvllm_b200_varlen_prefill_workspace_bytes(T, B, H, KVH, D)
 *
 * Cache rows at positions >= len_k are never used, whatever they hold.
 */
int nvllm_b200_paged_prefill(const void* q, const void* k_cache, const void* v_cache,
                             const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                             const int32_t* block_tables, const int32_t* cu_seqlens_q_host, void* out,
                             void* workspace, size_t workspace_bytes,
                             int64_t T, int B, int max_seqlen_q, int H, int KVH, int D,
                             int NB, int block_size, int MB, float scale, void* stream);

/*
 * qk_norm_rope_store: the step a Qwen3 layer runs between its QKV projection and
 * attention, fused into one pass over q, k, v (models/qwen3.py:157-166):
 *     q = q_norm(q); k = k_norm(k)          layers/layernorm.py:31-48 (RMSNorm over head_dim)
 *     q, k = rotary_emb(positions, q, k)    layers/rotary_embedding.py:13-37, 97-104
 *     store_kv_to_cache(k, v, ...)          layers/attention.py:42-77 (called at :465-467)
 * q and k are updated IN PLACE; the rotated k rows and the v rows are also written to
 * their cache slots (same slot rules as nvllm_b200_store_kvcache).
 *
 *   q [T, H, D], k [T, KVH, D], v [T, KVH, D]  bf16
 *   q_weight, k_weight  [D] fp32 (the RMSNorm scales); eps as layers/layernorm.py:27
 *   cos_sin_cache  [max_pos, D] fp32: cos (D/2) | sin (D/2) per position, the table of
 *                  layers/rotary_embedding.py:57-75; positions [T] int32, clamped to
 *                  [0, max_pos - 1]
 *
 * Arithmetic: RMSNorm in fp32, rounded to bf16 (the norm returns its input dtype, :47);
 * rotation in fp32 with separate multiplies and adds, rounded to bf16.  The sum of
 * squares is taken in one fixed order (documented in csrc/pre_attention.cuh), so a host
 * restatement reproduces every bf16 bit.
 */
int nvllm_b200_qk_norm_rope_store(void* q, void* k, const void* v, const float* q_weight, const float* k_weight,
                                  const float* cos_sin_cache, const int32_t* positions, void* k_cache, void* v_cache,
                                  const int32_t* slot_mapping, int64_t T, int H, int KVH, int D,
                                  int64_t num_slots, int64_t max_pos, float eps, void* stream);

/*
 * fused_decode_step: nvllm_b200_qk_norm_rope_store (T = B) followed by
 * nvllm_b200_paged_decode, in one C call and two kernel launches: everything a Qwen3
 * layer does between its QKV projection and its output projection in the decode phase
 * (models/qwen3.py:157-166 with layers/attention.py:436-480).  Argument meanings,
 * limits and workspace size are those of the two functions; q is rotated in place and
 * `out` receives the attention result.
 */
int nvllm_b200_fused_decode_step(void* q, void* k, const void* v, const float* q_weight, const float* k_weight,
                                 const float* cos_sin_cache, const int32_t* positions, int64_t max_pos, float eps,
                                 void* k_cache, void* v_cache, const int32_t* slot_mapping,
                                 const int32_t* block_tables, const int32_t* context_lens, void* out,
                                 void* workspace, size_t workspace_bytes,
                                 int B, int H, int KVH, int D, int NB, int block_size, int MB,
                                 float scale, void* stream);

/*
 * One-shot all-reduce (sum) over the tensor-parallel ranks of ONE node for decode-size bf16 messages, through
 * NVLink peer memory.  Replaces the collective behind the reference's row-parallel projections
 * (RowParallelLinear.__call__, layers/linear.py:486-510; o_proj models/qwen3.py:170, down_proj :230), optionally
 * fused with the residual add that follows it (models/qwen3.py:225-231).
 *
 * Set-up (these three DO allocate / map device memory; call them once, outside the serving loop):
 *   comm_alloc   allocates this rank's symmetric buffer (nvllm_b200_comm_buffer_bytes(max_bytes) bytes, zeroed) and
 *                returns its 64-byte CUDA IPC handle, to be sent to the other ranks by any means;
 *   comm_open    maps a peer's buffer from its handle; comm_close unmaps it; comm_free frees one's own.
 * allreduce_sum: out = sum over ranks of in (+ residual), `count` bf16 elements (a multiple of 8, count*2 <= max_bytes).
 *   buffers_host  HOST array of `world` device pointers: entry r = rank r's buffer as mapped in this process
 *   epoch         0: the kernel numbers the calls itself (a counter in the rank's buffer, advanced by every call;
 *                 all ranks count alike because they issue the same calls) -- the mode to use under CUDA-graph
 *                 capture, where kernel parameters are frozen; or 1, 2, 3, ...: the caller numbers the calls, the
 *                 same value on every rank for the same call, increasing by one per call.  One communicator uses
 *                 one mode throughout
 *   max_spins     bound of the wait for the peers' flags; when it runs out the call's kernel raises bit 6 (64) of
 *                 nvllm_b200_device_status, leaves `out` unwritten for the affected parts and returns
 * in, out and residual may alias one another.  Results are bit-identical on every rank (fixed summation order).
 * Every rank must issue the same sequence of calls; calls of one communicator must not overlap on the GPU.
 * allreduce_sum_emulated runs all ranks of a world on ONE device in one cooperative launch (single-GPU tests).
 */
size_t nvllm_b200_comm_buffer_bytes(size_t max_bytes);
int nvllm_b200_comm_alloc(size_t max_bytes, void** buffer, void* ipc_handle_64);
int nvllm_b200_comm_open(const void* ipc_handle_64, void** buffer);
int nvllm_b200_comm_close(void* buffer);
int nvllm_b200_comm_free(void* buffer);
int nvllm_b200_allreduce_sum(const void* in, void* out, const void* residual, void* const* buffers_host,
                             int rank, int world, int64_t count, size_t max_bytes, unsigned int epoch,
                             int64_t max_spins, void* stream);
int nvllm_b200_allreduce_sum_emulated(void* const* in, void* const* out, void* const* residual,
                                      void* const* buffers_host, int world, int64_t count, size_t max_bytes,
                                      unsigned int epoch, int64_t max_spins, void* stream);

/*
 * Clears the device-side error flags of the current device (see
 * nvllm_b200_device_status).  A host that has read and handled a non-zero status
 * calls this before it goes on.  Synchronises with the device.
 */
int nvllm_b200_device_status_reset(void);

#ifdef __cplusplus
}
#endif
#endif /* NVLLM_B200_ATTN_H_ */
