// XLA FFI adapter: custom-call handlers that forward XLA buffers to the C ABI of libnvllm_b200_attn.so.
//
// NOT compiled by the package's default build (it needs the XLA FFI headers that ship with jaxlib):
//   nanovllm_jax_b200.jax_ffi.build_ffi_adapter() compiles it against jax.ffi.include_dir() when JAX is installed.
// Written against the public XLA FFI API; never executed in the image this library was developed in (no JAX there).
//
// Each handler takes the stream from XLA, receives its scratch as an extra result buffer (allocated by XLA, so the
// handler itself never allocates) and only enqueues work.
#include <cuda_runtime_api.h>

#include "xla/ffi/api/ffi.h"
#include "nvllm_b200_attn.h"
namespace ffi = xla::ffi;

static ffi::Error Status(int rc) {
  return rc == 0 ? ffi::Error::Success()
                 : ffi::Error(ffi::ErrorCode::kInvalidArgument, nvllm_b200_last_error_string());
}

// store: k_cache/v_cache are aliased to the two results (input_output_aliases on the Python side), mirroring
// donate_argnums=(2, 3) at layers/attention.py:42.
static ffi::Error StoreImpl(cudaStream_t stream, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer k_cache,
                            ffi::AnyBuffer v_cache, ffi::Buffer<ffi::S32> slots,
                            ffi::Result<ffi::AnyBuffer> k_out, ffi::Result<ffi::AnyBuffer> v_out) {
  auto d = k.dimensions();            // [T, KVH, D]
  auto c = k_cache.dimensions();      // [num_slots, KVH, D]
  int dtype = k.element_type() == ffi::F32 ? NVLLM_B200_DTYPE_F32 : NVLLM_B200_DTYPE_BF16;
  return Status(nvllm_b200_store_kvcache(k.untyped_data(), v.untyped_data(), k_out->untyped_data(),
                                         v_out->untyped_data(), slots.typed_data(), d[0], d[1], d[2], c[0], dtype,
                                         stream));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(NvllmStore, StoreImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::S32>>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>());

static ffi::Error DecodeImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k_cache, ffi::AnyBuffer v_cache,
                             ffi::Buffer<ffi::S32> tables, ffi::Buffer<ffi::S32> ctx, float scale,
                             ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::Buffer<ffi::U8>> scratch) {
  auto qd = q.dimensions();           // [B, H, D]
  auto cd = k_cache.dimensions();     // [NB, block, KVH, D]
  auto td = tables.dimensions();      // [B, MB]
  return Status(nvllm_b200_paged_decode(q.untyped_data(), k_cache.untyped_data(), v_cache.untyped_data(),
                                        tables.typed_data(), ctx.typed_data(), out->untyped_data(),
                                        scratch->typed_data(), scratch->size_bytes(), qd[0], qd[1], cd[2], qd[2], cd[0],
                                        cd[1], td[1], scale, stream));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(NvllmDecode, DecodeImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>().Attr<float>("scale")
        .Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::U8>>());

static ffi::Error PrefillImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                              ffi::Buffer<ffi::S32> cu_q, ffi::Buffer<ffi::S32> cu_k, float scale, int32_t max_seqlen,
                              ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::Buffer<ffi::U8>> scratch) {
  auto qd = q.dimensions();           // [T, H, D]
  auto kd = k.dimensions();           // [T, KVH, D]
  return Status(nvllm_b200_varlen_prefill(q.untyped_data(), k.untyped_data(), v.untyped_data(), cu_q.typed_data(),
                                          cu_k.typed_data(), /*cu_seqlens_host=*/nullptr, out->untyped_data(),
                                          scratch->typed_data(), scratch->size_bytes(), qd[0],
                                          cu_q.dimensions()[0] - 1, max_seqlen, qd[1], kd[1], qd[2], scale, stream));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(NvllmPrefill, PrefillImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>().Attr<float>("scale")
        .Attr<int32_t>("max_seqlen").Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::U8>>());

// Prefill over a cached prefix: keys/values come from the paged cache through block_tables (nvllm_b200_paged_prefill).
static ffi::Error PagedPrefillImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k_cache, ffi::AnyBuffer v_cache,
                                   ffi::Buffer<ffi::S32> cu_q, ffi::Buffer<ffi::S32> cu_k, ffi::Buffer<ffi::S32> tables,
                                   float scale, int32_t max_seqlen, ffi::Result<ffi::AnyBuffer> out,
                                   ffi::Result<ffi::Buffer<ffi::U8>> scratch) {
  auto qd = q.dimensions();           // [T, H, D]
  auto cd = k_cache.dimensions();     // [NB, block, KVH, D]
  auto td = tables.dimensions();      // [B, MB]
  return Status(nvllm_b200_paged_prefill(q.untyped_data(), k_cache.untyped_data(), v_cache.untyped_data(),
                                         cu_q.typed_data(), cu_k.typed_data(), tables.typed_data(),
                                         /*cu_seqlens_q_host=*/nullptr, out->untyped_data(), scratch->typed_data(),
                                         scratch->size_bytes(), qd[0], cu_q.dimensions()[0] - 1, max_seqlen, qd[1], cd[2],
                                         qd[2], cd[0], cd[1], td[1], scale, stream));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(NvllmPagedPrefill, PagedPrefillImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
        .Attr<float>("scale").Attr<int32_t>("max_seqlen").Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::U8>>());

// ---- caches addressed by pointer (side-effecting calls; the caches are not XLA operands) ----------------------------
// The cache addresses arrive as 64-bit attributes: the buffers are owned by the model runner, allocated once, and
// never appear among the operands of the jitted step, so XLA can neither copy nor move them.
static ffi::Error StoreInPlaceImpl(cudaStream_t stream, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::Buffer<ffi::S32> slots,
                                   int64_t k_cache, int64_t v_cache, int64_t num_slots,
                                   ffi::Result<ffi::Buffer<ffi::S32>> token) {
  (void)token;  // a one-word result the caller threads into the attention call to keep the order store -> attend
  auto d = k.dimensions();            // [T, KVH, D]
  int dtype = k.element_type() == ffi::F32 ? NVLLM_B200_DTYPE_F32 : NVLLM_B200_DTYPE_BF16;
  return Status(nvllm_b200_store_kvcache(k.untyped_data(), v.untyped_data(), reinterpret_cast<void*>(k_cache),
                                         reinterpret_cast<void*>(v_cache), slots.typed_data(), d[0], d[1], d[2], num_slots,
                                         dtype, stream));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(NvllmStoreInPlace, StoreInPlaceImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::Buffer<ffi::S32>>().Attr<int64_t>("k_cache").Attr<int64_t>("v_cache").Attr<int64_t>("num_slots")
        .Ret<ffi::Buffer<ffi::S32>>());

static ffi::Error DecodeStepInPlaceImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                                        ffi::Buffer<ffi::S32> slots, ffi::Buffer<ffi::S32> tables, ffi::Buffer<ffi::S32> ctx,
                                        int64_t k_cache, int64_t v_cache, int32_t num_blocks, int32_t block_size,
                                        float scale, ffi::Result<ffi::AnyBuffer> out,
                                        ffi::Result<ffi::Buffer<ffi::U8>> scratch) {
  auto qd = q.dimensions();           // [B, H, D]
  auto kd = k.dimensions();           // [B, KVH, D]
  auto td = tables.dimensions();      // [B, MB]
  int dtype = k.element_type() == ffi::F32 ? NVLLM_B200_DTYPE_F32 : NVLLM_B200_DTYPE_BF16;
  return Status(nvllm_b200_decode_step(q.untyped_data(), k.untyped_data(), v.untyped_data(),
                                       reinterpret_cast<void*>(k_cache), reinterpret_cast<void*>(v_cache),
                                       slots.typed_data(), tables.typed_data(), ctx.typed_data(), out->untyped_data(),
                                       scratch->typed_data(), scratch->size_bytes(), qd[0], qd[1], kd[1], qd[2],
                                       num_blocks, block_size, td[1], scale, dtype, stream));
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(NvllmDecodeStepInPlace, DecodeStepInPlaceImpl,
    ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>().Arg<ffi::Buffer<ffi::S32>>()
        .Attr<int64_t>("k_cache").Attr<int64_t>("v_cache").Attr<int32_t>("num_blocks").Attr<int32_t>("block_size")
        .Attr<float>("scale").Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::U8>>());
