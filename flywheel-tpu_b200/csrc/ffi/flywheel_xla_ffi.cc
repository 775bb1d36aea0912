// XLA FFI handlers over the C ABI of include/flywheel_b200.h: what a JAX host
// registers as custom-call targets for platform "CUDA" in place of the
// reference's Pallas calls.
//
//   handler symbol             C entry point        reference call site it replaces
//   fw_decode_kvcache_ffi      fw_decode_kvcache    kernels/decode.py:2424-2448 (pl.pallas_call of the decode kernel)
//   fw_append_ragged_ffi       fw_append_ragged     kernels/kv_append.py:116-184
//   fw_write_kv_pages_ffi      fw_write_kv_pages    kernels/kv_cache_write.py:66-227
//   fw_prefill_paged_ffi       fw_prefill_paged     kernels/fwd_paged.py:1351-1491
//   fw_lse_combine_ffi         fw_lse_combine       patches/tpu-inference.patch:7174-7186 (_merge_states)
// (paths relative to the heavyball-research/flywheel-tpu project).
//
// Conventions shared by all handlers
//  * Every operand the reference allows to be traced (lengths, tables, descales,
//    sinks, num_active) is a device buffer and is handed to the kernels as a
//    pointer: one executable serves changing values.
//  * XLA FFI has no optional operands.  An absent operand is passed as an array
//    with zero elements; the handler turns it into NULL.
//  * The cache operand is aliased to the cache result by the caller
//    (input_output_aliases), so only the appended rows are written.
//  * Scratch memory is an extra u8 result buffer sized at trace time with the
//    matching fw_*_workspace_bytes call; XLA owns it, the handler never
//    allocates.  XLA does not zero result buffers and the first 256 bytes of a
//    workspace are the library's status block, which must start at zero: each
//    handler clears them on the stream before its launch (a memset node, still
//    capturable).
//  * Handlers enqueue on the stream XLA passes and return; they are declared
//    command-buffer compatible.
//  * Error mapping: FW_ERR_LAUNCH / FW_ERR_TIMEOUT -> kInternal, everything else
//    -> kInvalidArgument, with fw_last_error() as the message.
//
// This file needs jaxlib's header-only xla/ffi/api/ffi.h.  build.py compiles it
// into lib/libflywheel_b200_ffi.so only where `jax.ffi.include_dir()` resolves;
// nothing else in the library depends on it.
#include <cuda_runtime.h>

#include <cstdint>

#include "flywheel_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error to_error(int rc) {
  if (rc == FW_OK) return ffi::Error::Success();
  const bool internal = rc == FW_ERR_LAUNCH || rc == FW_ERR_TIMEOUT;
  return ffi::Error(internal ? ffi::ErrorCode::kInternal : ffi::ErrorCode::kInvalidArgument, fw_last_error());
}

// NULL for an absent (zero-element) operand.
template <typename BufferT>
void* data_or_null(BufferT& buffer) {
  return buffer.element_count() == 0 ? nullptr : buffer.untyped_data();
}

int kv_dtype_of(ffi::DataType type) {
  switch (type) {
    case ffi::DataType::BF16: return FW_DTYPE_BF16;
    case ffi::DataType::F8E4M3FN: return FW_DTYPE_E4M3;
    case ffi::DataType::F8E5M2: return FW_DTYPE_E5M2;
    default: return -1;  // refused by the library with FW_ERR_BAD_DTYPE
  }
}

ffi::Error clear_status_block(ffi::AnyBuffer& workspace, cudaStream_t stream) {
  if (workspace.size_bytes() < 256) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "workspace is smaller than its status block");
  if (cudaMemsetAsync(workspace.untyped_data(), 0, 256, stream) != cudaSuccess)
    return ffi::Error(ffi::ErrorCode::kInternal, "clearing the workspace status block failed");
  return ffi::Error::Success();
}

// ---------------------------------------------------------------- decode
// Operands: q (batch, seqlen_q, nheads, d) bf16; kv_cache: the merged pool
// (pages, page_size, cache_heads, d) or, with has_block_table = 0, k_cache of the
// contiguous pair; v_cache (contiguous pair only, else empty); k_new / v_new
// (batch, seqlen_q, nheads_k, d) or empty; cache_seqlens i32[batch]; block_table
// i32[batch, pages_per_seq] or empty; cache_batch_idx, num_active, k_descale,
// v_descale, sinks: as in FwDecodeArgs, or empty.
// Results: out, lse (f32[batch, nheads, seqlen_q] or empty), kv_cache_out
// (aliased to kv_cache), v_cache_out (aliased to v_cache, or empty), workspace.
ffi::Error DecodeImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer kv_cache, ffi::AnyBuffer v_cache,
                      ffi::AnyBuffer k_new, ffi::AnyBuffer v_new, ffi::AnyBuffer cache_seqlens,
                      ffi::AnyBuffer block_table, ffi::AnyBuffer cache_batch_idx, ffi::AnyBuffer num_active,
                      ffi::AnyBuffer k_descale, ffi::AnyBuffer v_descale, ffi::AnyBuffer sinks,
                      ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> lse,
                      ffi::Result<ffi::AnyBuffer> kv_cache_out, ffi::Result<ffi::AnyBuffer> v_cache_out,
                      ffi::Result<ffi::AnyBuffer> workspace, int32_t nheads_k, int32_t causal, int32_t window_left,
                      float softmax_scale, float softcap) {
  const auto qd = q.dimensions();
  const auto cd = kv_cache.dimensions();
  if (qd.size() != 4 || cd.size() != 4)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "q and the cache must be rank-4 arrays");
  const bool paged = block_table.element_count() != 0;
  FwDecodeArgs a = {};
  a.q = q.untyped_data();
  a.out = out->untyped_data();
  a.lse = static_cast<float*>(data_or_null(*lse));
  a.kv_cache = kv_cache_out->untyped_data();  // the same memory as kv_cache: the caller aliases them
  a.v_cache = paged ? nullptr : v_cache_out->untyped_data();
  a.k_new = data_or_null(k_new);
  a.v_new = data_or_null(v_new);
  a.cache_seqlens = static_cast<const int32_t*>(cache_seqlens.untyped_data());
  a.block_table = static_cast<const int32_t*>(data_or_null(block_table));
  a.cache_batch_idx = static_cast<const int32_t*>(data_or_null(cache_batch_idx));
  a.num_active = static_cast<const int32_t*>(data_or_null(num_active));
  a.k_descale = static_cast<const float*>(data_or_null(k_descale));
  a.v_descale = static_cast<const float*>(data_or_null(v_descale));
  a.sinks = static_cast<const float*>(data_or_null(sinks));
  a.workspace = workspace->untyped_data();
  a.workspace_bytes = workspace->size_bytes();
  a.num_pages = cd[0];
  a.page_size = static_cast<int32_t>(cd[1]);
  a.pages_per_seq = paged ? static_cast<int32_t>(block_table.dimensions()[1]) : 1;
  a.batch = static_cast<int32_t>(qd[0]);
  a.seqlen_q = static_cast<int32_t>(qd[1]);
  a.nheads = static_cast<int32_t>(qd[2]);
  a.nheads_k = nheads_k;
  a.head_dim = static_cast<int32_t>(qd[3]);
  a.kv_dtype = kv_dtype_of(kv_cache.element_type());
  a.causal = causal;
  a.window_left = window_left;
  a.softmax_scale = softmax_scale;
  a.softcap = softcap;
  if (ffi::Error err = clear_status_block(*workspace, stream); err.failure()) return err;
  return to_error(fw_decode_kvcache(&a, stream));
}

// ---------------------------------------------------------------- ragged append
// Operands: kv_cache pool; k_new / v_new (total_tokens, nheads_k, d) in the pool
// dtype; cu_seqlens_q i32[batch + 1]; cache_seqlens i32[batch]; block_table
// i32[batch, pages_per_seq]; num_active i32[1] or empty.
// Result: kv_cache_out (aliased to kv_cache).
ffi::Error AppendImpl(cudaStream_t stream, ffi::AnyBuffer kv_cache, ffi::AnyBuffer k_new, ffi::AnyBuffer v_new,
                      ffi::AnyBuffer cu_seqlens_q, ffi::AnyBuffer cache_seqlens, ffi::AnyBuffer block_table,
                      ffi::AnyBuffer num_active, ffi::Result<ffi::AnyBuffer> kv_cache_out) {
  const auto cd = kv_cache.dimensions();
  const auto kd = k_new.dimensions();
  if (cd.size() != 4 || kd.size() != 3 || block_table.dimensions().size() != 2)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pool must be rank 4, k / v rank 3, block_table rank 2");
  FwAppendArgs a = {};
  a.kv_cache = kv_cache_out->untyped_data();
  a.k_new = k_new.untyped_data();
  a.v_new = v_new.untyped_data();
  a.cu_seqlens_q = static_cast<const int32_t*>(cu_seqlens_q.untyped_data());
  a.cache_seqlens = static_cast<const int32_t*>(cache_seqlens.untyped_data());
  a.block_table = static_cast<const int32_t*>(block_table.untyped_data());
  a.num_active = static_cast<const int32_t*>(data_or_null(num_active));
  a.num_pages = cd[0];
  a.page_size = static_cast<int32_t>(cd[1]);
  a.pages_per_seq = static_cast<int32_t>(block_table.dimensions()[1]);
  a.batch = static_cast<int32_t>(cache_seqlens.element_count());
  a.total_tokens = static_cast<int32_t>(kd[0]);
  a.nheads_k = static_cast<int32_t>(kd[1]);
  a.head_dim = static_cast<int32_t>(kd[2]);
  a.kv_dtype = kv_dtype_of(kv_cache.element_type());
  return to_error(fw_append_ragged(&a, stream));
}

// ---------------------------------------------------------------- slice-table page writer
// Operands: kv_cache pool; k_new / v_new (total_tokens, nheads_k, d); slices
// i32[3, num_columns]; num_slices i32[1].  Result: kv_cache_out (aliased).
ffi::Error WritePagesImpl(cudaStream_t stream, ffi::AnyBuffer kv_cache, ffi::AnyBuffer k_new, ffi::AnyBuffer v_new,
                          ffi::AnyBuffer slices, ffi::AnyBuffer num_slices,
                          ffi::Result<ffi::AnyBuffer> kv_cache_out) {
  const auto cd = kv_cache.dimensions();
  const auto kd = k_new.dimensions();
  if (cd.size() != 4 || kd.size() != 3 || slices.dimensions().size() != 2)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "pool must be rank 4, k / v rank 3, slices rank 2");
  FwWritePagesArgs a = {};
  a.kv_cache = kv_cache_out->untyped_data();
  a.k_new = k_new.untyped_data();
  a.v_new = v_new.untyped_data();
  a.slices = static_cast<const int32_t*>(slices.untyped_data());
  a.num_slices = static_cast<const int32_t*>(num_slices.untyped_data());
  a.num_pages = cd[0];
  a.page_size = static_cast<int32_t>(cd[1]);
  a.num_columns = static_cast<int32_t>(slices.dimensions()[1]);
  a.total_tokens = static_cast<int32_t>(kd[0]);
  a.nheads_k = static_cast<int32_t>(kd[1]);
  a.head_dim = static_cast<int32_t>(kd[2]);
  a.kv_dtype = kv_dtype_of(kv_cache.element_type());
  return to_error(fw_write_kv_pages(&a, stream));
}

// ---------------------------------------------------------------- chunked prefill
// Operands: q head-major (nheads, total_q, d) bf16 (token_major = 1: (total_q,
// nheads, d)); kv_cache pool (read only); cu_seqlens_q i32[batch + 1]; seqused_k
// i32[batch]; block_table i32[batch, pages_per_seq]; num_active, k_descale,
// v_descale, sinks, rotary_cos, rotary_sin: as in FwPrefillArgs, or empty.
// Results: out like q; lse f32[nheads, total_q] or empty; workspace.
ffi::Error PrefillImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer kv_cache, ffi::AnyBuffer cu_seqlens_q,
                       ffi::AnyBuffer seqused_k, ffi::AnyBuffer block_table, ffi::AnyBuffer num_active,
                       ffi::AnyBuffer k_descale, ffi::AnyBuffer v_descale, ffi::AnyBuffer sinks,
                       ffi::AnyBuffer rotary_cos, ffi::AnyBuffer rotary_sin, ffi::Result<ffi::AnyBuffer> out,
                       ffi::Result<ffi::AnyBuffer> lse, ffi::Result<ffi::AnyBuffer> workspace, int32_t nheads_k,
                       int32_t max_seqlen_q, int32_t causal, int32_t window_left, int32_t token_major,
                       int32_t rotary_interleaved, float softmax_scale, float softcap) {
  const auto qd = q.dimensions();
  const auto cd = kv_cache.dimensions();
  if (qd.size() != 3 || cd.size() != 4 || block_table.dimensions().size() != 2)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "q must be rank 3, the pool rank 4, block_table rank 2");
  FwPrefillArgs a = {};
  a.q = q.untyped_data();
  a.out = out->untyped_data();
  a.lse = static_cast<float*>(data_or_null(*lse));
  a.kv_cache = kv_cache.untyped_data();
  a.cu_seqlens_q = static_cast<const int32_t*>(cu_seqlens_q.untyped_data());
  a.seqused_k = static_cast<const int32_t*>(seqused_k.untyped_data());
  a.block_table = static_cast<const int32_t*>(block_table.untyped_data());
  a.num_active = static_cast<const int32_t*>(data_or_null(num_active));
  a.k_descale = static_cast<const float*>(data_or_null(k_descale));
  a.v_descale = static_cast<const float*>(data_or_null(v_descale));
  a.sinks = static_cast<const float*>(data_or_null(sinks));
  a.workspace = workspace->untyped_data();
  a.workspace_bytes = workspace->size_bytes();
  a.num_pages = cd[0];
  a.page_size = static_cast<int32_t>(cd[1]);
  a.pages_per_seq = static_cast<int32_t>(block_table.dimensions()[1]);
  a.batch = static_cast<int32_t>(seqused_k.element_count());
  a.total_q = static_cast<int32_t>(token_major ? qd[0] : qd[1]);
  a.max_seqlen_q = max_seqlen_q;
  a.nheads = static_cast<int32_t>(token_major ? qd[1] : qd[0]);
  a.nheads_k = nheads_k;
  a.head_dim = static_cast<int32_t>(qd[2]);
  a.kv_dtype = kv_dtype_of(kv_cache.element_type());
  a.causal = causal;
  a.window_left = window_left;
  a.softmax_scale = softmax_scale;
  a.softcap = softcap;
  a.token_major = token_major;
  if (rotary_cos.element_count() != 0) {
    a.rotary_cos = rotary_cos.untyped_data();
    a.rotary_sin = rotary_sin.untyped_data();
    a.rotary_len = static_cast<int32_t>(rotary_cos.dimensions()[0]);
    a.rotary_interleaved = rotary_interleaved;
    a.rotary_bf16 = rotary_cos.element_type() == ffi::DataType::BF16;
  }
  a.route = FW_ROUTE_AUTO;
  if (ffi::Error err = clear_status_block(*workspace, stream); err.failure()) return err;
  return to_error(fw_prefill_paged(&a, stream));
}

// ---------------------------------------------------------------- (o, lse) merge
// Operands: partial_out f32[parts, rows, d]; partial_lse f32[parts, rows]; sinks
// f32[nheads] or empty.  Results: out bf16[rows, d]; lse f32[rows] or empty.
ffi::Error CombineImpl(cudaStream_t stream, ffi::AnyBuffer partial_out, ffi::AnyBuffer partial_lse,
                       ffi::AnyBuffer sinks, ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> lse,
                       int32_t nheads) {
  const auto pd = partial_out.dimensions();
  if (pd.size() != 3) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "partial_out must be (parts, rows, head_dim)");
  FwCombineArgs a = {};
  a.partial_out = static_cast<const float*>(partial_out.untyped_data());
  a.partial_lse = static_cast<const float*>(partial_lse.untyped_data());
  a.sinks = static_cast<const float*>(data_or_null(sinks));
  a.out = out->untyped_data();
  a.lse = static_cast<float*>(data_or_null(*lse));
  a.parts = static_cast<int32_t>(pd[0]);
  a.rows = static_cast<int32_t>(pd[1]);
  a.nheads = nheads;
  a.head_dim = static_cast<int32_t>(pd[2]);
  a.lse_head_stride = 1;   // lse[row], row = token * nheads + head
  a.lse_token_stride = nheads;
  return to_error(fw_lse_combine(&a, stream));
}

}  // namespace

#define FW_CUDA_STREAM ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>()

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    fw_decode_kvcache_ffi, DecodeImpl,
    FW_CUDA_STREAM.Arg<ffi::AnyBuffer>()  // q
        .Arg<ffi::AnyBuffer>()            // kv_cache
        .Arg<ffi::AnyBuffer>()            // v_cache
        .Arg<ffi::AnyBuffer>()            // k_new
        .Arg<ffi::AnyBuffer>()            // v_new
        .Arg<ffi::AnyBuffer>()            // cache_seqlens
        .Arg<ffi::AnyBuffer>()            // block_table
        .Arg<ffi::AnyBuffer>()            // cache_batch_idx
        .Arg<ffi::AnyBuffer>()            // num_active
        .Arg<ffi::AnyBuffer>()            // k_descale
        .Arg<ffi::AnyBuffer>()            // v_descale
        .Arg<ffi::AnyBuffer>()            // sinks
        .Ret<ffi::AnyBuffer>()            // out
        .Ret<ffi::AnyBuffer>()            // lse
        .Ret<ffi::AnyBuffer>()            // kv_cache_out
        .Ret<ffi::AnyBuffer>()            // v_cache_out
        .Ret<ffi::AnyBuffer>()            // workspace
        .Attr<int32_t>("nheads_k")
        .Attr<int32_t>("causal")
        .Attr<int32_t>("window_left")
        .Attr<float>("softmax_scale")
        .Attr<float>("softcap"),
    {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    fw_append_ragged_ffi, AppendImpl,
    FW_CUDA_STREAM.Arg<ffi::AnyBuffer>()  // kv_cache
        .Arg<ffi::AnyBuffer>()            // k_new
        .Arg<ffi::AnyBuffer>()            // v_new
        .Arg<ffi::AnyBuffer>()            // cu_seqlens_q
        .Arg<ffi::AnyBuffer>()            // cache_seqlens
        .Arg<ffi::AnyBuffer>()            // block_table
        .Arg<ffi::AnyBuffer>()            // num_active
        .Ret<ffi::AnyBuffer>(),           // kv_cache_out
    {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    fw_write_kv_pages_ffi, WritePagesImpl,
    FW_CUDA_STREAM.Arg<ffi::AnyBuffer>()  // kv_cache
        .Arg<ffi::AnyBuffer>()            // k_new
        .Arg<ffi::AnyBuffer>()            // v_new
        .Arg<ffi::AnyBuffer>()            // slices
        .Arg<ffi::AnyBuffer>()            // num_slices
        .Ret<ffi::AnyBuffer>(),           // kv_cache_out
    {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    fw_prefill_paged_ffi, PrefillImpl,
    FW_CUDA_STREAM.Arg<ffi::AnyBuffer>()  // q
        .Arg<ffi::AnyBuffer>()            // kv_cache
        .Arg<ffi::AnyBuffer>()            // cu_seqlens_q
        .Arg<ffi::AnyBuffer>()            // seqused_k
        .Arg<ffi::AnyBuffer>()            // block_table
        .Arg<ffi::AnyBuffer>()            // num_active
        .Arg<ffi::AnyBuffer>()            // k_descale
        .Arg<ffi::AnyBuffer>()            // v_descale
        .Arg<ffi::AnyBuffer>()            // sinks
        .Arg<ffi::AnyBuffer>()            // rotary_cos
        .Arg<ffi::AnyBuffer>()            // rotary_sin
        .Ret<ffi::AnyBuffer>()            // out
        .Ret<ffi::AnyBuffer>()            // lse
        .Ret<ffi::AnyBuffer>()            // workspace
        .Attr<int32_t>("nheads_k")
        .Attr<int32_t>("max_seqlen_q")
        .Attr<int32_t>("causal")
        .Attr<int32_t>("window_left")
        .Attr<int32_t>("token_major")
        .Attr<int32_t>("rotary_interleaved")
        .Attr<float>("softmax_scale")
        .Attr<float>("softcap"),
    {ffi::Traits::kCmdBufferCompatible});

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    fw_lse_combine_ffi, CombineImpl,
    FW_CUDA_STREAM.Arg<ffi::AnyBuffer>()  // partial_out
        .Arg<ffi::AnyBuffer>()            // partial_lse
        .Arg<ffi::AnyBuffer>()            // sinks
        .Ret<ffi::AnyBuffer>()            // out
        .Ret<ffi::AnyBuffer>()            // lse
        .Attr<int32_t>("nheads"),
    {ffi::Traits::kCmdBufferCompatible});
