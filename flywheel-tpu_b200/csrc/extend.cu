// fw_extend_mixed: one mixed serving step (decode rows + prefill chunks of one
// batch) as one launch sequence.  Follows flywheel_tpu_extend of the reference
// project's serving backend (patches/tpu-inference.patch:8219-8320): page write,
// decode kernel over the leading one-token requests, paged prefill over the
// rest.  The reference slides the request window past the decode rows on the
// host side of the trace; here the counts stay on the device and the prefill's
// plan kernel simply starts at request *num_decode.
#include "common.cuh"

using namespace fw;

namespace {

constexpr uint64_t kStatusBytes = 256;

struct ExtendPlan {
  FwPrefillArgs prefill;
  FwDecodeArgs decode;
  uint64_t prefill_bytes, decode_bytes, bytes;
};

uint64_t align256(uint64_t n) { return (n + 255) & ~255ull; }

int plan_extend(const FwExtendArgs* a, ExtendPlan* plan) {
  if (a == nullptr) {
    set_error("args is NULL");
    return FW_ERR_BAD_SHAPE;
  }
  const FwPrefillArgs& in = a->attn;
  if (!in.token_major) {
    set_error("a mixed step takes token-major q (total_q, nheads, head_dim): set attn.token_major.");
    return FW_ERR_BAD_SHAPE;
  }
  if (in.lse != nullptr || in.rotary_cos != nullptr || in.rotary_sin != nullptr) {
    set_error("a mixed step returns no lse and takes no rotary tables.");
    return FW_ERR_UNSUPPORTED;
  }
  if (in.block_table == nullptr || in.seqused_k == nullptr || in.cu_seqlens_q == nullptr ||
      a->num_decode == nullptr) {
    set_error("block_table, seqused_k, cu_seqlens_q and num_decode must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if ((a->k_new == nullptr) != (a->v_new == nullptr) || (a->k_new != nullptr && (a->slices == nullptr ||
                                                                               a->num_slices == nullptr))) {
    set_error("k_new, v_new, slices and num_slices must be passed together, or all left out.");
    return FW_ERR_BAD_SHAPE;
  }
  if (in.batch <= 0 || in.total_q <= 0) {
    set_error("batch and total_q must be positive.");
    return FW_ERR_BAD_SHAPE;
  }
  plan->prefill = in;
  plan->prefill.first_request = a->num_decode;
  plan->prefill.workspace = nullptr;
  plan->prefill.workspace_bytes = 0;
  plan->prefill_bytes = align256(fw_prefill_workspace_bytes(&plan->prefill));
  if (plan->prefill_bytes == 0) return FW_ERR_UNSUPPORTED;  // fw_last_error says why

  // The decode rows: request b < *num_decode owns packed row b (one token each),
  // so q and out are read as (rows, 1, nheads, head_dim).  Rows that are not
  // decode requests come back as zeros and are then written by the prefill, or
  // cleared by its plan kernel, or are real zeros (past the last request).
  FwDecodeArgs& d = plan->decode;
  d = FwDecodeArgs{};
  d.q = in.q;
  d.out = in.out;
  d.kv_cache = const_cast<void*>(in.kv_cache);
  d.cache_seqlens = in.seqused_k;  // the step's tokens are in the pool already: nothing to append
  d.block_table = in.block_table;
  d.num_active = a->num_decode;
  d.k_descale = in.k_descale;
  d.v_descale = in.v_descale;
  d.sinks = in.sinks;
  d.num_pages = in.num_pages;
  d.page_size = in.page_size;
  d.pages_per_seq = in.pages_per_seq;
  d.batch = in.batch < in.total_q ? in.batch : in.total_q;
  d.seqlen_q = 1;
  d.nheads = in.nheads;
  d.nheads_k = in.nheads_k;
  d.head_dim = in.head_dim;
  d.kv_dtype = in.kv_dtype;
  d.causal = 1;
  d.window_left = in.window_left;
  d.softmax_scale = in.softmax_scale;
  d.softcap = in.softcap;
  plan->decode_bytes = align256(fw_decode_workspace_bytes(&d));
  if (plan->decode_bytes == 0) return FW_ERR_UNSUPPORTED;
  plan->bytes = plan->prefill_bytes + plan->decode_bytes;
  return FW_OK;
}

}  // namespace

extern "C" uint64_t fw_extend_workspace_bytes(const FwExtendArgs* a) {
  ExtendPlan plan;
  return plan_extend(a, &plan) == FW_OK ? plan.bytes : 0;
}

extern "C" int fw_extend_mixed(const FwExtendArgs* a, void* stream_ptr) {
  ExtendPlan plan;
  int rc = plan_extend(a, &plan);
  if (rc != FW_OK) return rc;
  const FwPrefillArgs& in = a->attn;
  if (in.workspace == nullptr || in.workspace_bytes < plan.bytes || (reinterpret_cast<uintptr_t>(in.workspace) & 255)) {
    set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
              static_cast<unsigned long long>(plan.bytes), static_cast<unsigned long long>(in.workspace_bytes));
    return FW_ERR_WORKSPACE;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (a->k_new != nullptr) {
    FwWritePagesArgs w = {};
    w.kv_cache = const_cast<void*>(in.kv_cache);
    w.k_new = a->k_new;
    w.v_new = a->v_new;
    w.slices = a->slices;
    w.num_slices = a->num_slices;
    w.num_pages = in.num_pages;
    w.page_size = in.page_size;
    w.num_columns = a->num_columns;
    w.total_tokens = a->total_tokens;
    w.nheads_k = in.nheads_k;
    w.head_dim = in.head_dim;
    w.kv_dtype = in.kv_dtype;
    rc = fw_write_kv_pages(&w, stream);
    if (rc != FW_OK) return rc;
  }
  // [prefill scratch (status block at its head) | decode scratch]; the decode
  // kernels report into the same status word.
  uint8_t* ws = static_cast<uint8_t*>(in.workspace);
  plan.decode.workspace = ws + plan.prefill_bytes;
  plan.decode.workspace_bytes = plan.decode_bytes;
  rc = decode_with_status(&plan.decode, reinterpret_cast<int*>(ws), stream);
  if (rc != FW_OK) return rc;
  plan.prefill.workspace = ws;
  plan.prefill.workspace_bytes = plan.prefill_bytes;
  return fw_prefill_paged(&plan.prefill, stream);
}
