// fw_prefill_paged: chunked prefill over the paged merged cache
// (flash_attn_varlen_func with block_table; reference
// flywheel_tpu/softmax_attention/prefill.py:437-661).  Picks the kernel.
#include <cstdlib>
#include <cstring>

#include "common.cuh"

using namespace fw;

static int check_prefill_args(const FwPrefillArgs* a) {
  if (a == nullptr) {
    set_error("args is NULL");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->kv_dtype != FW_DTYPE_BF16 && a->kv_dtype != FW_DTYPE_E4M3 && a->kv_dtype != FW_DTYPE_E5M2) {
    set_error("kv_dtype must be bf16, e4m3 or e5m2; got %d", a->kv_dtype);
    return FW_ERR_BAD_DTYPE;
  }
  if (a->head_dim != 128) {
    set_error("head_dim %d is not built; this library serves head_dim 128.", a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  if (a->total_q < 0 || a->batch <= 0) {
    set_error("batch must be positive and total_q non-negative.");
    return FW_ERR_BAD_SHAPE;
  }
  return FW_OK;
}

// Chunks of at least this many tokens go to the tensor-core kernel; shorter
// ones are KV-streaming work and go to the split-KV kernel.  The environment
// variable FLYWHEEL_PREFILL_KERNEL=tcgen05|splitkv pins the choice (tests and
// profiling).
static constexpr int kTensorCoreMinChunk = 64;

static bool use_tensor_core_kernel(const FwPrefillArgs* a) {
  if (!tcgen05_prefill_supported(a)) return false;
  const char* pin = std::getenv("FLYWHEEL_PREFILL_KERNEL");
  if (pin != nullptr && std::strcmp(pin, "splitkv") == 0) return false;
  if (pin != nullptr && std::strcmp(pin, "tcgen05") == 0) return true;
  return a->max_seqlen_q >= kTensorCoreMinChunk;
}

extern "C" uint64_t fw_prefill_workspace_bytes(const FwPrefillArgs* a) {
  if (check_prefill_args(a) != FW_OK) return 0;
  if (use_tensor_core_kernel(a)) return tcgen05_prefill_workspace_bytes(a);
  return splitkv_prefill_workspace_bytes(a);
}

extern "C" int fw_prefill_paged(const FwPrefillArgs* a, void* stream) {
  int rc = check_prefill_args(a);
  if (rc != FW_OK) return rc;
  if (a->total_q == 0) return FW_OK;
  if (use_tensor_core_kernel(a)) return tcgen05_prefill(a, static_cast<cudaStream_t>(stream));
  return splitkv_prefill(a, static_cast<cudaStream_t>(stream));
}
