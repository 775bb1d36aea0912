// Chunked prefill over the paged merged cache (flash_attn_varlen_func with
// block_table).  Placeholder entry points until the kernel lands.
#include "common.cuh"

using namespace fw;

extern "C" uint64_t fw_prefill_workspace_bytes(const FwPrefillArgs* args) {
  (void)args;
  return 0;
}

extern "C" int fw_prefill_paged(const FwPrefillArgs* args, void* stream) {
  (void)args;
  (void)stream;
  set_error("fw_prefill_paged is not built yet.");
  return FW_ERR_UNSUPPORTED;
}
