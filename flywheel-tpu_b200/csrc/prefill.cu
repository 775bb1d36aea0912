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
  if (a->head_dim != 128 && a->head_dim != 256) {
    set_error("head_dim %d is not built; this library serves head_dim 128 and 256.", a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  if (a->total_q < 0 || a->batch <= 0) {
    set_error("batch must be positive and total_q non-negative.");
    return FW_ERR_BAD_SHAPE;
  }
  if ((a->rotary_cos == nullptr) != (a->rotary_sin == nullptr)) {
    set_error("rotary_cos and rotary_sin must be provided together.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->rotary_cos != nullptr && a->rotary_len <= 0) {
    set_error("rotary tables need a positive rotary_len.");
    return FW_ERR_BAD_SHAPE;
  }
  return FW_OK;
}

// ---------------------------------------------------------------- Q-only RoPE
// Rotates packed q into a scratch copy before attention: token t of request r
// sits at position seqused_k[r] - len_q(r) + t (its own K/V position), the
// rotation runs in f32 and rounds once to bf16.  Rows outside every request
// and positions past the table are copied unrotated.
struct RopeParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* q_out;
  const void* cos;
  const void* sin;
  const int* cu;       // token ownership: request r holds rows [cu[r], cu[r + 1])
  const int* seqused;  // request r's key count, or NULL: then it is cu_k[r + 1] - cu_k[r]
  const int* cu_k;
  long long tok_stride, head_stride;
  int batch, total_q, nheads, rotary_len, interleaved, table_bf16, head_dim;
};

__device__ __forceinline__ float table_value(const void* table, long long index, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(table)[index])
                 : static_cast<const float*>(table)[index];
}

// One thread per (token, head, 8 rotation pairs): head_dim / 16 threads per row.
__global__ void __launch_bounds__(256) rope_q_kernel(const RopeParams p) {
  const int parts = p.head_dim / 16, half = p.head_dim / 2;
  const long long total = static_cast<long long>(p.total_q) * p.nheads * parts;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int part = static_cast<int>(idx % parts);
    const long long th = idx / parts;
    const int hq = static_cast<int>(th % p.nheads);
    const int tok = static_cast<int>(th / p.nheads);
    const long long base = static_cast<long long>(tok) * p.tok_stride + static_cast<long long>(hq) * p.head_stride;
    // request owning the token: largest r with cu[r] <= tok
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.cu[mid] <= tok) lo = mid; else hi = mid;
    }
    int pos = -1;
    if (tok >= p.cu[lo] && tok < p.cu[lo + 1]) {
      const int used = p.seqused ? p.seqused[lo] : p.cu_k[lo + 1] - p.cu_k[lo];
      pos = used - (p.cu[lo + 1] - p.cu[lo]) + (tok - p.cu[lo]);
    }
    const bool rotate = pos >= 0 && pos < p.rotary_len;
    // This thread's 8 pairs: split halves pair element i with i + head_dim / 2;
    // interleaved pairs (2i, 2i + 1).
    if (!p.interleaved) {
      const int i0 = part * 8;
      uint4 a = *reinterpret_cast<const uint4*>(p.q + base + i0);
      uint4 b = *reinterpret_cast<const uint4*>(p.q + base + half + i0);
      if (rotate) {
        __nv_bfloat16* x1 = reinterpret_cast<__nv_bfloat16*>(&a);
        __nv_bfloat16* x2 = reinterpret_cast<__nv_bfloat16*>(&b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float c = table_value(p.cos, static_cast<long long>(pos) * half + i0 + i, p.table_bf16);
          const float s = table_value(p.sin, static_cast<long long>(pos) * half + i0 + i, p.table_bf16);
          const float u = __bfloat162float(x1[i]), w = __bfloat162float(x2[i]);
          x1[i] = __float2bfloat16_rn(u * c - w * s);
          x2[i] = __float2bfloat16_rn(u * s + w * c);
        }
      }
      *reinterpret_cast<uint4*>(p.q_out + base + i0) = a;
      *reinterpret_cast<uint4*>(p.q_out + base + half + i0) = b;
    } else {
      const int e0 = part * 16;
      uint4 a = *reinterpret_cast<const uint4*>(p.q + base + e0);
      uint4 b = *reinterpret_cast<const uint4*>(p.q + base + e0 + 8);
      if (rotate) {
        __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(&a);
        __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(&b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          __nv_bfloat16* pair = i < 4 ? x + 2 * i : y + 2 * (i - 4);
          const float c = table_value(p.cos, static_cast<long long>(pos) * half + part * 8 + i, p.table_bf16);
          const float s = table_value(p.sin, static_cast<long long>(pos) * half + part * 8 + i, p.table_bf16);
          const float u = __bfloat162float(pair[0]), w = __bfloat162float(pair[1]);
          pair[0] = __float2bfloat16_rn(u * c - w * s);
          pair[1] = __float2bfloat16_rn(u * s + w * c);
        }
      }
      *reinterpret_cast<uint4*>(p.q_out + base + e0) = a;
      *reinterpret_cast<uint4*>(p.q_out + base + e0 + 8) = b;
    }
  }
}

static uint64_t rope_bytes(const FwPrefillArgs* a) {
  if (a->rotary_cos == nullptr) return 0;
  return (static_cast<uint64_t>(a->total_q) * a->nheads * a->head_dim * 2 + 255) & ~255ull;
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

static uint64_t attention_workspace_bytes(const FwPrefillArgs* a) {
  const uint64_t n = use_tensor_core_kernel(a) ? tcgen05_prefill_workspace_bytes(a)
                                               : splitkv_prefill_workspace_bytes(a);
  return n == 0 ? 0 : (n + 255) & ~255ull;
}

extern "C" uint64_t fw_prefill_workspace_bytes(const FwPrefillArgs* a) {
  if (check_prefill_args(a) != FW_OK) return 0;
  const uint64_t n = attention_workspace_bytes(a);
  return n == 0 ? 0 : n + rope_bytes(a);
}

extern "C" int fw_prefill_paged(const FwPrefillArgs* a, void* stream_ptr) {
  int rc = check_prefill_args(a);
  if (rc != FW_OK) return rc;
  if (a->total_q == 0) return FW_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  FwPrefillArgs local = *a;
  if (a->rotary_cos != nullptr) {
    // The rotated copy of q lives behind the attention kernels' own scratch.
    const uint64_t head = attention_workspace_bytes(a);
    if (head == 0) return FW_ERR_UNSUPPORTED;
    if (a->workspace == nullptr || a->workspace_bytes < head + rope_bytes(a) ||
        (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
      set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
                static_cast<unsigned long long>(head + rope_bytes(a)),
                static_cast<unsigned long long>(a->workspace_bytes));
      return FW_ERR_WORKSPACE;
    }
    if (a->q == nullptr || a->cu_seqlens_q == nullptr || a->seqused_k == nullptr) {
      set_error("q, cu_seqlens_q and seqused_k must not be NULL.");
      return FW_ERR_BAD_SHAPE;
    }
    RopeParams rp;
    rp.q = static_cast<const __nv_bfloat16*>(a->q);
    rp.q_out = reinterpret_cast<__nv_bfloat16*>(static_cast<uint8_t*>(a->workspace) + head);
    rp.cos = a->rotary_cos;
    rp.sin = a->rotary_sin;
    rp.cu = a->cu_seqlens_q;
    rp.seqused = a->seqused_k;
    rp.cu_k = nullptr;
    rp.tok_stride = a->token_major ? static_cast<long long>(a->nheads) * a->head_dim : a->head_dim;
    rp.head_stride = a->token_major ? a->head_dim : static_cast<long long>(a->total_q) * a->head_dim;
    rp.head_dim = a->head_dim;
    rp.batch = a->batch;
    rp.total_q = a->total_q;
    rp.nheads = a->nheads;
    rp.rotary_len = a->rotary_len;
    rp.interleaved = a->rotary_interleaved;
    rp.table_bf16 = a->rotary_bf16;
    const long long threads = static_cast<long long>(a->total_q) * a->nheads * (a->head_dim / 16);
    const long long want = (threads + 255) / 256, cap = static_cast<long long>(sm_count()) * 32;
    rope_q_kernel<<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(rp);
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
      set_error("rope kernel launch: %s", cudaGetErrorString(err));
      return FW_ERR_LAUNCH;
    }
    local.q = rp.q_out;
    local.workspace_bytes = head;
  }
  if (use_tensor_core_kernel(&local)) return tcgen05_prefill(&local, stream);
  return splitkv_prefill(&local, stream);
}

// ---------------------------------------------------------------- packed K/V
// flash_attn_varlen_func without a block table and flash_attn_func of the
// reference project (flywheel_tpu/softmax_attention/prefill.py:818-963 and
// 62-341): the tensor-core kernel with K and V addressed by token row.
static int check_packed_args(const FwPrefillArgs* a) {
  int rc = check_prefill_args(a);
  if (rc != FW_OK) return rc;
  if (a->block_table != nullptr || a->seqused_k != nullptr || a->num_active != nullptr ||
      a->k_descale != nullptr || a->v_descale != nullptr) {
    set_error("block_table, seqused_k, num_active and the descales describe a paged cache; packed K/V takes"
              " cu_seqlens_k.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->kv_dtype != FW_DTYPE_BF16) {
    set_error("packed K/V is bfloat16.");
    return FW_ERR_BAD_DTYPE;
  }
  if (a->v_packed == nullptr || a->cu_seqlens_k == nullptr || a->total_k <= 0) {
    set_error("v, cu_seqlens_k and a positive total_k are required.");
    return FW_ERR_BAD_SHAPE;
  }
  if (!tcgen05_prefill_supported(a)) {
    set_error("packed K/V attention is built for head_dim 128 and nheads / nheads_k up to 128;"
              " got head_dim %d, nheads %d, nheads_k %d.", a->head_dim, a->nheads, a->nheads_k);
    return FW_ERR_UNSUPPORTED;
  }
  return FW_OK;
}

static uint64_t packed_rope_k_bytes(const FwPrefillArgs* a) {
  if (a->rotary_cos == nullptr || !a->rotary_k) return 0;
  return (static_cast<uint64_t>(a->total_k) * a->nheads_k * a->head_dim * 2 + 255) & ~255ull;
}

extern "C" uint64_t fw_attention_packed_workspace_bytes(const FwPrefillArgs* a) {
  if (check_packed_args(a) != FW_OK) return 0;
  return ((tcgen05_prefill_workspace_bytes(a) + 255) & ~255ull) + rope_bytes(a) + packed_rope_k_bytes(a);
}

static int launch_rope(const RopeParams& rp, long long rows, cudaStream_t stream) {
  const long long threads = rows * rp.nheads * (rp.head_dim / 16);
  const long long want = (threads + 255) / 256, cap = static_cast<long long>(sm_count()) * 32;
  rope_q_kernel<<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(rp);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("rope kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_attention_packed(const FwPrefillArgs* a, void* stream_ptr) {
  int rc = check_packed_args(a);
  if (rc != FW_OK) return rc;
  if (a->total_q == 0) return FW_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  FwPrefillArgs local = *a;
  const uint64_t head = (tcgen05_prefill_workspace_bytes(a) + 255) & ~255ull;
  if (a->rotary_cos != nullptr) {
    const uint64_t need = head + rope_bytes(a) + packed_rope_k_bytes(a);
    if (a->workspace == nullptr || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
      set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
                static_cast<unsigned long long>(need), static_cast<unsigned long long>(a->workspace_bytes));
      return FW_ERR_WORKSPACE;
    }
    if (a->q == nullptr || a->kv_cache == nullptr || a->cu_seqlens_q == nullptr) {
      set_error("q, k and cu_seqlens_q must not be NULL.");
      return FW_ERR_BAD_SHAPE;
    }
    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    RopeParams rp;
    rp.q = static_cast<const __nv_bfloat16*>(a->q);
    rp.q_out = reinterpret_cast<__nv_bfloat16*>(ws + head);
    rp.cos = a->rotary_cos;
    rp.sin = a->rotary_sin;
    rp.cu = a->cu_seqlens_q;
    rp.seqused = nullptr;
    rp.cu_k = a->cu_seqlens_k;
    rp.tok_stride = a->token_major ? static_cast<long long>(a->nheads) * a->head_dim : a->head_dim;
    rp.head_stride = a->token_major ? a->head_dim : static_cast<long long>(a->total_q) * a->head_dim;
    rp.batch = a->batch;
    rp.total_q = a->total_q;
    rp.nheads = a->nheads;
    rp.rotary_len = a->rotary_len;
    rp.interleaved = a->rotary_interleaved;
    rp.table_bf16 = a->rotary_bf16;
    rp.head_dim = a->head_dim;
    rc = launch_rope(rp, a->total_q, stream);
    if (rc != FW_OK) return rc;
    local.q = rp.q_out;
    if (a->rotary_k) {
      // K's token t of a request sits at position t: rotate it as a tensor whose
      // rows are its own keys (length = key count).
      RopeParams rk = rp;
      rk.q = static_cast<const __nv_bfloat16*>(a->kv_cache);
      rk.q_out = reinterpret_cast<__nv_bfloat16*>(ws + head + rope_bytes(a));
      rk.cu = a->cu_seqlens_k;
      rk.tok_stride = a->kv_token_major ? static_cast<long long>(a->nheads_k) * a->head_dim : a->head_dim;
      rk.head_stride = a->kv_token_major ? a->head_dim : static_cast<long long>(a->total_k) * a->head_dim;
      rk.total_q = a->total_k;
      rk.nheads = a->nheads_k;
      rc = launch_rope(rk, a->total_k, stream);
      if (rc != FW_OK) return rc;
      local.kv_cache = rk.q_out;
    }
    local.workspace_bytes = head;
  }
  return tcgen05_prefill(&local, stream);
}
