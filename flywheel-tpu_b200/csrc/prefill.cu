// fw_prefill_paged: chunked prefill over the paged merged cache
// (flash_attn_varlen_func with block_table; reference
// flywheel_tpu/softmax_attention/prefill.py:437-661).  Picks the kernel.
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
  const bool packed_kv = a->block_table == nullptr && a->v_packed != nullptr;
  if (a->head_dim != 128 && a->head_dim != 256 && !(a->head_dim == 64 && packed_kv)) {
    set_error("head_dim %d is not built; the paged paths serve head_dim 128 and 256, packed K/V also 64.",
              a->head_dim);
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
  if (a->route != FW_ROUTE_AUTO && a->route != FW_ROUTE_TENSOR_CORE && a->route != FW_ROUTE_SPLIT_KV) {
    set_error("route must be FW_ROUTE_AUTO, FW_ROUTE_TENSOR_CORE or FW_ROUTE_SPLIT_KV; got %d.", a->route);
    return FW_ERR_BAD_SHAPE;
  }
  return FW_OK;
}

// ---------------------------------------------------------------- RoPE pre-pass
// The tensor-core kernels rotate Q themselves, in shared memory, right after the
// TMA copy of the Q tile (tcgen05.cuh).  This kernel remains for what they do not
// cover: Q on the split-KV route (short chunks) and K of packed K/V.  It rotates
// packed rows into a scratch copy: token t of request r sits at position
// seqused_k[r] - len_q(r) + t (its own K/V position), the rotation runs in f32
// and rounds once to bf16.  Rows outside every request and positions past the
// table are copied unrotated.
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

// Scratch for a rotated copy of q: only the split-KV route needs one.
static uint64_t rope_copy_bytes(const FwPrefillArgs* a) {
  if (a->rotary_cos == nullptr) return 0;
  return (static_cast<uint64_t>(a->total_q) * a->nheads * a->head_dim * 2 + 255) & ~255ull;
}

// ---------------------------------------------------------------- gather for the tensor-core kernel
// The tensor-core kernels read K/V through 64-token TMA boxes; the head_dim 128
// kernel reads bf16 and fp8 pools in place (it widens fp8 tiles itself).  Pools
// they cannot read in place (pages that are not a multiple of 64 tokens; fp8 at
// head_dim 256) are first copied, request by request, into bf16 K and V scratch tensors of
// (batch * capacity, nheads_k, head_dim), capacity = pages_per_seq * page_size:
// request r's key t lands in row r * capacity + t.  fp8 widens exactly to bf16;
// the descales stay where they were (score scale and output scale).  One block
// per (page, request); pages past the request's length are skipped.
struct GatherParams {
  const uint8_t* pool;
  const int* block_table;
  const int* seqused;
  const int* num_active;
  __nv_bfloat16* k_out;
  __nv_bfloat16* v_out;
  int* status;
  long long num_pages;
  int batch, page_size, pages_per_seq, nheads_k, cache_heads, head_dim, kv_dtype;
};

template <int KVT>
__device__ __forceinline__ uint4 widen8(uint2 raw) {
  // eight fp8 values -> eight bf16 (exact: fp8 -> f16 -> f32 -> bf16 loses nothing)
  uint32_t h[4] = {fp8x2_to_f16x2<KVT>(raw.x & 0xffff), fp8x2_to_f16x2<KVT>(raw.x >> 16),
                   fp8x2_to_f16x2<KVT>(raw.y & 0xffff), fp8x2_to_f16x2<KVT>(raw.y >> 16)};
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[i]));
    o[i] = pack_bf16(f.x, f.y);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void __launch_bounds__(256) gather_kv_kernel(const GatherParams p) {
  const int page_idx = blockIdx.x, r = blockIdx.y;
  const int n_active = p.num_active ? min(p.batch, max(0, *p.num_active)) : p.batch;
  if (r >= n_active) return;
  const int used = p.seqused[r];
  const int tok0 = page_idx * p.page_size;
  if (tok0 >= used) return;
  int page = p.block_table[static_cast<long long>(r) * p.pages_per_seq + page_idx];
  if (page < 0 || page >= p.num_pages) {
    if (threadIdx.x == 0) report_status(p.status, FW_STATUS_BAD_PAGE);
    page = 0;
  }
  const int itemsize = p.kv_dtype == FW_DTYPE_BF16 ? 2 : 1;
  const int tokens = min(p.page_size, used - tok0);
  const int chunks_per_plane = p.head_dim / 8;                 // 16-byte output chunks per head plane
  const long long row_bytes = static_cast<long long>(p.cache_heads) * p.head_dim * itemsize;
  const uint8_t* src_page = p.pool + static_cast<long long>(page) * p.page_size * row_bytes;
  const long long capacity = static_cast<long long>(p.pages_per_seq) * p.page_size;
  const int per_token = 2 * p.nheads_k * chunks_per_plane;
  for (int i = threadIdx.x; i < tokens * per_token; i += blockDim.x) {
    const int t = i / per_token, rem = i - t * per_token;
    const int plane = rem / chunks_per_plane, c = rem - plane * chunks_per_plane;  // plane = 2 * head + is_v
    const uint8_t* src = src_page + t * row_bytes + (static_cast<long long>(plane) * p.head_dim + c * 8) * itemsize;
    uint4 value;
    if (p.kv_dtype == FW_DTYPE_BF16) value = *reinterpret_cast<const uint4*>(src);
    else if (p.kv_dtype == FW_DTYPE_E4M3) value = widen8<FW_DTYPE_E4M3>(*reinterpret_cast<const uint2*>(src));
    else value = widen8<FW_DTYPE_E5M2>(*reinterpret_cast<const uint2*>(src));
    __nv_bfloat16* dst = ((plane & 1) ? p.v_out : p.k_out) +
                         ((r * capacity + tok0 + t) * p.nheads_k + (plane >> 1)) * p.head_dim + c * 8;
    *reinterpret_cast<uint4*>(dst) = value;
  }
}

// Chunks of at least this many tokens go to the tensor-core kernel; shorter
// ones are KV-streaming work and go to the split-KV kernel.  Pools the
// tensor-core kernel cannot read in place take the gather above first, which
// pays off once a chunk is a few hundred tokens (the copy is linear in the key
// count, the attention is chunk times that).  FwPrefillArgs.route pins the
// choice for one call (tests and profiling); nothing process-wide is consulted.
static constexpr int kTensorCoreMinChunk = 64;
static constexpr int kGatherMinChunk = 256;

enum class PrefillRoute { kTensorCore, kGatherTensorCore, kSplitKv };

static bool gather_route_possible(const FwPrefillArgs* a) {
  if (a->block_table == nullptr || a->page_size <= 0 || a->pages_per_seq <= 0) return false;
  if (a->page_size % 16) return false;  // the split-KV kernel reports the shape error
  // what the tensor-core kernel will be asked after the copy: bf16, and no page
  // size to object to (64 stands for "any")
  FwPrefillArgs as_packed = *a;
  as_packed.kv_dtype = FW_DTYPE_BF16;
  as_packed.page_size = 64;
  if (!tcgen05_prefill_supported(&as_packed)) return false;
  const long long rows = static_cast<long long>(a->batch) * a->pages_per_seq * a->page_size;
  return rows < (1ll << 31);
}

static PrefillRoute pick_route(const FwPrefillArgs* a) {
  const bool pin_split = a->route == FW_ROUTE_SPLIT_KV;
  const bool pin_tensor = a->route == FW_ROUTE_TENSOR_CORE;
  if (pin_split) return PrefillRoute::kSplitKv;
  if (tcgen05_prefill_supported(a))
    return pin_tensor || a->max_seqlen_q >= kTensorCoreMinChunk ? PrefillRoute::kTensorCore : PrefillRoute::kSplitKv;
  if (gather_route_possible(a) && (pin_tensor || a->max_seqlen_q >= kGatherMinChunk))
    return PrefillRoute::kGatherTensorCore;
  return PrefillRoute::kSplitKv;
}

static uint64_t gather_scratch_bytes(const FwPrefillArgs* a) {
  const uint64_t rows = static_cast<uint64_t>(a->batch) * a->pages_per_seq * a->page_size;
  return (rows * a->nheads_k * a->head_dim * 2 + 255) & ~255ull;  // one of K / V
}

static uint64_t attention_workspace_bytes(const FwPrefillArgs* a) {
  uint64_t n = 0;
  switch (pick_route(a)) {
    case PrefillRoute::kTensorCore: n = tcgen05_prefill_workspace_bytes(a); break;
    case PrefillRoute::kGatherTensorCore: n = tcgen05_prefill_workspace_bytes(a); break;
    case PrefillRoute::kSplitKv: n = splitkv_prefill_workspace_bytes(a); break;
  }
  return n == 0 ? 0 : (n + 255) & ~255ull;
}

static uint64_t rope_bytes(const FwPrefillArgs* a) {
  return pick_route(a) == PrefillRoute::kSplitKv ? rope_copy_bytes(a) : 0;
}

extern "C" uint64_t fw_prefill_workspace_bytes(const FwPrefillArgs* a) {
  if (check_prefill_args(a) != FW_OK) return 0;
  const uint64_t n = attention_workspace_bytes(a);
  if (n == 0) return 0;
  const uint64_t gather = pick_route(a) == PrefillRoute::kGatherTensorCore ? 2 * gather_scratch_bytes(a) : 0;
  return n + rope_bytes(a) + gather;
}

extern "C" int fw_prefill_paged(const FwPrefillArgs* a, void* stream_ptr) {
  int rc = check_prefill_args(a);
  if (rc != FW_OK) return rc;
  if (a->total_q == 0) return FW_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  FwPrefillArgs local = *a;
  const PrefillRoute route = pick_route(a);
  if (a->rotary_cos != nullptr && route == PrefillRoute::kSplitKv) {
    // The split-KV kernel reads q from global memory: rotate a copy first.  It
    // lives behind the attention kernel's own scratch.
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
    local.rotary_cos = local.rotary_sin = nullptr;  // done
    local.workspace_bytes = head;
  }
  switch (route) {
    case PrefillRoute::kTensorCore: return tcgen05_prefill(&local, stream);
    case PrefillRoute::kSplitKv: return splitkv_prefill(&local, stream);
    case PrefillRoute::kGatherTensorCore: break;
  }
  // Gather route: [attention scratch | rotated q | K scratch | V scratch].
  const uint64_t head = attention_workspace_bytes(a), rope = rope_bytes(a), plane = gather_scratch_bytes(a);
  if (a->workspace == nullptr || a->workspace_bytes < head + rope + 2 * plane ||
      (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
    set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
              static_cast<unsigned long long>(head + rope + 2 * plane),
              static_cast<unsigned long long>(a->workspace_bytes));
    return FW_ERR_WORKSPACE;
  }
  if (a->kv_cache == nullptr || a->seqused_k == nullptr || a->block_table == nullptr) {
    set_error("kv_cache, seqused_k and block_table must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  const int itemsize = a->kv_dtype == FW_DTYPE_BF16 ? 2 : 1;
  const int heads_per_word = itemsize == 1 ? 2 : 1;
  GatherParams gp;
  gp.pool = static_cast<const uint8_t*>(a->kv_cache);
  gp.block_table = a->block_table;
  gp.seqused = a->seqused_k;
  gp.num_active = a->num_active;
  gp.k_out = reinterpret_cast<__nv_bfloat16*>(ws + head + rope);
  gp.v_out = reinterpret_cast<__nv_bfloat16*>(ws + head + rope + plane);
  gp.status = reinterpret_cast<int*>(ws);
  gp.num_pages = a->num_pages;
  gp.batch = a->batch;
  gp.page_size = a->page_size;
  gp.pages_per_seq = a->pages_per_seq;
  gp.nheads_k = a->nheads_k;
  gp.cache_heads = 2 * ((a->nheads_k + heads_per_word - 1) / heads_per_word * heads_per_word);
  gp.head_dim = a->head_dim;
  gp.kv_dtype = a->kv_dtype;
  gather_kv_kernel<<<dim3(a->pages_per_seq, a->batch), 256, 0, stream>>>(gp);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("gather kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  // The same request table, now over packed bf16 K / V: request r's keys start
  // at row r * capacity, seqused_k still counts them.
  local.kv_cache = gp.k_out;
  local.v_packed = gp.v_out;
  local.block_table = nullptr;
  local.kv_dtype = FW_DTYPE_BF16;
  local.kv_token_major = 1;
  local.kv_request_stride = a->pages_per_seq * a->page_size;
  local.total_k = a->batch * local.kv_request_stride;
  local.workspace_bytes = head;
  return tcgen05_prefill(&local, stream);
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
    set_error("packed K/V attention is built for head_dim 64, 128 and 256 and nheads / nheads_k up to 128;"
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
  return ((tcgen05_prefill_workspace_bytes(a) + 255) & ~255ull) + packed_rope_k_bytes(a);
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
  if (a->rotary_cos != nullptr && a->rotary_k) {
    // Q is rotated inside the attention kernel.  K's token t of a request sits at
    // position t: rotate it into a scratch copy as a tensor whose rows are its own
    // keys (length = key count).
    const uint64_t need = head + packed_rope_k_bytes(a);
    if (a->workspace == nullptr || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
      set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
                static_cast<unsigned long long>(need), static_cast<unsigned long long>(a->workspace_bytes));
      return FW_ERR_WORKSPACE;
    }
    if (a->kv_cache == nullptr) {
      set_error("k must not be NULL.");
      return FW_ERR_BAD_SHAPE;
    }
    uint8_t* ws = static_cast<uint8_t*>(a->workspace);
    RopeParams rk;
    rk.q = static_cast<const __nv_bfloat16*>(a->kv_cache);
    rk.q_out = reinterpret_cast<__nv_bfloat16*>(ws + head);
    rk.cos = a->rotary_cos;
    rk.sin = a->rotary_sin;
    rk.cu = a->cu_seqlens_k;
    rk.seqused = nullptr;
    rk.cu_k = a->cu_seqlens_k;
    rk.tok_stride = a->kv_token_major ? static_cast<long long>(a->nheads_k) * a->head_dim : a->head_dim;
    rk.head_stride = a->kv_token_major ? a->head_dim : static_cast<long long>(a->total_k) * a->head_dim;
    rk.batch = a->batch;
    rk.total_q = a->total_k;
    rk.nheads = a->nheads_k;
    rk.rotary_len = a->rotary_len;
    rk.interleaved = a->rotary_interleaved;
    rk.table_bf16 = a->rotary_bf16;
    rk.head_dim = a->head_dim;
    rc = launch_rope(rk, a->total_k, stream);
    if (rc != FW_OK) return rc;
    local.kv_cache = rk.q_out;
    local.workspace_bytes = head;
  }
  return tcgen05_prefill(&local, stream);
}
