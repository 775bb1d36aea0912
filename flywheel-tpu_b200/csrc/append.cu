// Ragged append of packed new K/V rows into merged pages, and the standalone
// log-sum-exp merge of gathered partial states.
//
// append: one 16-byte chunk per thread, all tokens in parallel (the reference
// walks requests x pages serially, kernels/kv_append.py:32-113).  Token t of
// request r < num_active lands at position cache_seqlens[r] + t, page
// block_table[r, pos / page_size], slot pos % page_size, as whole merged rows
// [k0, v0, k1, v1, ...]; an fp8 pool with an odd head count gets its pad head
// zeroed.  Bits are moved, never values.
#include "common.cuh"

namespace fw {

struct AppendParams {
  uint8_t* pool;
  const uint8_t* k_new;
  const uint8_t* v_new;
  const int* cu;
  const int* cache_seqlens;
  const int* block_table;
  const int* num_active;
  long long num_pages;
  int page_size, pages_per_seq, batch, total_tokens, nheads_k, cache_heads;
  int plane_bytes, row_bytes;
};

__global__ void __launch_bounds__(256) append_kernel(const AppendParams p) {
  const int chunks_per_row = p.row_bytes >> 4;
  const int chunks_per_plane = p.plane_bytes >> 4;
  const long long total = static_cast<long long>(p.total_tokens) * chunks_per_row;
  const int n_active = p.num_active ? min(p.batch, max(0, *p.num_active)) : p.batch;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int tok = static_cast<int>(idx / chunks_per_row);
    const int within = static_cast<int>(idx - static_cast<long long>(tok) * chunks_per_row);
    // request owning packed row tok: largest r with cu[r] <= tok
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.cu[mid] <= tok) lo = mid; else hi = mid;
    }
    const int r = lo;
    if (r >= n_active || tok < p.cu[r] || tok >= p.cu[r + 1]) continue;
    const int pos = max(p.cache_seqlens[r], 0) + (tok - p.cu[r]);
    const int page_idx = pos / p.page_size;
    if (page_idx >= p.pages_per_seq) continue;
    const int page = p.block_table[static_cast<long long>(r) * p.pages_per_seq + page_idx];
    if (page < 0 || page >= p.num_pages) continue;
    const int plane = within / chunks_per_plane;       // merged head row: 2*h + is_v
    const int c = within - plane * chunks_per_plane;
    const int h = plane >> 1, is_v = plane & 1;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (h < p.nheads_k) {
      const uint8_t* src = (is_v ? p.v_new : p.k_new) +
                           (static_cast<long long>(tok) * p.nheads_k + h) * p.plane_bytes + (c << 4);
      val = *reinterpret_cast<const uint4*>(src);
    }
    uint8_t* dst = p.pool + (static_cast<long long>(page) * p.page_size + (pos - page_idx * p.page_size)) *
                                p.row_bytes + (static_cast<long long>(within) << 4);
    *reinterpret_cast<uint4*>(dst) = val;
  }
}

struct WritePagesParams {
  uint8_t* pool;
  const uint8_t* k_new;
  const uint8_t* v_new;
  const int* slices;
  const int* num_slices;
  long long cache_rows;
  int num_columns, total_tokens, nheads_k, plane_bytes, row_bytes;
};

// One block column per slice-table column; the blocks of a column stride over
// its (row, 16-byte chunk) pairs.
__global__ void __launch_bounds__(256) write_pages_kernel(const WritePagesParams p) {
  const int column = blockIdx.x;
  if (column >= min(*p.num_slices, p.num_columns)) return;
  const int cache_row0 = p.slices[column];
  const int new_row0 = p.slices[p.num_columns + column];
  const int length = p.slices[2 * p.num_columns + column];
  const int chunks_per_row = p.row_bytes >> 4, chunks_per_plane = p.plane_bytes >> 4;
  const long long total = static_cast<long long>(max(length, 0)) * chunks_per_row;
  for (long long idx = blockIdx.y * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.y) * blockDim.x) {
    const int r = static_cast<int>(idx / chunks_per_row);
    const int within = static_cast<int>(idx - static_cast<long long>(r) * chunks_per_row);
    const long long cache_row = static_cast<long long>(cache_row0) + r;
    const int tok = new_row0 + r;
    if (cache_row < 0 || cache_row >= p.cache_rows || tok < 0 || tok >= p.total_tokens) continue;
    const int plane = within / chunks_per_plane, c = within - plane * chunks_per_plane;
    const int h = plane >> 1, is_v = plane & 1;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (h < p.nheads_k)
      val = *reinterpret_cast<const uint4*>((is_v ? p.v_new : p.k_new) +
                                            (static_cast<long long>(tok) * p.nheads_k + h) * p.plane_bytes + (c << 4));
    *reinterpret_cast<uint4*>(p.pool + cache_row * p.row_bytes + (static_cast<long long>(within) << 4)) = val;
  }
}

struct MergeParams {
  const float* partial_out;
  const float* partial_lse;
  const float* sinks;
  __nv_bfloat16* out;
  float* lse;
  int parts, rows, nheads, lse_head_stride, lse_token_stride;
  long long stride_out, stride_lse;
  int head_dim;
};

// One warp per (token, head) row; a lane owns four columns of every
// 128-column block of the head (one block at head_dim 128, two at 256).
__global__ void __launch_bounds__(128) merge_kernel(const MergeParams p) {
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= p.rows) return;
  const int head = row % p.nheads, tok = row / p.nheads;
  const float sink = p.sinks ? p.sinks[head] : -INFINITY;
  float top = sink;
  for (int i = 0; i < p.parts; ++i) top = fmaxf(top, p.partial_lse[i * p.stride_lse + row]);
  float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
  const int blocks = p.head_dim / 128;
  float den = 0.f;
  if (top != -INFINITY) {
    for (int i = 0; i < p.parts; ++i) {
      const float l = p.partial_lse[i * p.stride_lse + row];
      if (l == -INFINITY) continue;
      const float w = __expf(l - top);
      den += w;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        if (nb >= blocks) break;
        const float4 o = *reinterpret_cast<const float4*>(
            p.partial_out + i * p.stride_out + static_cast<long long>(row) * p.head_dim + nb * 128 + lane * 4);
        acc[nb].x += o.x * w;
        acc[nb].y += o.y * w;
        acc[nb].z += o.z * w;
        acc[nb].w += o.w * w;
      }
    }
    if (sink != -INFINITY) den += __expf(sink - top);
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
  for (int nb = 0; nb < 2; ++nb) {
    if (nb >= blocks) break;
    uint2 packed;
    packed.x = pack_bf16(acc[nb].x * inv, acc[nb].y * inv);
    packed.y = pack_bf16(acc[nb].z * inv, acc[nb].w * inv);
    *reinterpret_cast<uint2*>(p.out + static_cast<long long>(row) * p.head_dim + nb * 128 + lane * 4) = packed;
  }
  if (p.lse != nullptr && lane == 0)
    p.lse[static_cast<long long>(head) * p.lse_head_stride + static_cast<long long>(tok) * p.lse_token_stride] =
        den > 0.f ? top + logf(den) : -INFINITY;
}

}  // namespace fw

using namespace fw;

extern "C" int fw_append_ragged(const FwAppendArgs* a, void* stream_ptr) {
  if (a == nullptr || a->kv_cache == nullptr || a->k_new == nullptr || a->v_new == nullptr ||
      a->cu_seqlens_q == nullptr || a->cache_seqlens == nullptr || a->block_table == nullptr) {
    set_error("kv_cache, k, v, cu_seqlens_q, cache_seqlens and block_table must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->kv_dtype != FW_DTYPE_BF16 && a->kv_dtype != FW_DTYPE_E4M3 && a->kv_dtype != FW_DTYPE_E5M2) {
    set_error("kv_dtype must be bf16, e4m3 or e5m2; got %d", a->kv_dtype);
    return FW_ERR_BAD_DTYPE;
  }
  if (a->batch <= 0 || a->nheads_k <= 0 || a->page_size <= 0 || a->pages_per_seq <= 0 || a->num_pages <= 0 ||
      a->total_tokens < 0) {
    set_error("batch, nheads_k, page_size, pages_per_seq and num_pages must be positive.");
    return FW_ERR_BAD_SHAPE;
  }
  const int itemsize = a->kv_dtype == FW_DTYPE_BF16 ? 2 : 1;
  if ((a->head_dim * itemsize) % 16) {
    set_error("head_dim * itemsize must be a multiple of 16 bytes; got head_dim %d.", a->head_dim);
    return FW_ERR_BAD_SHAPE;
  }
  if ((reinterpret_cast<uintptr_t>(a->kv_cache) & 15) || (reinterpret_cast<uintptr_t>(a->k_new) & 15) ||
      (reinterpret_cast<uintptr_t>(a->v_new) & 15)) {
    set_error("kv_cache, k and v must be 16-byte aligned.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->total_tokens == 0) return FW_OK;
  AppendParams p;
  p.pool = static_cast<uint8_t*>(a->kv_cache);
  p.k_new = static_cast<const uint8_t*>(a->k_new);
  p.v_new = static_cast<const uint8_t*>(a->v_new);
  p.cu = a->cu_seqlens_q;
  p.cache_seqlens = a->cache_seqlens;
  p.block_table = a->block_table;
  p.num_active = a->num_active;
  p.num_pages = a->num_pages;
  p.page_size = a->page_size;
  p.pages_per_seq = a->pages_per_seq;
  p.batch = a->batch;
  p.total_tokens = a->total_tokens;
  p.nheads_k = a->nheads_k;
  const int heads_per_word = itemsize == 1 ? 2 : 1;
  p.cache_heads = 2 * ((a->nheads_k + heads_per_word - 1) / heads_per_word * heads_per_word);
  p.plane_bytes = a->head_dim * itemsize;
  p.row_bytes = p.cache_heads * p.plane_bytes;
  const long long chunks = static_cast<long long>(a->total_tokens) * (p.row_bytes >> 4);
  const long long want = (chunks + 255) / 256, cap = static_cast<long long>(sm_count()) * 16;
  const int blocks = static_cast<int>(want < cap ? want : cap);
  append_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(p);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("append kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_write_kv_pages(const FwWritePagesArgs* a, void* stream_ptr) {
  if (a == nullptr || a->kv_cache == nullptr || a->k_new == nullptr || a->v_new == nullptr ||
      a->slices == nullptr || a->num_slices == nullptr) {
    set_error("kv_cache, k, v, slices and num_slices must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->kv_dtype != FW_DTYPE_BF16 && a->kv_dtype != FW_DTYPE_E4M3 && a->kv_dtype != FW_DTYPE_E5M2) {
    set_error("kv_dtype must be bf16, e4m3 or e5m2; got %d", a->kv_dtype);
    return FW_ERR_BAD_DTYPE;
  }
  if (a->nheads_k <= 0 || a->page_size <= 0 || a->num_pages <= 0 || a->num_columns < 0 || a->total_tokens < 0) {
    set_error("nheads_k, page_size and num_pages must be positive.");
    return FW_ERR_BAD_SHAPE;
  }
  const int itemsize = a->kv_dtype == FW_DTYPE_BF16 ? 2 : 1;
  if ((a->head_dim * itemsize) % 16) {
    set_error("head_dim * itemsize must be a multiple of 16 bytes; got head_dim %d.", a->head_dim);
    return FW_ERR_BAD_SHAPE;
  }
  if ((reinterpret_cast<uintptr_t>(a->kv_cache) & 15) || (reinterpret_cast<uintptr_t>(a->k_new) & 15) ||
      (reinterpret_cast<uintptr_t>(a->v_new) & 15)) {
    set_error("kv_cache, k and v must be 16-byte aligned.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->num_columns == 0 || a->total_tokens == 0) return FW_OK;
  WritePagesParams p;
  p.pool = static_cast<uint8_t*>(a->kv_cache);
  p.k_new = static_cast<const uint8_t*>(a->k_new);
  p.v_new = static_cast<const uint8_t*>(a->v_new);
  p.slices = a->slices;
  p.num_slices = a->num_slices;
  p.cache_rows = a->num_pages * a->page_size;
  p.num_columns = a->num_columns;
  p.total_tokens = a->total_tokens;
  p.nheads_k = a->nheads_k;
  const int heads_per_word = itemsize == 1 ? 2 : 1;
  const int cache_heads = 2 * ((a->nheads_k + heads_per_word - 1) / heads_per_word * heads_per_word);
  p.plane_bytes = a->head_dim * itemsize;
  p.row_bytes = cache_heads * p.plane_bytes;
  const long long chunks = static_cast<long long>(a->page_size) * (p.row_bytes >> 4);
  const int per_column = static_cast<int>(chunks / 1024 < 1 ? 1 : (chunks / 1024 > 16 ? 16 : chunks / 1024));
  dim3 grid(a->num_columns, per_column);
  write_pages_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream_ptr)>>>(p);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("page writer launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_lse_combine(const FwCombineArgs* a, void* stream_ptr) {
  if (a == nullptr || a->partial_out == nullptr || a->partial_lse == nullptr || a->out == nullptr) {
    set_error("partial_out, partial_lse and out must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->head_dim != 128 && a->head_dim != 256) {
    set_error("head_dim %d is not built; this library serves head_dim 128 and 256.", a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  if (a->parts <= 0 || a->rows < 0 || a->nheads <= 0) {
    set_error("parts and nheads must be positive, rows non-negative.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->rows == 0) return FW_OK;
  MergeParams p{a->partial_out, a->partial_lse, a->sinks, static_cast<__nv_bfloat16*>(a->out), a->lse,
                a->parts, a->rows, a->nheads, a->lse_head_stride, a->lse_token_stride,
                a->part_stride_out ? a->part_stride_out : static_cast<long long>(a->rows) * a->head_dim,
                a->part_stride_lse ? a->part_stride_lse : static_cast<long long>(a->rows), a->head_dim};
  merge_kernel<<<(a->rows + 3) / 4, 128, 0, static_cast<cudaStream_t>(stream_ptr)>>>(p);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("merge kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}
