// Split-KV decode over a paged (merged [k0,v0,k1,v1,...]) or contiguous KV
// cache with the new tokens' K/V append fused into the same launch, plus the
// log-sum-exp combine of the per-CTA partial states.
//
// Behaviour follows flash_attn_with_kvcache of the reference project
// (flywheel_tpu/softmax_attention/decode.py:189-625 and the kernel it calls,
// kernels/decode.py:463-1914): append at cache_seqlens[b] + t, bottom-right
// aligned causal / left-window mask, softcap before masking, sinks in the
// denominator only, out 0 / lse -inf (or the sink) for rows that see no key.
//
// Design (B200): the flattened list of 16-token KV tiles of all requests is cut
// into equal contiguous ranges, one per persistent CTA (one CTA per SM), so
// every SM streams the same number of bytes whatever the length distribution.
// A CTA owns up to 8 KV heads of its token rows: one producer warp walks the
// block table and issues one tiled TMA copy per 16-token stage (128-byte
// swizzle, token-major inside each 128-byte head segment, so ldmatrix is
// bank-conflict free), guarded by full/empty mbarriers with bounded waits.
// Consumer warp w owns one KV head (and one 16-row slice of its GQA query
// rows): QK^T and PV run on mma.sync m16n8k16 with the softmax state in
// registers (quad shuffles for row max / row sum), so each KV byte is read
// from HBM once and from shared memory once per 16 query rows.  fp8 pages are
// widened to f16 in registers straight out of ldmatrix.  Each (CTA, request)
// segment leaves an un-normalised (o, m, l) partial; the combine kernel merges
// the segments of a request, folds the sink and v_descale and writes bf16.
#include <mutex>

#include "common.cuh"
#include "exchange.cuh"

namespace fw {

constexpr int kTile = 16;          // smallest stage: tokens per MMA k-step; page sizes are multiples of it
#ifndef FW_BF16_MULTI_SLICE_STAGE_TOKENS
#define FW_BF16_MULTI_SLICE_STAGE_TOKENS 32  // bf16 stage size when two or more warps share a KV head (16 or 32)
#endif
#ifndef FW_VERIFY_STAGE_TOKENS
#define FW_VERIFY_STAGE_TOKENS 32  // fp8 stage size when two or more warps share a KV head (16, 32 or 64)
#endif
constexpr int kMaxStages = 8;
constexpr int kMaxConsumerWarps = 8;
constexpr int kMaxHeadDim = 256;   // head_dim 64 (bf16), 128 and 256 are built
constexpr int kMaxInlineBatch = 2048;  // requests whose tile counts fit the CTA-local scan

struct DecodeParams {
  const __nv_bfloat16* q;
  const uint8_t* k_new;
  const uint8_t* v_new;
  uint8_t* k_base;
  uint8_t* v_base;
  const int* cache_seqlens;
  const int* block_table;
  const int* cache_batch_idx;
  const int* num_active;
  const int* append_enable;  // NULL, or one device int: 0 = treat this call as if there were no new tokens
  const float* k_descale;
  float* part_o;
  float* part_ml;
  int* tile_prefix;  // (batch + 1) exclusive tile prefix, written by CTA (0, 0) for the combine
  int* status;
  long long num_pages;
  int page_size, pages_per_seq, batch, seqlen_q, nheads, nheads_k, group;
  int hpc, mt, nhg, ncta;
  int merged;
  int row_bytes;    // bytes of one token row of the tensor k_base points at
  int plane_bytes;  // head_dim * itemsize
  int spp;          // 128-byte segments per head plane
  int stages, stage_bytes;
  int tile;         // tokens per pipeline stage (16, 32 or 64)
  int head_dim;     // 64, 128 or 256
  int has_new, causal, window_left;
  int zero_pad_head;  // fp8 merged pool with an odd nheads_k: append zeroes the pad head
  float scale, softcap;
  // Item mode (chunked prefill through the split-KV kernel): "request" b is a
  // block of up to seqlen_q query tokens of packed request items[8b]; see
  // prefill_plan_kernel for the table.  NULL = plain decode.
  const int* items;
  long long q_tok_stride, q_head_stride;  // elements; q and out share them
  int total_q;
};

struct Span {
  int total, cache_len, first_tile, n_tiles;
  int kv_end;     // keys [0, kv_end) exist for this request / item
  int diag_base;  // query token t sits on diagonal diag_base + t
  int req;        // block-table row
  int q_row0;     // first packed q row
  int q_valid;    // query tokens that are real rows
};

__device__ __forceinline__ Span request_span(const DecodeParams& p, int b, int n_active) {
  Span s{0, 0, 0, 0, 0, 0, b, b * p.seqlen_q, p.seqlen_q};
  if (p.items != nullptr) {
    const int4 it = *reinterpret_cast<const int4*>(p.items + 8 * b);  // req, q_row0, q_valid, total
    const int kv_limit = p.items[8 * b + 4];
    s.req = it.x;
    s.q_row0 = it.y;
    s.q_valid = it.z;
    s.total = it.w;
    s.kv_end = p.causal ? min(it.w, kv_limit) : kv_limit;
    s.cache_len = s.kv_end;
    s.diag_base = s.total - p.seqlen_q;
    if (s.q_valid <= 0 || s.kv_end <= 0) return s;
    const int first_key = (p.window_left >= 0) ? max(0, s.diag_base - p.window_left) : 0;
    s.first_tile = first_key / p.tile;
    s.n_tiles = max(0, (s.kv_end + p.tile - 1) / p.tile - s.first_tile);
    return s;
  }
  if (b >= n_active) return s;
  int len = max(p.cache_seqlens[b], 0);
  s.cache_len = len;
  const bool has_new = p.has_new && (p.append_enable == nullptr || *p.append_enable != 0);
  s.total = len + (has_new ? p.seqlen_q : 0);
  s.kv_end = s.total;
  s.diag_base = s.total - p.seqlen_q;
  if (s.total <= 0) return s;
  int first_key = (p.window_left >= 0) ? max(0, s.total - p.seqlen_q - p.window_left) : 0;
  s.first_tile = first_key / p.tile;
  s.n_tiles = (s.total + p.tile - 1) / p.tile - s.first_tile;
  return s;
}

__device__ __forceinline__ int load_num_active(const DecodeParams& p) {
  return p.num_active ? min(p.batch, max(0, *p.num_active)) : p.batch;
}

// Exclusive prefix of per-request tile counts into pre[0..batch]; every thread
// of the block must call it.  pre lives in shared memory.
__device__ __forceinline__ void scan_tiles(const DecodeParams& p, int n_active, int* pre) {
  const int tid = threadIdx.x, nthreads = blockDim.x;
  for (int b = tid; b < p.batch; b += nthreads) pre[b + 1] = request_span(p, b, n_active).n_tiles;
  if (tid == 0) pre[0] = 0;
  __syncthreads();
  if (tid < 32) {
    int carry = 0;
    for (int base = 0; base < p.batch; base += 32) {
      int idx = base + tid;
      int v = idx < p.batch ? pre[idx + 1] : 0;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, v, off);
        if (tid >= off) v += n;
      }
      if (idx < p.batch) pre[idx + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
}

// Largest b with pre[b] <= f (f < pre[batch]).
__device__ __forceinline__ int find_request(const int* pre, int batch, int f) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    int mid = (lo + hi) >> 1;
    if (pre[mid] <= f) lo = mid; else hi = mid;
  }
  return lo;
}

__device__ __forceinline__ void cta_range(long long nt, int ncta, int cta, int& f0, int& f1) {
  f0 = static_cast<int>(nt * cta / ncta);
  f1 = static_cast<int>(nt * (cta + 1) / ncta);
}

// Segment index of head hl's K / V plane inside a stage, in units of
// (kTile * 128) bytes.
__device__ __forceinline__ int k_seg(const DecodeParams& p, int hl) {
  return p.merged ? 2 * hl * p.spp : hl * p.spp;
}
__device__ __forceinline__ int v_seg(const DecodeParams& p, int hl) {
  return p.merged ? (2 * hl + 1) * p.spp : (p.hpc + hl) * p.spp;
}

// D = head_dim.  At 256 a thread carries 128 output and 64 query registers, so
// the block is sized for four consumer warps instead of eight.
// Nine warps put three on one SM sub-partition (16384 registers each), which
// caps a thread at 168 registers; the launch bound tells the compiler so.
template <int KVT, int TILE, int D = 128>
__global__ void __launch_bounds__(((D > 128 ? kMaxConsumerWarps / 2 : kMaxConsumerWarps) + 1) * 32, 1)
decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
              const DecodeParams p) {
  constexpr bool kFp8 = KVT != FW_DTYPE_BF16;
  constexpr int NU = TILE / 16;  // 16-key MMA sub-tiles per stage
  constexpr int KS = D / 16;     // 16-wide k-steps over head_dim
  constexpr int ND = D / 8;      // 8-wide output column tiles
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.stages * p.stage_bytes);
  uint64_t* empty_bar = full_bar + kMaxStages;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kMaxStages);
  int* pre = const_cast<int*>(abort_flag) + 4;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, hg = blockIdx.y;
  const int heads_here = min(p.hpc, p.nheads_k - hg * p.hpc);
  const int consumer_warps = heads_here * p.mt;
  const int producer_warp = p.hpc * p.mt;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], consumer_warps);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  const int n_active = load_num_active(p);
  scan_tiles(p, n_active, pre);  // contains __syncthreads
  // the combine grid may be set up from here on; it still waits for this grid to finish
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const long long nt = pre[p.batch];
  if (cta == 0 && hg == 0)
    for (int i = threadIdx.x; i <= p.batch; i += blockDim.x) p.tile_prefix[i] = pre[i];
  int f0, f1;
  cta_range(nt, p.ncta, cta, f0, f1);
  if (f0 >= f1) return;

  // ------------------------------------------------------------ producer
  if (warp == producer_warp) {
    if (lane != 0) return;
    tma_prefetch_desc(&map_k);
    if (!p.merged) tma_prefetch_desc(&map_v);
    int stage = 0;
    uint32_t phase = 0;
    int issued = 0;
    bool ok = true;
    int b = find_request(pre, p.batch, f0);
    for (int f = f0; f < f1 && ok;) {
      while (pre[b + 1] <= f) ++b;
      const Span sp = request_span(p, b, n_active);
      const int seg_end = min(f1, pre[b + 1]);
      int cur_page_idx = -1, cur_page = 0;
      for (; f < seg_end; ++f) {
        const int pos0 = (f - pre[b] + sp.first_tile) * TILE;
        const int page_idx = pos0 / p.page_size;
        if (page_idx != cur_page_idx) {
          cur_page_idx = page_idx;
          // A position past the table row (or past a contiguous cache's capacity)
          // has no page: the table is not read there.
          int page = -1;
          if (page_idx < p.pages_per_seq)
            page = p.merged ? p.block_table[static_cast<long long>(sp.req) * p.pages_per_seq + page_idx]
                            : (p.cache_batch_idx ? p.cache_batch_idx[b] : b);
          if (page < 0 || page >= p.num_pages) {
            report_status(p.status, FW_STATUS_BAD_PAGE);
            page = 0;  // some page must be read; the result of this request is void
          }
          cur_page = page;
        }
        if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* dst = stage_base + stage * p.stage_bytes;
        mbar_arrive_expect_tx(&full_bar[stage], p.stage_bytes);
        const int tok = pos0 - page_idx * p.page_size;
        if (p.merged) {
          tma_load_4d(dst, &map_k, &full_bar[stage], 0, tok, hg * p.hpc * 2 * p.spp, cur_page);
        } else {
          tma_load_4d(dst, &map_k, &full_bar[stage], 0, tok, hg * p.hpc * p.spp, cur_page);
          tma_load_4d(dst + p.stage_bytes / 2, &map_v, &full_bar[stage], 0, tok,
                      hg * p.hpc * p.spp, cur_page);
        }
        ++issued;
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) {
      // A wait gave up: record it, tell the consumers, and let the copies that
      // are still in flight land before this CTA's shared memory goes away.
      *abort_flag = 1;
      report_status(p.status, FW_STATUS_WAIT_TIMEOUT);
      const int pending = min(issued, p.stages);
      for (int i = 0; i < pending; ++i) {
        if (stage == 0) {
          stage = p.stages;
          phase ^= 1;
        }
        --stage;
        for (uint32_t spin = 0; spin < (1u << 16) && !mbar_try_wait(&full_bar[stage], phase); ++spin) {
          __nanosleep(64);
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------ consumers
  if (warp >= consumer_warps) return;
  const int hl = warp / p.mt, mti = warp - hl * p.mt;
  const int h = hg * p.hpc + hl;             // KV head
  const int rows_per_head = p.seqlen_q * p.group;
  const int quad = lane >> 2, tq = lane & 3;
  const int row0 = mti * 16 + quad, row1 = row0 + 8;
  const bool row0_in = row0 < rows_per_head, row1_in = row1 < rows_per_head;
  const int t0 = row0 / p.group, g0 = row0 - t0 * p.group;
  const int t1 = row1 / p.group, g1 = row1 - t1 * p.group;
  const int rq = p.seqlen_q * p.nheads;      // partial rows per slot
  const int seg_bytes = TILE * 128;
  const uint32_t stage_u32 = smem_u32(stage_base);
  const int kseg = k_seg(p, hl), vseg = v_seg(p, hl);

  const float kd = p.k_descale ? *p.k_descale : 1.0f;
  const float c1 = p.softcap > 0.f ? p.scale * kd / p.softcap : p.scale * kd * kLog2e;
  const float c2 = p.softcap * kLog2e;

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  bool next_full = false;  // the stage of the coming tile was seen full (valid across requests: one ring)

  int b = find_request(pre, p.batch, f0);
  for (int f = f0; f < f1 && ok;) {
    while (pre[b + 1] <= f) ++b;
    const Span sp = request_span(p, b, n_active);
    const int seg_end = min(f1, pre[b + 1]);
    const bool row0_ok = row0_in && t0 < sp.q_valid, row1_ok = row1_in && t1 < sp.q_valid;

    // ---- Q fragments of this warp's 16 rows (zero for rows past the window)
    uint32_t qa[KS][4];
    {
      const __nv_bfloat16* q0 = p.q + (static_cast<long long>(sp.q_row0) + t0) * p.q_tok_stride +
                                static_cast<long long>(h * p.group + g0) * p.q_head_stride;
      const __nv_bfloat16* q1 = p.q + (static_cast<long long>(sp.q_row0) + t1) * p.q_tok_stride +
                                static_cast<long long>(h * p.group + g1) * p.q_head_stride;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        if constexpr (!kFp8) {
          const int d = ks * 16 + 2 * tq;
          qa[ks][0] = row0_ok ? *reinterpret_cast<const uint32_t*>(q0 + d) : 0u;
          qa[ks][1] = row1_ok ? *reinterpret_cast<const uint32_t*>(q1 + d) : 0u;
          qa[ks][2] = row0_ok ? *reinterpret_cast<const uint32_t*>(q0 + d + 8) : 0u;
          qa[ks][3] = row1_ok ? *reinterpret_cast<const uint32_t*>(q1 + d + 8) : 0u;
        } else {
          // fp8 K comes out of ldmatrix four consecutive head_dim elements per
          // thread, so the contraction index is permuted the same way here.
          const int d = ks * 16 + 4 * tq;
          uint2 v0 = row0_ok ? *reinterpret_cast<const uint2*>(q0 + d) : make_uint2(0u, 0u);
          uint2 v1 = row1_ok ? *reinterpret_cast<const uint2*>(q1 + d) : make_uint2(0u, 0u);
          auto to_f16 = [](uint32_t two_bf16) {
            float lo = __uint_as_float(two_bf16 << 16), hi = __uint_as_float(two_bf16 & 0xffff0000u);
            return pack_f16(lo, hi);
          };
          qa[ks][0] = to_f16(v0.x);
          qa[ks][1] = to_f16(v1.x);
          qa[ks][2] = to_f16(v0.y);
          qa[ks][3] = to_f16(v1.y);
        }
      }
    }
    float o[ND][4];
#pragma unroll
    for (int i = 0; i < ND; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // Bottom-right diagonals of the two rows this thread owns.
    const int diag0 = sp.diag_base + t0, diag1 = sp.diag_base + t1;

    for (; f < seg_end; ++f) {
      const int pos0 = (f - pre[b] + sp.first_tile) * TILE;
      // (the previous tile has usually seen this stage full already, under its PV MMAs)
      if (!next_full && !mbar_wait_bounded(&full_bar[stage], phase, abort_flag)) {
        ok = false;
        break;
      }
      const uint32_t st = stage_u32 + stage * p.stage_bytes;
      uint8_t* st_ptr = stage_base + stage * p.stage_bytes;

      // ---- boundary tile: patch in the new tokens (and write them to their
      // page), and zero V rows past the valid length so 0 * NaN never forms.
      if (pos0 + TILE > sp.cache_len) {
        const int chunks = p.plane_bytes >> 4;  // 16-byte chunks per head plane
        for (int tk = 0; tk < TILE; ++tk) {
          const int pos = pos0 + tk;
          if (pos < sp.cache_len) continue;
          const bool is_new = p.has_new && pos < sp.total;
          const int tnew = pos - sp.cache_len;
          uint8_t* gk = nullptr;
          uint8_t* gv = nullptr;
          if (is_new && mti == 0) {
            // The new row goes to its page only when that page exists: a table
            // entry outside the pool, or a position past the table row / the
            // contiguous capacity, is reported and nothing is stored (the row is
            // still attended from shared memory), so no other request's page is
            // ever overwritten.
            const int page_idx = pos / p.page_size;
            int page = -1;
            if (page_idx < p.pages_per_seq)
              page = p.merged ? p.block_table[static_cast<long long>(sp.req) * p.pages_per_seq + page_idx]
                              : (p.cache_batch_idx ? p.cache_batch_idx[b] : b);
            if (page < 0 || page >= p.num_pages) {
              if (lane == 0) report_status(p.status, FW_STATUS_BAD_PAGE);
            } else {
              const long long row = (static_cast<long long>(page) * p.page_size + (pos - page_idx * p.page_size)) *
                                    p.row_bytes;
              if (p.merged) {
                gk = p.k_base + row + static_cast<long long>(2 * h) * p.plane_bytes;
                gv = gk + p.plane_bytes;
              } else {
                gk = p.k_base + row + static_cast<long long>(h) * p.plane_bytes;
                gv = p.v_base + row + static_cast<long long>(h) * p.plane_bytes;
              }
            }
          }
          for (int i = lane; i < 2 * chunks; i += 32) {
            const int is_v = i >= chunks;
            const int c = is_v ? i - chunks : i;
            const int seg = (is_v ? vseg : kseg) + (c >> 3);
            uint4* dst = reinterpret_cast<uint4*>(st_ptr + seg * seg_bytes + tk * 128 +
                                                  (((c & 7) ^ (tk & 7)) << 4));
            if (is_new) {
              const uint8_t* src = (is_v ? p.v_new : p.k_new) +
                                   ((static_cast<long long>(b) * p.seqlen_q + tnew) * p.nheads_k + h) *
                                       p.plane_bytes + (c << 4);
              const uint4 val = *reinterpret_cast<const uint4*>(src);
              *dst = val;
              if (gk != nullptr) *reinterpret_cast<uint4*>((is_v ? gv : gk) + (c << 4)) = val;
              if (gk != nullptr && p.zero_pad_head && h == p.nheads_k - 1) {
                // the fp8 pad head sits right after the last real head's V plane
                *reinterpret_cast<uint4*>((is_v ? gv : gk) + 2 * p.plane_bytes + (c << 4)) =
                    make_uint4(0u, 0u, 0u, 0u);
              }
            } else if (is_v) {
              *dst = make_uint4(0u, 0u, 0u, 0u);
            }
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
      }

      // ---- S = Q K^T: NU sub-tiles of 16 keys (two 8-key n-tiles each), all
      // independent accumulators, so the MMAs of a stage pipeline.
      float s[NU][2][4];
#pragma unroll
      for (int u = 0; u < NU; ++u)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) s[u][nt][0] = s[u][nt][1] = s[u][nt][2] = s[u][nt][3] = 0.f;
      // The k-steps run outermost and the sub-tiles innermost, so consecutive
      // MMAs go to different accumulators (2 * NU chains in flight instead of two).
      if constexpr (!kFp8) {
        const int mi = lane >> 3;
        // A one-sub-tile stage would leave two chains of KS dependent MMAs: the
        // odd k-steps go to a second pair of accumulators, summed at the end.
        float s_odd[2][4];
        if constexpr (NU == 1) {
#pragma unroll
          for (int nt = 0; nt < 2; ++nt) s_odd[nt][0] = s_odd[nt][1] = s_odd[nt][2] = s_odd[nt][3] = 0.f;
        }
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
          for (int u = 0; u < NU; ++u) {
            const int key = u * 16 + ((mi >> 1) << 3) + (lane & 7);
            const int chunk = ks * 2 + (mi & 1);
            const uint32_t addr = st + (kseg + (chunk >> 3)) * seg_bytes + key * 128 +
                                  (((chunk & 7) ^ (key & 7)) << 4);
            uint32_t r0, r1, r2, r3;
            ldmatrix_x4(addr, r0, r1, r2, r3);
            if (NU == 1 && (ks & 1)) {
              mma_bf16(s_odd[0], qa[ks], r0, r1);
              mma_bf16(s_odd[1], qa[ks], r2, r3);
            } else {
              mma_bf16(s[u][0], qa[ks], r0, r1);
              mma_bf16(s[u][1], qa[ks], r2, r3);
            }
          }
        }
        if constexpr (NU == 1) {
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[0][nt][i] += s_odd[nt][i];
        }
      } else {
        const int mi = lane >> 3;
#pragma unroll
        for (int kp = 0; kp < KS / 2; ++kp) {
#pragma unroll
          for (int u = 0; u < NU; ++u) {
            const int key = u * 16 + ((mi & 1) << 3) + (lane & 7);
            const int chunk = kp * 2 + (mi >> 1);
            const uint32_t addr = st + (kseg + (chunk >> 3)) * seg_bytes + key * 128 +
                                  (((chunk & 7) ^ (key & 7)) << 4);
            uint32_t r0, r1, r2, r3;  // (keys 0-7, c), (keys 8-15, c), (keys 0-7, c+1), (keys 8-15, c+1)
            ldmatrix_x4(addr, r0, r1, r2, r3);
            mma_f16(s[u][0], qa[2 * kp], fp8_half_to_f16x2<KVT, false>(r0), fp8_half_to_f16x2<KVT, true>(r0));
            mma_f16(s[u][1], qa[2 * kp], fp8_half_to_f16x2<KVT, false>(r1), fp8_half_to_f16x2<KVT, true>(r1));
            mma_f16(s[u][0], qa[2 * kp + 1], fp8_half_to_f16x2<KVT, false>(r2), fp8_half_to_f16x2<KVT, true>(r2));
            mma_f16(s[u][1], qa[2 * kp + 1], fp8_half_to_f16x2<KVT, false>(r3), fp8_half_to_f16x2<KVT, true>(r3));
          }
        }
      }

      // ---- scale (+ softcap), mask.  With a softcap the logit is
      // c2 * tanh(s * c1) = c2 - 2 c2 / (2^(s * c1 * 2 log2e) + 1): the constants
      // are folded so a score costs mul, min, ex2, add, rcp, fma, and the
      // multiplies / adds run two scores per instruction (f32x2).
      if (p.softcap > 0.f) {
        const float a = c1 * (2.0f * kLog2e), m2c2 = -2.0f * c2;
        const uint64_t a2 = pack2(a, a), one2 = pack2(1.f, 1.f), m2c22 = pack2(m2c2, m2c2), c22 = pack2(c2, c2);
#pragma unroll
        for (int u = 0; u < NU; ++u)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; i += 2) {
              float x0, x1;
              unpack2(mul2(pack2(s[u][nt][i], s[u][nt][i + 1]), a2), x0, x1);
              const float e0 = fast_exp2(fminf(x0, 80.0f)), e1 = fast_exp2(fminf(x1, 80.0f));
              float d0, d1;
              unpack2(add2(pack2(e0, e1), one2), d0, d1);
              unpack2(fma2(pack2(fast_rcp(d0), fast_rcp(d1)), m2c22, c22), s[u][nt][i], s[u][nt][i + 1]);
            }
      } else {
#pragma unroll
        for (int u = 0; u < NU; ++u)
#pragma unroll
          for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) s[u][nt][i] *= c1;
      }
      const bool mask_right = pos0 + TILE > min(sp.diag_base, sp.kv_end);
      const bool mask_left = p.window_left >= 0 && pos0 < sp.total - 1 - p.window_left;
      if (mask_right || mask_left) {
#pragma unroll
        for (int u = 0; u < NU; ++u)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int j = pos0 + u * 16 + nt * 8 + 2 * tq + (i & 1);
            const int diag = (i < 2) ? diag0 : diag1;
            bool vis = j < sp.kv_end && (!p.causal || j <= diag);
            if (p.window_left >= 0) vis = vis && (j >= diag - p.window_left);
            if (!vis) s[u][nt][i] = -INFINITY;
          }
      }

      // ---- online softmax (rows quad and quad + 8); the subtraction of the row
      // base and the row sum run two scores per instruction
      float alpha[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float mx = -INFINITY;
#pragma unroll
        for (int u = 0; u < NU; ++u)
          mx = fmaxf(mx, fmaxf(fmaxf(s[u][0][2 * r], s[u][0][2 * r + 1]), fmaxf(s[u][1][2 * r], s[u][1][2 * r + 1])));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run[r], mx);
        const float base = m_new == -INFINITY ? 0.f : m_new;
        alpha[r] = fast_exp2(m_run[r] - base);
        m_run[r] = m_new;
        const uint64_t nbase2 = pack2(-base, -base);
        uint64_t sum2 = pack2(0.f, 0.f);
#pragma unroll
        for (int u = 0; u < NU; ++u)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          float y0, y1;
          unpack2(add2(pack2(s[u][nt][2 * r], s[u][nt][2 * r + 1]), nbase2), y0, y1);
          s[u][nt][2 * r] = fast_exp2(y0);
          s[u][nt][2 * r + 1] = fast_exp2(y1);
          sum2 = add2(sum2, pack2(s[u][nt][2 * r], s[u][nt][2 * r + 1]));
        }
        float sum_lo, sum_hi;
        unpack2(sum2, sum_lo, sum_hi);
        l_run[r] = l_run[r] * alpha[r] + (sum_lo + sum_hi);
      }
      if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          o[i][0] *= alpha[0];
          o[i][1] *= alpha[0];
          o[i][2] *= alpha[1];
          o[i][3] *= alpha[1];
        }
      }

      // Is the next stage full yet?  Asked here, without blocking, so that the
      // answer's latency hides under the PV MMAs instead of opening the next tile.
      {
        const int ns = stage + 1 == p.stages ? 0 : stage + 1;
        next_full = mbar_test_wait(&full_bar[ns], ns == 0 ? phase ^ 1 : phase);
      }
      // ---- O += P V, one 16-key k-step per sub-tile
#pragma unroll
      for (int u = 0; u < NU; ++u) {
      uint32_t pa[4];
      if constexpr (!kFp8) {
        pa[0] = pack_bf16(s[u][0][0], s[u][0][1]);
        pa[1] = pack_bf16(s[u][0][2], s[u][0][3]);
        pa[2] = pack_bf16(s[u][1][0], s[u][1][1]);
        pa[3] = pack_bf16(s[u][1][2], s[u][1][3]);
        const int mi = lane >> 3;
        const int key = u * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int cp = 0; cp < ND / 2; ++cp) {
          const int chunk = cp * 2 + (mi >> 1);
          const uint32_t addr = st + (vseg + (chunk >> 3)) * seg_bytes + key * 128 +
                                (((chunk & 7) ^ (key & 7)) << 4);
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4_trans(addr, r0, r1, r2, r3);
          mma_bf16(o[2 * cp], pa, r0, r1);
          mma_bf16(o[2 * cp + 1], pa, r2, r3);
        }
      } else {
        pa[0] = pack_f16(s[u][0][0], s[u][0][1]);
        pa[1] = pack_f16(s[u][0][2], s[u][0][3]);
        pa[2] = pack_f16(s[u][1][0], s[u][1][1]);
        pa[3] = pack_f16(s[u][1][2], s[u][1][3]);
        const int mi = lane >> 3;
        const int key = u * 16 + ((mi & 1) << 3) + (lane & 7);
#pragma unroll
        for (int cp = 0; cp < ND / 4; ++cp) {
          const int chunk = cp * 2 + (mi >> 1);
          const uint32_t addr = st + (vseg + (chunk >> 3)) * seg_bytes + key * 128 +
                                (((chunk & 7) ^ (key & 7)) << 4);
          uint32_t r0, r1, r2, r3;  // (keys 0-7, c), (keys 8-15, c), (keys 0-7, c+1), (keys 8-15, c+1)
          ldmatrix_x4_trans(addr, r0, r1, r2, r3);
          // Each register holds keys (2tq, 2tq+1) x head_dim (2u, 2u+1); regroup
          // to [even d: k0 k1 | odd d: k0 k1].
          r0 = __byte_perm(r0, 0, 0x3120);
          r1 = __byte_perm(r1, 0, 0x3120);
          r2 = __byte_perm(r2, 0, 0x3120);
          r3 = __byte_perm(r3, 0, 0x3120);
          mma_f16(o[4 * cp + 0], pa, fp8_half_to_f16x2<KVT, false>(r0), fp8_half_to_f16x2<KVT, false>(r1));
          mma_f16(o[4 * cp + 1], pa, fp8_half_to_f16x2<KVT, true>(r0), fp8_half_to_f16x2<KVT, true>(r1));
          mma_f16(o[4 * cp + 2], pa, fp8_half_to_f16x2<KVT, false>(r2), fp8_half_to_f16x2<KVT, false>(r3));
          mma_f16(o[4 * cp + 3], pa, fp8_half_to_f16x2<KVT, true>(r2), fp8_half_to_f16x2<KVT, true>(r3));
        }
      }
      }

      // Every lane's ldmatrix reads of this stage must be performed before lane 0
      // tells the producer the stage is free: without the fence the arrive could
      // overtake a read still in flight, and a stage refilled at once (a block
      // that waited for its slowest warp) was seen half old, half new - rarely,
      // by one warp, in one 16-column block of O.
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
      if (++stage == p.stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (!ok) break;

    // ---- partial state of this (CTA, request) segment
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    const long long slot = static_cast<long long>(b) + cta;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (!(r ? row1_ok : row0_ok)) continue;
      const int t = r ? t1 : t0, g = r ? g1 : g0;
      const long long prow = slot * rq + t * p.nheads + h * p.group + g;
      if (tq == 0) {
        p.part_ml[prow * 2] = m_run[r];
        p.part_ml[prow * 2 + 1] = l_run[r];
      }
      float* po = p.part_o + prow * D;
      if constexpr (!kFp8) {
#pragma unroll
        for (int nd = 0; nd < ND; ++nd)
          *reinterpret_cast<float2*>(po + nd * 8 + 2 * tq) = make_float2(o[nd][2 * r], o[nd][2 * r + 1]);
      } else {
#pragma unroll
        for (int c = 0; c < ND / 2; ++c)
          *reinterpret_cast<float4*>(po + c * 16 + 4 * tq) =
              make_float4(o[2 * c][2 * r], o[2 * c + 1][2 * r], o[2 * c][2 * r + 1], o[2 * c + 1][2 * r + 1]);
      }
    }
  }
  if (!ok && lane == 0) {
    *abort_flag = 1;
    report_status(p.status, FW_STATUS_WAIT_TIMEOUT);
  }
}

// ---------------------------------------------------------------- combine
struct CombineParams {
  DecodeParams d;
  __nv_bfloat16* out;
  float* lse;
  float* partial_out;
  float* partial_lse;
  const float* v_descale;
  const float* sinks;
  // xchg.world > 0: the sink-free normalised state of every row goes straight
  // into every rank's exchange buffer (peer stores over NVLink) as {value,
  // epoch} pairs instead of partial_out / partial_lse.
  PeerSlots xchg;
};

constexpr int kCombineWarps = 4;

// Merges the segments of (token, head) rows.  WPR warps share one row and split
// its segments between them: 1 when there are many rows with few segments
// each (serving batches), 16 when few rows have many segments (one long
// request cut over every SM).  Reads the tile prefix the decode kernel left in
// the workspace, so the two agree on which CTAs touched the request.
template <int WPR, int D>
__global__ void __launch_bounds__((WPR > kCombineWarps ? WPR : kCombineWarps) * 32)
combine_kernel(const CombineParams cp) {
  constexpr int kWarps = WPR > kCombineWarps ? WPR : kCombineWarps;  // warps per block
  constexpr int kRowsPerBlock = kWarps / WPR;
  // a lane owns four columns of every 128-column block; at head_dim 64 two columns of the one block
  constexpr int NB = D >= 128 ? D / 128 : 1;
  constexpr bool kNarrow = D < 128;
  const DecodeParams& p = cp.d;
  __shared__ float4 red_acc[kWarps][NB][32];
  __shared__ float red_den[kWarps], red_max[kWarps];
  const int b = blockIdx.x;
  const int warp_in_block = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = warp_in_block % WPR, warp = warp_in_block / WPR;
  // everything below reads what the decode kernel wrote
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // e.g. the state exchange
  const int n_active = load_num_active(p);
  const int before = p.tile_prefix[b];
  const int total_tiles = p.tile_prefix[p.batch];
  const Span sp = request_span(p, b, n_active);
  const int rq = p.seqlen_q * p.nheads;

  // CTAs [c_lo, c_hi] touched this request; the same for every row of it.
  int c_lo = 0, c_hi = -1;
  if (sp.n_tiles > 0) {
    const long long nt = total_tiles;
    const long long end = static_cast<long long>(before) + sp.n_tiles;
    c_lo = static_cast<int>(((before + 1LL) * p.ncta + nt - 1) / nt) - 1;
    c_hi = static_cast<int>((end * p.ncta + nt - 1) / nt) - 1;
    c_lo = max(c_lo, 0);
    c_hi = min(c_hi, p.ncta - 1);
    // The closed forms above are exact; the loops keep the two kernels in
    // agreement even if that ever changes.
    int f0, f1;
    for (cta_range(nt, p.ncta, c_lo, f0, f1); f1 <= before && c_lo < p.ncta - 1;) cta_range(nt, p.ncta, ++c_lo, f0, f1);
    for (cta_range(nt, p.ncta, c_hi, f0, f1); f0 >= end && c_hi > 0;) cta_range(nt, p.ncta, --c_hi, f0, f1);
  }
  // With at most 32 segments (every serving batch) which of them hold tiles is
  // worked out once per warp instead of once per row and segment.
  // (With at least one tile per CTA, every CTA holds tiles.)
  const bool all_live = total_tiles >= p.ncta;
  const bool few = c_hi - c_lo < 32;
  unsigned live = 0;
  if (few && !all_live) {
    bool has_tiles = false;
    if (c_lo + lane <= c_hi) {
      int f0, f1;
      cta_range(total_tiles, p.ncta, c_lo + lane, f0, f1);
      has_tiles = f1 > f0;
    }
    live = __ballot_sync(0xffffffffu, has_tiles);
  }
  const float vd = cp.v_descale ? *cp.v_descale : 1.0f;
  const bool scatter = cp.xchg.world > 0;
  const uint32_t epoch = scatter ? step_epoch(cp.xchg.peers[cp.xchg.rank]) : 0u;

  for (int row = blockIdx.y * kRowsPerBlock + warp; row < rq; row += gridDim.y * kRowsPerBlock) {
    const int t = row / p.nheads, hq = row - t * p.nheads;
    if (t >= sp.q_valid) {
      if (!scatter) break;  // rows are token-major: the rest are not real query rows either
      // the peers wait for every row of the step: a row that is no query row travels as the empty state
      if (sub == 0) {
        const long long orow = static_cast<long long>(b) * rq + row;
        for (int r = 0; r < cp.xchg.world; ++r) {
          uint2* slot = slot_of(cp.xchg.peers[r], epoch, cp.xchg.world, cp.xchg.rank, cp.xchg.slot_pairs);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            uint2* dst = slot + orow * D + nb * 128 + lane * 4;
            store_pairs2(dst, 0.f, 0.f, epoch);
            store_pairs2(dst + 2, 0.f, 0.f, epoch);
          }
          if (lane == 0) store_pair(slot + static_cast<long long>(p.total_q) * p.nheads * D + orow, -INFINITY, epoch);
        }
      }
      continue;
    }

    // One pass: every segment is folded into a running (max, sum, acc) state,
    // so a row costs one round of loads, not a max pass and then a sum pass.
    float m_max = -INFINITY;
    float4 acc[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) acc[nb] = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
#pragma unroll 4
    for (int c = c_lo + sub; c <= c_hi; c += WPR) {
      bool has_tiles = true;
      if (all_live) {
      } else if (few) {
        has_tiles = (live >> (c - c_lo)) & 1u;
      } else {
        int f0, f1;
        cta_range(total_tiles, p.ncta, c, f0, f1);
        has_tiles = f1 > f0;
      }
      const long long prow = (static_cast<long long>(b) + c) * rq + row;
      const float2 ml = *reinterpret_cast<const float2*>(p.part_ml + prow * 2);
      float4 o[NB];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        if constexpr (kNarrow) {
          const float2 two = *reinterpret_cast<const float2*>(p.part_o + prow * D + lane * 2);
          o[nb] = make_float4(two.x, two.y, 0.f, 0.f);
        } else {
          o[nb] = *reinterpret_cast<const float4*>(p.part_o + prow * D + nb * 128 + lane * 4);
        }
      }
      const float x = has_tiles ? ml.x : -INFINITY;  // a segment that saw no key carries -inf
      const float m_new = fmaxf(m_max, x);
      const float base = m_new == -INFINITY ? 0.f : m_new;
      const float keep = fast_exp2(m_max - base), w = fast_exp2(x - base);  // 2^-inf = 0
      den = den * keep + (w == 0.f ? 0.f : ml.y * w);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        acc[nb].x = acc[nb].x * keep + (w == 0.f ? 0.f : o[nb].x * w);
        acc[nb].y = acc[nb].y * keep + (w == 0.f ? 0.f : o[nb].y * w);
        acc[nb].z = acc[nb].z * keep + (w == 0.f ? 0.f : o[nb].z * w);
        acc[nb].w = acc[nb].w * keep + (w == 0.f ? 0.f : o[nb].w * w);
      }
      m_max = m_new;
    }
    if constexpr (WPR > 1) {
      // A block of the wide form holds one row, so its warps take every branch
      // of this loop together.  Their states merge like segments do.
      __syncthreads();
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) red_acc[warp_in_block][nb][lane] = acc[nb];
      if (lane == 0) {
        red_den[warp_in_block] = den;
        red_max[warp_in_block] = m_max;
      }
      __syncthreads();
      if (sub != 0) continue;
      float top = m_max;
#pragma unroll
      for (int w = 1; w < WPR; ++w) top = fmaxf(top, red_max[warp * WPR + w]);
      const float base = top == -INFINITY ? 0.f : top;
      const float keep = fast_exp2(m_max - base);
      den *= keep;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        acc[nb].x *= keep;
        acc[nb].y *= keep;
        acc[nb].z *= keep;
        acc[nb].w *= keep;
      }
#pragma unroll
      for (int w = 1; w < WPR; ++w) {
        const float scale = fast_exp2(red_max[warp * WPR + w] - base);
        if (scale == 0.f) continue;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          const float4 o = red_acc[warp * WPR + w][nb][lane];
          acc[nb].x += o.x * scale;
          acc[nb].y += o.y * scale;
          acc[nb].z += o.z * scale;
          acc[nb].w += o.w * scale;
        }
        den += red_den[warp * WPR + w] * scale;
      }
      m_max = top;
    }

    if (scatter) {
      // Sink-free normalised state, delivered to every rank (this one included).
      if constexpr (!kNarrow) {
        const long long orow = static_cast<long long>(b) * rq + row;
        const float inv = den > 0.f ? vd / den : 0.f;
        const float row_lse = den > 0.f ? (m_max + log2f(den)) * kLn2 : -INFINITY;
        for (int r = 0; r < cp.xchg.world; ++r) {
          uint2* slot = slot_of(cp.xchg.peers[r], epoch, cp.xchg.world, cp.xchg.rank, cp.xchg.slot_pairs);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            uint2* dst = slot + orow * D + nb * 128 + lane * 4;
            store_pairs2(dst, acc[nb].x * inv, acc[nb].y * inv, epoch);
            store_pairs2(dst + 2, acc[nb].z * inv, acc[nb].w * inv, epoch);
          }
          if (lane == 0) store_pair(slot + static_cast<long long>(p.total_q) * p.nheads * D + orow, row_lse, epoch);
        }
      }
      continue;
    }
    if (cp.partial_out != nullptr) {
      // Sink-free normalised state for a cross-GPU merge.
      const long long orow = static_cast<long long>(b) * rq + row;
      const float inv = den > 0.f ? 1.f / den : 0.f;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        if constexpr (kNarrow)
          *reinterpret_cast<float2*>(cp.partial_out + orow * D + lane * 2) =
              make_float2(acc[nb].x * inv * vd, acc[nb].y * inv * vd);
        else
          *reinterpret_cast<float4*>(cp.partial_out + orow * D + nb * 128 + lane * 4) = make_float4(
              acc[nb].x * inv * vd, acc[nb].y * inv * vd, acc[nb].z * inv * vd, acc[nb].w * inv * vd);
      }
      if (lane == 0) cp.partial_lse[orow] = den > 0.f ? (m_max + log2f(den)) * kLn2 : -INFINITY;
      continue;
    }

    // Fold the sink: it joins the denominator only.  Rows of requests past
    // num_active are not attention rows at all: out 0, lse -inf, sink or not.
    const bool live_request = p.items != nullptr || b < n_active;
    const float sink2 = cp.sinks && live_request ? cp.sinks[hq] * kLog2e : -INFINITY;
    const float m_all = fmaxf(m_max, sink2);
    float out_scale = 0.f, lse = -INFINITY;
    if (m_all != -INFINITY) {
      const float w_keys = m_max == -INFINITY ? 0.f : fast_exp2(m_max - m_all);
      const float den_all = den * w_keys + (sink2 == -INFINITY ? 0.f : fast_exp2(sink2 - m_all));
      if (den_all > 0.f) {
        out_scale = w_keys * vd / den_all;
        lse = (m_all + log2f(den_all)) * kLn2;
      }
    }
    const long long ooff = (static_cast<long long>(sp.q_row0) + t) * p.q_tok_stride +
                           static_cast<long long>(hq) * p.q_head_stride;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      uint2 packed;
      packed.x = pack_bf16(acc[nb].x * out_scale, acc[nb].y * out_scale);
      packed.y = pack_bf16(acc[nb].z * out_scale, acc[nb].w * out_scale);
      if constexpr (kNarrow) *reinterpret_cast<uint32_t*>(cp.out + ooff + lane * 2) = packed.x;
      else *reinterpret_cast<uint2*>(cp.out + ooff + nb * 128 + lane * 4) = packed;
    }
    if (cp.lse != nullptr && lane == 0) {
      if (p.items != nullptr)
        cp.lse[static_cast<long long>(hq) * p.total_q + sp.q_row0 + t] = lse;
      else
        cp.lse[(static_cast<long long>(b) * p.nheads + hq) * p.seqlen_q + t] = lse;
    }
  }
}

// ---------------------------------------------------------------- host
struct DecodePlan {
  DecodeParams p;
  int itemsize;
  int rows_q;
  long long slots;
  uint64_t off_prefix, off_ml, off_o, bytes;
  size_t smem;
};

static int plan_decode(const FwDecodeArgs* a, DecodePlan* plan, int max_batch = kMaxInlineBatch) {
  if (a == nullptr) {
    set_error("args is NULL");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->kv_dtype != FW_DTYPE_BF16 && a->kv_dtype != FW_DTYPE_E4M3 && a->kv_dtype != FW_DTYPE_E5M2) {
    set_error("kv_dtype must be bf16, e4m3 or e5m2; got %d", a->kv_dtype);
    return FW_ERR_BAD_DTYPE;
  }
  const bool paged = a->block_table != nullptr;
  if (a->batch <= 0 || a->seqlen_q <= 0) {
    set_error("batch and seqlen_q must be positive.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->nheads_k <= 0 || a->nheads <= 0 || a->nheads % a->nheads_k) {
    set_error("nheads=%d must be a multiple of nheads_k=%d.", a->nheads, a->nheads_k);
    return FW_ERR_BAD_SHAPE;
  }
  if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != kMaxHeadDim) {
    set_error("head_dim %d is not built; this library serves head_dim 64, 128 and 256.", a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  if (a->head_dim == 64 && a->kv_dtype != FW_DTYPE_BF16) {
    // a 64-element fp8 plane is 64 bytes: K and V of a head would share one 128-byte segment
    set_error("head_dim 64 is built for bfloat16 caches; fp8 caches take head_dim 128 or 256.");
    return FW_ERR_UNSUPPORTED;
  }
  if (paged) {
    if (a->v_cache != nullptr) {
      set_error("With block_table, pass one merged cache as kv_cache and v_cache=NULL.");
      return FW_ERR_BAD_SHAPE;
    }
    if (a->cache_batch_idx != nullptr) {
      set_error("block_table and cache_batch_idx are mutually exclusive.");
      return FW_ERR_BAD_SHAPE;
    }
    if (a->page_size <= 0 || a->page_size % kTile) {
      set_error("page_size must be a positive multiple of %d; got %d.", kTile, a->page_size);
      return FW_ERR_BAD_SHAPE;
    }
    if (a->pages_per_seq <= 0 || a->num_pages <= 0) {
      set_error("block_table must be (batch, max_pages_per_seq) over a non-empty pool.");
      return FW_ERR_BAD_SHAPE;
    }
  } else {
    if (a->v_cache == nullptr) {
      set_error("Without block_table, kv_cache and v_cache must be separate caches.");
      return FW_ERR_BAD_SHAPE;
    }
    if (a->kv_dtype != FW_DTYPE_BF16) {
      set_error("the contiguous K/V pair is bfloat16 only; fp8 needs the paged pool.");
      return FW_ERR_BAD_DTYPE;
    }
    if (a->seqlen_q != 1) {
      set_error("the contiguous K/V pair serves single-token decode only.");
      return FW_ERR_UNSUPPORTED;
    }
    if (a->page_size <= 0 || a->page_size % kTile || a->num_pages <= 0) {
      set_error("capacity must be a positive multiple of %d; got %d.", kTile, a->page_size);
      return FW_ERR_BAD_SHAPE;
    }
  }
  if ((a->k_new == nullptr) != (a->v_new == nullptr)) {
    set_error("k and v must be passed together, or both left out.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->softcap < 0.f) {
    set_error("softcap must be non-negative; got %f.", a->softcap);
    return FW_ERR_BAD_SHAPE;
  }
  if (a->window_left < -1) {
    set_error("window_left must be -1 (unbounded) or non-negative; got %d.", a->window_left);
    return FW_ERR_BAD_SHAPE;
  }
  if (a->batch > max_batch) {
    set_error("batch %d exceeds %d per call; split the batch.", a->batch, max_batch);
    return FW_ERR_UNSUPPORTED;
  }
  if ((a->partial_out == nullptr) != (a->partial_lse == nullptr)) {
    set_error("partial_out and partial_lse must be passed together.");
    return FW_ERR_BAD_SHAPE;
  }
  const int group = a->nheads / a->nheads_k;
  const int rows_per_head = a->seqlen_q * group;
  const int mt = (rows_per_head + 15) / 16;
  // head_dim 256 doubles the registers a warp needs; its block has four consumer warps.
  const int max_warps = a->head_dim > 128 ? kMaxConsumerWarps / 2 : kMaxConsumerWarps;
  if (mt > max_warps) {
    set_error("seqlen_q * (nheads / nheads_k) = %d exceeds %d query rows per KV head at head_dim %d.",
              rows_per_head, 16 * max_warps, a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  const int itemsize = a->kv_dtype == FW_DTYPE_BF16 ? 2 : 1;
  DecodeParams& p = plan->p;
  p = DecodeParams{};
  p.plane_bytes = a->head_dim * itemsize;
  p.spp = p.plane_bytes / 128;
  p.merged = paged ? 1 : 0;
  p.mt = mt;
  p.head_dim = a->head_dim;
  // Heads per CTA: as many as there are warps for, and no more than keep a
  // 16-token stage within 64 KiB.
  p.hpc = max(1, min(a->nheads_k, max_warps / mt));
  p.hpc = max(1, min(p.hpc, 64 * 1024 / (2 * p.spp * kTile * 128)));
  p.nhg = (a->nheads_k + p.hpc - 1) / p.hpc;
  const int heads_per_word = itemsize == 1 ? 2 : 1;
  const int cache_heads = paged ? 2 * ((a->nheads_k + heads_per_word - 1) / heads_per_word * heads_per_word)
                                : a->nheads_k;
  p.zero_pad_head = paged && cache_heads != 2 * a->nheads_k;
  p.row_bytes = cache_heads * p.plane_bytes;
  const int segs_per_stage = p.hpc * 2 * p.spp;
  // Stage size: 16 tokens for bf16 rows (64 KiB for 8 heads).  fp8 rows are half
  // as wide and cost twice the conversion work per byte, which makes the kernel
  // latency-bound rather than bound by bytes in flight: they take as many
  // tokens per stage as fit 64 KiB (up to 64) so each warp has independent
  // MMAs to pipeline.  (Registers allow one CTA per SM either way.)  The stage
  // must divide the page.
  p.tile = kTile;
  const int smem_for_stages = 200 * 1024;
  {
    // fp8: verify windows (two or more 16-row slices per head) measured best at 32.
    // bf16 with two or more slices per head is bound by its consumers too (every
    // byte feeds two warps' MMAs): 32-token stages halve the per-stage costs.
    const int max_tile = a->head_dim != 128 ? kTile
                         : itemsize == 1    ? (mt >= 2 ? FW_VERIFY_STAGE_TOKENS : 64)
                                            : (mt >= 2 ? FW_BF16_MULTI_SLICE_STAGE_TOKENS : kTile);
    while (p.tile < max_tile && segs_per_stage * (p.tile * 2) * 128 <= 64 * 1024 && a->page_size % (p.tile * 2) == 0)
      p.tile *= 2;
  }
  p.stage_bytes = segs_per_stage * p.tile * 128;
  // A block with few consumer warps (few KV heads on this GPU) must not take the
  // whole SM's shared memory for its ring: as many blocks share an SM as it
  // takes to put max_warps consumer warps there, each with at least two stages.
  const int share = max(1, min(max_warps / (p.hpc * mt), smem_for_stages / (2 * p.stage_bytes)));
  p.stages = min(kMaxStages, smem_for_stages / share / p.stage_bytes);
  if (p.stages < 2) {
    set_error("stage of %d bytes leaves fewer than two pipeline stages.", p.stage_bytes);
    return FW_ERR_UNSUPPORTED;
  }
  plan->smem = static_cast<size_t>(p.stages) * p.stage_bytes + 1024 /*alignment*/ +
               2 * kMaxStages * sizeof(uint64_t) + 16 + (a->batch + 1) * sizeof(int) + 64;
  // Small CTAs share an SM; size the grid so every SM is covered.
  const int threads = (p.hpc * p.mt + 1) * 32;
  int per_sm = min(static_cast<int>(220 * 1024 / plan->smem), 2048 / threads);
  per_sm = min(per_sm, 65536 / (threads * (a->head_dim > 128 ? 255 : 168)));  // registers per thread of the kernels
  per_sm = max(1, min(per_sm, 8));
  p.ncta = a->num_ctas > 0 ? a->num_ctas : max(1, sm_count() * per_sm / p.nhg);
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.k_new = static_cast<const uint8_t*>(a->k_new);
  p.v_new = static_cast<const uint8_t*>(a->v_new);
  p.k_base = static_cast<uint8_t*>(a->kv_cache);
  p.v_base = static_cast<uint8_t*>(paged ? a->kv_cache : a->v_cache);
  p.cache_seqlens = a->cache_seqlens;
  p.block_table = a->block_table;
  p.cache_batch_idx = a->cache_batch_idx;
  p.num_active = a->num_active;
  p.append_enable = a->k_new != nullptr ? a->append_enable : nullptr;
  p.k_descale = a->k_descale;
  p.num_pages = a->num_pages;
  p.page_size = a->page_size;
  p.pages_per_seq = paged ? a->pages_per_seq : 1;
  p.batch = a->batch;
  p.seqlen_q = a->seqlen_q;
  p.nheads = a->nheads;
  p.nheads_k = a->nheads_k;
  p.group = group;
  p.has_new = a->k_new != nullptr;
  p.causal = a->causal != 0;
  p.window_left = a->window_left;
  p.scale = a->softmax_scale;
  p.softcap = a->softcap;
  p.items = nullptr;
  p.q_tok_stride = static_cast<long long>(a->nheads) * a->head_dim;
  p.q_head_stride = a->head_dim;
  p.total_q = a->batch * a->seqlen_q;
  plan->itemsize = itemsize;
  plan->rows_q = a->seqlen_q * a->nheads;
  plan->slots = static_cast<long long>(a->batch) + p.ncta;
  plan->off_prefix = 256;
  plan->off_ml = (plan->off_prefix + (static_cast<uint64_t>(a->batch) + 1) * sizeof(int) + 255) & ~255ull;
  const uint64_t ml_bytes = static_cast<uint64_t>(plan->slots) * plan->rows_q * 2 * sizeof(float);
  plan->off_o = (plan->off_ml + ml_bytes + 255) & ~255ull;
  plan->bytes = plan->off_o + static_cast<uint64_t>(plan->slots) * plan->rows_q * a->head_dim * sizeof(float);
  return FW_OK;
}

}  // namespace fw

namespace fw {

// Enqueues decode_kernel + combine_kernel for a finished plan.
static int launch_decode(DecodePlan& plan, void* workspace, cudaStream_t stream, int kv_dtype, void* out,
                         float* lse, float* partial_out, float* partial_lse, const float* v_descale,
                         const float* sinks, int* status = nullptr, const PeerSlots* xchg = nullptr) {
  int rc;
  DecodeParams& p = plan.p;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  p.status = status != nullptr ? status : reinterpret_cast<int*>(ws);  // by default the head of the workspace
  p.tile_prefix = reinterpret_cast<int*>(ws + plan.off_prefix);
  p.part_ml = reinterpret_cast<float*>(ws + plan.off_ml);
  p.part_o = reinterpret_cast<float*>(ws + plan.off_o);

  // Tensor maps: bytes (128) x tokens-in-page x 128-byte segments x pages, so a
  // stage lands token-major inside each head segment.
  CUtensorMap map_k, map_v;
  const uint64_t segs = static_cast<uint64_t>(p.row_bytes) / 128;
  const uint64_t dims[4] = {128, static_cast<uint64_t>(p.page_size), segs, static_cast<uint64_t>(p.num_pages)};
  const uint64_t strides[3] = {static_cast<uint64_t>(p.row_bytes), 128,
                               static_cast<uint64_t>(p.page_size) * p.row_bytes};
  const uint32_t box[4] = {128, static_cast<uint32_t>(p.tile),
                           static_cast<uint32_t>(p.merged ? p.hpc * 2 * p.spp : p.hpc * p.spp), 1};
  rc = encode_tensor_map_u8_4d(&map_k, p.k_base, dims, strides, box);
  if (rc != FW_OK) return rc;
  rc = encode_tensor_map_u8_4d(&map_v, p.v_base, dims, strides, box);
  if (rc != FW_OK) return rc;

  using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const DecodeParams);
  Kernel kernel = nullptr;
  if (p.head_dim == kMaxHeadDim) {
    if (kv_dtype == FW_DTYPE_BF16) {
      kernel = decode_kernel<FW_DTYPE_BF16, 16, 256>;
    } else if (kv_dtype == FW_DTYPE_E4M3) {
      kernel = decode_kernel<FW_DTYPE_E4M3, 16, 256>;
    } else {
      kernel = decode_kernel<FW_DTYPE_E5M2, 16, 256>;
    }
  } else if (p.head_dim == 64) {
    kernel = decode_kernel<FW_DTYPE_BF16, 16, 64>;
  } else if (kv_dtype == FW_DTYPE_BF16) {
    kernel = p.tile == 32 ? decode_kernel<FW_DTYPE_BF16, 32> : decode_kernel<FW_DTYPE_BF16, 16>;
  } else if (kv_dtype == FW_DTYPE_E4M3) {
    kernel = p.tile == 64   ? decode_kernel<FW_DTYPE_E4M3, 64>
             : p.tile == 32 ? decode_kernel<FW_DTYPE_E4M3, 32>
                            : decode_kernel<FW_DTYPE_E4M3, 16>;
  } else {
    kernel = p.tile == 64   ? decode_kernel<FW_DTYPE_E5M2, 64>
             : p.tile == 32 ? decode_kernel<FW_DTYPE_E5M2, 32>
                            : decode_kernel<FW_DTYPE_E5M2, 16>;
  }
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(plan.smem));
  if (err != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%zu bytes): %s", plan.smem, cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  dim3 grid(p.ncta, p.nhg);
  dim3 block((p.hpc * p.mt + 1) * 32);
  kernel<<<grid, block, plan.smem, stream>>>(map_k, map_v, p);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("decode kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  CombineParams cp;
  cp.d = p;
  cp.out = static_cast<__nv_bfloat16*>(out);
  cp.lse = lse;
  cp.partial_out = partial_out;
  cp.partial_lse = partial_lse;
  cp.v_descale = v_descale;
  cp.sinks = sinks;
  cp.xchg = xchg != nullptr ? *xchg : PeerSlots{};
  // Few rows with many segments each (a long request cut over every SM): 16
  // warps share a row, so its ~150 segments are read in a few rounds.
  const bool wide = static_cast<long long>(p.batch) * plan.rows_q <= 2048;
  const bool d256 = p.head_dim == kMaxHeadDim, d64 = p.head_dim == 64;
  // The combine is launched as a programmatic dependent of the decode kernel:
  // its grid is set up while the decode kernel still runs and its blocks wait
  // (griddepcontrol.wait) for the decode grid to complete and flush, which
  // takes the launch latency out of the step.
  cudaLaunchAttribute pdl{};
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  if (wide) {
    cfg.gridDim = dim3(p.batch, plan.rows_q);
    cfg.blockDim = dim3(16 * 32);
    if (d256)
      cudaLaunchKernelEx(&cfg, combine_kernel<16, 256>, cp);
    else if (d64)
      cudaLaunchKernelEx(&cfg, combine_kernel<16, 64>, cp);
    else
      cudaLaunchKernelEx(&cfg, combine_kernel<16, 128>, cp);
  } else {
    // Each warp walks several rows of its request, so the per-request
    // bookkeeping is paid once per warp; enough blocks to fill the machine.
    const int blocks_per_request = (plan.rows_q + kCombineWarps - 1) / kCombineWarps;
    const int wanted = (8 * sm_count() + p.batch - 1) / p.batch;
    cfg.gridDim = dim3(p.batch, max(1, min(blocks_per_request, wanted)));
    cfg.blockDim = dim3(kCombineWarps * 32);
    if (d256)
      cudaLaunchKernelEx(&cfg, combine_kernel<1, 256>, cp);
    else if (d64)
      cudaLaunchKernelEx(&cfg, combine_kernel<1, 64>, cp);
    else
      cudaLaunchKernelEx(&cfg, combine_kernel<1, 128>, cp);
  }
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("combine kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

}  // namespace fw

using namespace fw;

extern "C" uint64_t fw_decode_workspace_bytes(const FwDecodeArgs* args) {
  DecodePlan plan;
  if (plan_decode(args, &plan) != FW_OK) return 0;
  return plan.bytes;
}

extern "C" int fw_decode_kvcache(const FwDecodeArgs* a, void* stream_ptr) {
  return fw::decode_with_status(a, nullptr, static_cast<cudaStream_t>(stream_ptr));
}

// fw_decode_kvcache; `status` (or NULL = the head of the workspace) is where the
// kernels report.  A caller that runs several kernels on one workspace gives
// them one status word.
int fw::decode_with_status(const FwDecodeArgs* a, int* status, cudaStream_t stream) {
  DecodePlan plan;
  int rc = plan_decode(a, &plan);
  if (rc != FW_OK) return rc;
  if (a->q == nullptr || a->kv_cache == nullptr || a->cache_seqlens == nullptr ||
      (a->out == nullptr && a->partial_out == nullptr)) {
    set_error("q, kv_cache, cache_seqlens and out must be device pointers, not NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->workspace == nullptr || a->workspace_bytes < plan.bytes ||
      (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
    set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
              static_cast<unsigned long long>(plan.bytes), static_cast<unsigned long long>(a->workspace_bytes));
    return FW_ERR_WORKSPACE;
  }
  if ((reinterpret_cast<uintptr_t>(a->kv_cache) & 15) || (reinterpret_cast<uintptr_t>(a->v_cache) & 15) ||
      (reinterpret_cast<uintptr_t>(a->q) & 15) || (reinterpret_cast<uintptr_t>(a->k_new) & 15) ||
      (reinterpret_cast<uintptr_t>(a->v_new) & 15) || (reinterpret_cast<uintptr_t>(a->out) & 15)) {
    set_error("q, out, caches and new k/v must be 16-byte aligned.");
    return FW_ERR_BAD_SHAPE;
  }
  return launch_decode(plan, a->workspace, stream, a->kv_dtype, a->out, a->lse, a->partial_out, a->partial_lse,
                       a->v_descale, a->sinks, status);
}

// One request whose pages are split over the GPUs of a node, the whole step:
// decode kernel over this rank's pages, combine kernel that delivers the rank's
// sink-free state to every rank's exchange buffer, merge kernel that waits for
// all ranks' states and writes the final rows.  Three launches, no flag, fence
// or collective call.
extern "C" int fw_sharded_decode_step(const FwShardedDecodeArgs* s, void* stream_ptr) {
  if (s == nullptr || s->peer_buffers == nullptr) {
    set_error("args and peer_buffers must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  const FwDecodeArgs* a = &s->decode;
  if (s->world <= 0 || s->world > kMaxRanks || s->rank < 0 || s->rank >= s->world) {
    set_error("world must be in [1, %d] and rank inside it; got world %d rank %d.", kMaxRanks, s->world, s->rank);
    return FW_ERR_BAD_SHAPE;
  }
  if (a->head_dim != 128 && a->head_dim != 256) {
    set_error("the state exchange serves head_dim 128 and 256; got %d.", a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  if (a->batch != 1 && a->seqlen_q != 1) {
    set_error("the sharded step takes one request (any seqlen_q) or one-token requests; got batch %d, seqlen_q %d.",
              a->batch, a->seqlen_q);
    return FW_ERR_UNSUPPORTED;
  }
  if (a->partial_out != nullptr || a->partial_lse != nullptr) {
    set_error("partial_out / partial_lse must be NULL: the state goes to the exchange buffers.");
    return FW_ERR_BAD_SHAPE;
  }
  if (s->global_len != nullptr && (s->local_len == nullptr || s->append_enable == nullptr || s->advance < 0)) {
    set_error("global_len needs local_len and append_enable, and advance >= 0.");
    return FW_ERR_BAD_SHAPE;
  }
  DecodePlan plan;
  int rc = plan_decode(a, &plan);
  if (rc != FW_OK) return rc;
  if (a->q == nullptr || a->kv_cache == nullptr || a->cache_seqlens == nullptr ||
      (a->out == nullptr && !s->deliver_only)) {
    set_error("q, kv_cache, cache_seqlens and out must be device pointers, not NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->workspace == nullptr || a->workspace_bytes < plan.bytes ||
      (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
    set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
              static_cast<unsigned long long>(plan.bytes), static_cast<unsigned long long>(a->workspace_bytes));
    return FW_ERR_WORKSPACE;
  }
  if ((reinterpret_cast<uintptr_t>(a->kv_cache) & 15) || (reinterpret_cast<uintptr_t>(a->q) & 15) ||
      (reinterpret_cast<uintptr_t>(a->k_new) & 15) || (reinterpret_cast<uintptr_t>(a->v_new) & 15) ||
      (reinterpret_cast<uintptr_t>(a->out) & 15)) {
    set_error("q, out, the cache and new k/v must be 16-byte aligned.");
    return FW_ERR_BAD_SHAPE;
  }
  const int rows = a->batch * a->seqlen_q * a->nheads;
  MergeParams m{};
  for (int r = 0; r < s->world; ++r) {
    if (s->peer_buffers[r] == nullptr) {
      set_error("peer_buffers[%d] is NULL.", r);
      return FW_ERR_BAD_SHAPE;
    }
    m.slots.peers[r] = static_cast<uint8_t*>(s->peer_buffers[r]);
  }
  m.slots.world = s->world;
  m.slots.rank = s->rank;
  m.slots.slot_pairs = slot_pairs_of(rows, a->head_dim);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  // the sink joins once, at the merge; v_descale scales this rank's state
  rc = launch_decode(plan, a->workspace, stream, a->kv_dtype, nullptr, nullptr, nullptr, nullptr, a->v_descale,
                     nullptr, nullptr, &m.slots);
  if (rc != FW_OK || s->deliver_only) return rc;
  m.sinks = a->sinks;
  m.out = static_cast<__nv_bfloat16*>(a->out);
  m.lse = a->lse;
  m.status = static_cast<int*>(a->workspace);
  m.rows = rows;
  m.nheads = a->nheads;
  m.head_dim = a->head_dim;
  // lse is (batch, nheads, seqlen_q); a merge row is (token, head) with token = b * seqlen_q + t
  m.lse_head_stride = a->batch == 1 ? a->seqlen_q : 1;
  m.lse_token_stride = a->batch == 1 ? 1 : a->nheads;
  m.global_len = s->global_len;
  m.local_len = s->local_len;
  m.append_enable = s->append_enable;
  m.page_size = a->page_size;
  m.advance = s->advance;
  return launch_gather_merge(m, stream);
}

// ---------------------------------------------------------------- split-KV prefill
// Chunked prefill through the split-KV kernel: each packed request is cut into
// blocks of qb = 128 / group query tokens ("items"); an item is to the decode
// kernel what a request with a qb-token verify window is, with its own causal
// diagonal.  Right for short chunks over long prefixes (the work is KV
// streaming); long chunks go to the tensor-core prefill kernel.
namespace fw {

constexpr int kMaxItems = 8192;
constexpr int kSortBuckets = 2048;

struct PrefillPlanParams {
  const int* cu;
  const int* cu_k;     // packed K/V: request r's keys are rows [cu_k[r], cu_k[r + 1]); else NULL
  int kv_stride;       // packed K/V in fixed slots: request r's keys start at row r * kv_stride
  const int* seqused;  // paged: request r's key count
  const int* num_active;
  const int* first_request;  // NULL, or requests below this one get no query blocks
  int* items;
  int* status;  // status block of the launch that follows, or NULL
  __nv_bfloat16* out;
  float* lse;
  long long tok_stride, head_stride;
  int batch, qb, max_items, total_q, nheads, causal, head_dim;
  int right;  // right reach of the mask for the sort key: 0 causal, > 0 a window, -1 none
};

// Block 0 writes the item table {request, first q row, valid tokens, diagonal
// anchor, kv length} (8 ints per item, zero past the last item); all blocks
// clear the packed rows that belong to no active request (out 0, lse -inf).
__global__ void __launch_bounds__(256) prefill_plan_kernel(const PrefillPlanParams pp) {
  __shared__ int off[kMaxInlineBatch + 1];
  __shared__ int bucket[kSortBuckets];
  // the attention kernel behind this one may be set up now; it waits for this grid to finish
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int n_active = pp.num_active ? min(pp.batch, max(0, *pp.num_active)) : pp.batch;
  auto used_of = [&](int r) { return pp.cu_k ? max(0, pp.cu_k[r + 1] - pp.cu_k[r]) : pp.seqused[r]; };
  if (blockIdx.x == 0) {
    // nothing an earlier launch reported may switch the coming one off
    if (threadIdx.x == 0 && pp.status != nullptr) pp.status[kStatusLaunchVoidWord] = 0;
    const int first = pp.first_request ? min(n_active, max(0, *pp.first_request)) : 0;
    for (int r = threadIdx.x; r < pp.batch; r += blockDim.x) {
      const int c = r >= first && r < n_active ? max(0, pp.cu[r + 1] - pp.cu[r]) : 0;
      off[r + 1] = (c + pp.qb - 1) / pp.qb;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      off[0] = 0;
      for (int r = 0; r < pp.batch; ++r) off[r + 1] += off[r];
    }
    __syncthreads();
    const int n_items = min(off[pp.batch], pp.max_items);
    // Items are laid out longest key range first (a counting sort on the key
    // count in 64-token buckets): CTAs are dispatched in item order, and the
    // long ones must not be the last to start.
    for (int i = threadIdx.x; i < kSortBuckets; i += blockDim.x) bucket[i] = 0;
    __syncthreads();
    auto key_of = [&](int r, int j, int c, int used) {
      const int anchor = used - c + (j + 1) * pp.qb;
      const int kv_end = pp.right >= 0 ? min(anchor + pp.right, used) : used;
      return kSortBuckets - 1 - min(max(kv_end, 0) >> 6, kSortBuckets - 1);  // long ranges get small keys
    };
    for (int r = threadIdx.x; r < pp.batch; r += blockDim.x) {
      const int blocks = off[r + 1] - off[r];
      const int c = blocks ? pp.cu[r + 1] - pp.cu[r] : 0, used = blocks ? used_of(r) : 0;
      for (int j = 0; j < blocks; ++j)
        if (off[r] + j < pp.max_items) atomicAdd(&bucket[key_of(r, j, c, used)], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int i = 0; i < kSortBuckets; ++i) {
        const int n = bucket[i];
        bucket[i] = run;
        run += n;
      }
    }
    __syncthreads();
    for (int r = threadIdx.x; r < pp.batch; r += blockDim.x) {
      const int blocks = off[r + 1] - off[r];
      if (blocks == 0) continue;
      const int c = pp.cu[r + 1] - pp.cu[r];
      const int used = used_of(r);
      for (int j = 0; j < blocks; ++j) {
        if (off[r] + j >= pp.max_items) break;
        const int idx = atomicAdd(&bucket[key_of(r, j, c, used)], 1);
        int* it = pp.items + 8 * idx;
        it[0] = r;
        it[1] = pp.cu[r] + j * pp.qb;
        it[2] = min(pp.qb, c - j * pp.qb);
        it[3] = used - c + (j + 1) * pp.qb;  // token t of the block sits on diagonal it[3] - qb + t
        it[4] = used;
        it[5] = pp.cu_k ? pp.cu_k[r] : r * pp.kv_stride;  // first key row of a packed request
        it[6] = it[7] = 0;
      }
    }
    for (int idx = n_items + threadIdx.x; idx < pp.max_items; idx += blockDim.x) {
      int* it = pp.items + 8 * idx;
#pragma unroll
      for (int k = 0; k < 8; ++k) it[k] = 0;
    }
  }
  const int pad_start = min(max(pp.cu[n_active], 0), pp.total_q);
  const long long pad_rows = pp.total_q - pad_start;
  const long long chunks = pad_rows * pp.nheads * (pp.head_dim / 8);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < chunks;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % (pp.head_dim / 8));
    const long long rh = i / (pp.head_dim / 8);
    const int hq = static_cast<int>(rh % pp.nheads);
    const long long row = pad_start + rh / pp.nheads;
    *reinterpret_cast<uint4*>(pp.out + row * pp.tok_stride + hq * pp.head_stride + c * 8) =
        make_uint4(0u, 0u, 0u, 0u);
    if (c == 0 && pp.lse != nullptr) pp.lse[static_cast<long long>(hq) * pp.total_q + row] = -INFINITY;
  }
}

int launch_prefill_plan(const FwPrefillArgs* a, int qb, int max_items, int* items, long long tok_stride,
                        long long head_stride, int* status, cudaStream_t stream) {
  if (a->batch > kMaxInlineBatch) {
    set_error("batch %d exceeds %d per call; split the batch.", a->batch, kMaxInlineBatch);
    return FW_ERR_UNSUPPORTED;
  }
  PrefillPlanParams pp;
  pp.cu = a->cu_seqlens_q;
  pp.cu_k = a->block_table == nullptr ? a->cu_seqlens_k : nullptr;
  pp.kv_stride = a->block_table == nullptr && a->cu_seqlens_k == nullptr ? a->kv_request_stride : 0;
  pp.seqused = a->seqused_k;
  pp.num_active = a->num_active;
  pp.first_request = a->first_request;
  pp.items = items;
  pp.status = status;
  pp.out = static_cast<__nv_bfloat16*>(a->out);
  pp.lse = a->lse;
  pp.tok_stride = tok_stride;
  pp.head_stride = head_stride;
  pp.batch = a->batch;
  pp.qb = qb;
  pp.head_dim = a->head_dim;
  pp.max_items = max_items;
  pp.total_q = a->total_q;
  pp.nheads = a->nheads;
  pp.causal = a->causal != 0;
  pp.right = a->causal ? 0 : (a->block_table == nullptr && a->window_right > 0 ? a->window_right : -1);
  prefill_plan_kernel<<<min(sm_count(), 64), 256, 0, stream>>>(pp);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("prefill plan kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

struct SplitKvPrefillPlan {
  DecodePlan decode;
  int qb, max_items;
  uint64_t off_items, bytes;
};

static int plan_splitkv_prefill(const FwPrefillArgs* a, SplitKvPrefillPlan* sp) {
  if (a == nullptr) {
    set_error("args is NULL");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->batch <= 0 || a->total_q <= 0 || a->nheads <= 0 || a->nheads_k <= 0 || a->nheads % a->nheads_k) {
    set_error("batch, total_q must be positive and nheads=%d a multiple of nheads_k=%d.", a->nheads,
              a->nheads_k);
    return FW_ERR_BAD_SHAPE;
  }
  if (a->batch > kMaxInlineBatch) {
    set_error("batch %d exceeds %d per call; split the batch.", a->batch, kMaxInlineBatch);
    return FW_ERR_UNSUPPORTED;
  }
  const int group = a->nheads / a->nheads_k;
  if (group > 128) {
    set_error("nheads / nheads_k = %d exceeds 128 query heads per KV head.", group);
    return FW_ERR_UNSUPPORTED;
  }
  sp->qb = (a->head_dim > 128 ? 64 : 128) / group;  // query rows per KV head a decode block takes
  if (sp->qb < 1) {
    set_error("nheads / nheads_k = %d exceeds 64 query heads per KV head at head_dim %d.", group, a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  sp->max_items = (a->total_q + sp->qb - 1) / sp->qb + a->batch;
  if (sp->max_items > kMaxItems) {
    set_error("total_q %d makes %d query blocks; the split-KV prefill takes at most %d per call.", a->total_q,
              sp->max_items, kMaxItems);
    return FW_ERR_UNSUPPORTED;
  }
  FwDecodeArgs fa = {};
  fa.block_table = a->block_table != nullptr ? a->block_table : reinterpret_cast<const int32_t*>(16);
  fa.num_pages = a->num_pages;
  fa.page_size = a->page_size;
  fa.pages_per_seq = a->pages_per_seq;
  fa.batch = sp->max_items;
  fa.seqlen_q = sp->qb;
  fa.nheads = a->nheads;
  fa.nheads_k = a->nheads_k;
  fa.head_dim = a->head_dim;
  fa.kv_dtype = a->kv_dtype;
  fa.causal = a->causal;
  fa.window_left = a->window_left;
  fa.softmax_scale = a->softmax_scale;
  fa.softcap = a->softcap;
  int rc = plan_decode(&fa, &sp->decode, kMaxItems);
  if (rc != FW_OK) return rc;
  DecodeParams& p = sp->decode.p;
  p.k_base = p.v_base = static_cast<uint8_t*>(const_cast<void*>(a->kv_cache));
  p.block_table = a->block_table;
  p.k_descale = a->k_descale;
  p.total_q = a->total_q;
  if (a->token_major) {
    p.q_tok_stride = static_cast<long long>(a->nheads) * a->head_dim;
    p.q_head_stride = a->head_dim;
  } else {
    p.q_tok_stride = a->head_dim;
    p.q_head_stride = static_cast<long long>(a->total_q) * a->head_dim;
  }
  sp->off_items = (sp->decode.bytes + 255) & ~255ull;
  sp->bytes = sp->off_items + static_cast<uint64_t>(sp->max_items) * 8 * sizeof(int);
  return FW_OK;
}

uint64_t splitkv_prefill_workspace_bytes(const FwPrefillArgs* a) {
  SplitKvPrefillPlan sp;
  return plan_splitkv_prefill(a, &sp) == FW_OK ? sp.bytes : 0;
}

int splitkv_prefill(const FwPrefillArgs* a, cudaStream_t stream) {
  SplitKvPrefillPlan sp;
  int rc = plan_splitkv_prefill(a, &sp);
  if (rc != FW_OK) return rc;
  if (a->q == nullptr || a->out == nullptr || a->kv_cache == nullptr || a->cu_seqlens_q == nullptr ||
      a->seqused_k == nullptr || a->block_table == nullptr) {
    set_error("q, out, kv_cache, cu_seqlens_q, seqused_k and block_table must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->workspace == nullptr || a->workspace_bytes < sp.bytes || (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
    set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
              static_cast<unsigned long long>(sp.bytes), static_cast<unsigned long long>(a->workspace_bytes));
    return FW_ERR_WORKSPACE;
  }
  if ((reinterpret_cast<uintptr_t>(a->kv_cache) & 15) || (reinterpret_cast<uintptr_t>(a->q) & 15) ||
      (reinterpret_cast<uintptr_t>(a->out) & 15)) {
    set_error("q, out and the cache must be 16-byte aligned.");
    return FW_ERR_BAD_SHAPE;
  }
  DecodeParams& p = sp.decode.p;
  int* items = reinterpret_cast<int*>(static_cast<uint8_t*>(a->workspace) + sp.off_items);
  p.q = static_cast<const __nv_bfloat16*>(a->q);
  p.items = items;
  rc = launch_prefill_plan(a, sp.qb, sp.max_items, items, p.q_tok_stride, p.q_head_stride,
                           static_cast<int*>(a->workspace), stream);
  if (rc != FW_OK) return rc;
  return launch_decode(sp.decode, a->workspace, stream, a->kv_dtype, a->out, a->lse, nullptr, nullptr,
                       a->v_descale, a->sinks);
}

}  // namespace fw

// ---------------------------------------------------------------- static scratch
// Decode for callers that cannot allocate device memory.  The split-KV partial
// states live in a fixed array inside this library's device image instead of a
// caller-provided workspace.
namespace fw {

static __device__ __align__(256) unsigned char g_decode_static_scratch[FW_STATIC_SCRATCH_BYTES];

// The array's name is only a host-side handle; kernels need the device address,
// which differs per GPU.  Looked up once per device, with that device current.
static int static_scratch_address(void** address) {
  static std::mutex guard;
  static void* per_device[64] = {nullptr};
  int dev = -1;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess || dev < 0 || dev >= 64) {
    set_error("cudaGetDevice: %s (device %d)", cudaGetErrorString(err), dev);
    return FW_ERR_LAUNCH;
  }
  std::lock_guard<std::mutex> lock(guard);
  if (per_device[dev] == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      set_error("cudaGetSymbolAddress(static scratch) on device %d: %s", dev, cudaGetErrorString(err));
      return FW_ERR_LAUNCH;
    }
    per_device[dev] = ptr;
  }
  *address = per_device[dev];
  return FW_OK;
}

}  // namespace fw

extern "C" int fw_decode_kvcache_static(const FwDecodeArgs* a, void* stream_ptr) {
  DecodePlan plan;
  int rc = plan_decode(a, &plan);
  if (rc != FW_OK) return rc;
  if (plan.bytes > FW_STATIC_SCRATCH_BYTES) {
    set_error("this call needs %llu bytes of scratch; the built-in scratch holds %llu. Use fw_decode_kvcache "
              "with a caller workspace, or a smaller batch.",
              static_cast<unsigned long long>(plan.bytes),
              static_cast<unsigned long long>(FW_STATIC_SCRATCH_BYTES));
    return FW_ERR_WORKSPACE;
  }
  void* scratch = nullptr;
  rc = static_scratch_address(&scratch);
  if (rc != FW_OK) return rc;
  // The array keeps whatever the previous call left.  Only the status word has
  // to start at zero; every partial state the combine reads is rewritten by
  // this call's decode kernel first.
  cudaError_t err = cudaMemsetAsync(scratch, 0, 256, static_cast<cudaStream_t>(stream_ptr));
  if (err != cudaSuccess) {
    set_error("clearing the status word: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  FwDecodeArgs with_scratch = *a;
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = FW_STATIC_SCRATCH_BYTES;
  return fw_decode_kvcache(&with_scratch, stream_ptr);
}

// The status word of the built-in scratch on the current device.  It describes
// the most recent fw_decode_kvcache_static call there, which cleared it first.
extern "C" int fw_read_status_static(void* stream_ptr, int32_t* status) {
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != FW_OK) return rc;
  return fw_read_status(scratch, stream_ptr, status);
}
