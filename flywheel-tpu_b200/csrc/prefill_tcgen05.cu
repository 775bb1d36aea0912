// Chunked prefill over the paged merged bf16 cache on the 5th-generation tensor
// cores: QK^T and PV are tcgen05.mma with f32 accumulators in tensor memory,
// Q and the paged K/V tiles are staged by tiled (non-multicast) TMA copies.
//
// Follows the block_table branch of flash_attn_varlen_func in the reference
// project (flywheel_tpu/softmax_attention/prefill.py:437-661 and
// kernels/fwd_paged.py:331-1019): bottom-right aligned causal / left-window
// mask per packed request, softcap before masking, sinks in the denominator,
// out 0 / lse -inf for padding rows.  Fully masked KV tiles are never loaded.
//
// One CTA = one query block of one KV head: two "streams" of 128 rows, each
// (128 / group) tokens x the `group` query heads that share the KV head (rows
// ordered head-major), so every K/V tile is fetched from L2 once per 256 query
// rows.  KV advances in 128-key tiles (two 64-token boxes: pages of 64, or
// slices of larger pages) through a 2-stage TMA ring whose K and V halves are
// released separately.  Warp roles: warp 0 issues
// TMA, warp 1 owns tensor memory and issues the MMAs of both streams, warps
// 2-5 and 6-9 are the two softmax groups (one thread per row: tcgen05.ld of
// S, online softmax with lazy rescale, P written back over S in tensor memory
// as the A operand of the PV MMA), so one stream's softmax overlaps the other
// stream's MMAs.  One CTA per SM (192 KiB shared memory, all 512 TMEM columns).
#include "tcgen05.cuh"

namespace fw {

constexpr int kBN = 128;       // keys per KV tile
constexpr int kStreams = 2;     // 128-row query tiles per CTA, one softmax warp group each
constexpr int kKvStages = 2;
constexpr int kTmemCols = 512;  // per stream: O 128 columns, S 128 columns (P overwrites S)

constexpr int kSmemQ = 0;                      // streams x 2 halves x [128 rows][128 B]
constexpr int kSmemK = kStreams * 32768;       // stages x 2 halves x [128 keys][128 B]
constexpr int kSmemV = kSmemK + kKvStages * 32768;
constexpr int kSmemBar = kSmemV + kKvStages * 32768;
constexpr int kSmemBytes = kSmemBar + 256;
// fp8 pools: one more region behind the barriers, where TMA lands the fp8 K and V
// tiles ([128 keys][128 B] each) that the converter warps widen into the bf16
// operand buffers above.
constexpr int kSmemF8K = (kSmemBytes + 1023) & ~1023;  // swizzled TMA destinations sit on 1024-byte boundaries
constexpr int kSmemF8V = kSmemF8K + 16384;
constexpr int kSmemBytesFp8 = kSmemF8V + 16384;
static_assert(kSmemBytesFp8 <= 227 * 1024, "shared memory budget of the fp8 variant");
constexpr int kConverterWarps = 2;

struct Bars {
  uint64_t q_full;
  uint64_t k_full[kKvStages], v_full[kKvStages], k_empty[kKvStages], v_empty[kKvStages];
  uint64_t s_full[kStreams], p_full[kStreams], pv_done[kStreams];
  uint64_t drain;  // abort path: completion of the MMAs issued so far
  uint64_t q_rotated;  // rotary embedding: every softmax warp has rotated its rows of Q
  uint64_t f8k_full, f8k_empty, f8v_full, f8v_empty;  // fp8 pools: the staging tiles
  uint32_t tmem_base;
  int abort_flag;
};

// Tensor-memory columns of stream t: O at [256 t, 256 t + 128), S at
// [256 t + 128, 256 t + 256); P (bf16 pairs) overwrites the first 64 columns of S.
__device__ __forceinline__ uint32_t tmem_o(uint32_t base, int t) { return base + t * 256; }
__device__ __forceinline__ uint32_t tmem_s(uint32_t base, int t) { return base + t * 256 + 128; }

// D = head_dim, 128 or 64 (64 for packed K/V only).  Shared memory keeps the
// 128-wide layout either way: operands are stored as 64-element (128-byte) halves,
// and at 64 the second half of every tile simply stays unused.
//
// KVT = pool element type.  A bf16 pool is copied by TMA straight into the
// operand buffers.  An fp8 pool (e4m3 / e5m2, head_dim 128, paged) is read in
// place too: TMA lands each fp8 K and V tile in a staging buffer and two
// converter warps (10, 11) widen it - exactly: every fp8 value is a bf16 value -
// into the swizzled bf16 operand buffer the MMAs read, tile by tile, inside the
// kernel (the reference widens per block inside its kernel as well,
// kernels/fwd_paged.py:260-328).  The descales stay in the score scale and the
// output scale.
template <int D, int KVT = FW_DTYPE_BF16>
__global__ void __launch_bounds__(64 + kStreams * 128 + (KVT == FW_DTYPE_BF16 ? 0 : kConverterWarps * 32), 1)
prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                       const __grid_constant__ CUtensorMap map_v, const Tc05Params p) {
  constexpr bool kFp8 = KVT != FW_DTYPE_BF16;
  constexpr bool kF16 = kFp8;  // fp8 pools: Q, K, V and P go to the tensor core as f16 (bf16 pools: bf16)
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.y, h = blockIdx.x;  // heads vary fastest: items start longest first across all heads

  // An item is up to kStreams * tpb query tokens of one request; stream t owns
  // tokens [t * tpb, (t + 1) * tpb) x the `group` heads of KV head h.
  // launched as a programmatic dependent of the plan kernel, which writes the item table
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int4 it = *reinterpret_cast<const int4*>(p.items + 8 * item);
  const int req = it.x, q_row0 = it.y, q_valid = it.z, anchor = it.w;
  const int kv_limit = p.items[8 * item + 4];
  const int kv_start = p.items[8 * item + 5];  // packed K/V: first key row of the request
  const int kv_end = p.right >= 0 ? min(anchor + p.right, kv_limit) : kv_limit;  // the item's last row sits on diagonal anchor - 1
  if (q_valid <= 0) return;  // uniform across the CTA: nothing allocated yet
  // Once any CTA has reported a failed wait the launch is void: later CTAs
  // leave at once instead of each running into its own time limit.
  if (launch_is_void(p.status)) return;
  const int n_streams = q_valid > p.tpb ? kStreams : 1;
  const int diag_base = anchor - kStreams * p.tpb;  // token t of the item sits on diagonal diag_base + t
  const int first_key = p.window_left >= 0 ? max(0, diag_base - p.window_left) : 0;
  const int tile_lo = first_key / kBN;
  const int tile_hi = kv_end > 0 ? (kv_end + kBN - 1) / kBN : 0;  // exclusive
  const int n_tiles = max(0, tile_hi - tile_lo);

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kKvStages; ++s) {
      // filled by TMA (one arrival with a byte count), or by the converter warps
      mbar_init(&bars->k_full[s], kFp8 ? kConverterWarps : 1);
      mbar_init(&bars->v_full[s], kFp8 ? kConverterWarps : 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    mbar_init(&bars->f8k_full, 1);
    mbar_init(&bars->f8v_full, 1);
    mbar_init(&bars->f8k_empty, kConverterWarps);
    mbar_init(&bars->f8v_empty, kConverterWarps);
    for (int t = 0; t < kStreams; ++t) {
      mbar_init(&bars->s_full[t], 1);
      mbar_init(&bars->p_full[t], 4);
      mbar_init(&bars->pv_done[t], 1);
    }
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->q_rotated, 4 * n_streams);
    bars->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1 && n_tiles > 0) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (n_tiles > 0 && warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_kv);
      if (p.packed) tma_prefetch_desc(&map_v);
      mbar_arrive_expect_tx(&bars->q_full, n_streams * p.group * p.tpb * D * 2);
      for (int t = 0; t < n_streams; ++t)
        for (int g = 0; g < p.group; ++g)
          for (int half = 0; half < D / 64; ++half)
            tma_load_3d(smem + kSmemQ + t * 32768 + half * 16384 + g * p.tpb * 128, &map_q, &bars->q_full,
                        half * 64, q_row0 + t * p.tpb, h * p.group + g);
      bool ok = true;
      int k_armed = 0, v_armed = 0;  // tiles whose K / V copies have been issued
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kKvStages;
        const uint32_t round = j / kKvStages;
        // K of a stage is free once the QK MMAs of its tile are done, V once
        // the PV MMAs are: K therefore runs further ahead than V.  (fp8: the
        // staging tile is free once the converters have widened it.)
        if (!(kFp8 ? FW_WAIT(1, j, &bars->f8k_empty, (j & 1) ^ 1) : FW_WAIT(1, j, &bars->k_empty[s], (round & 1) ^ 1))) {
          ok = false;
          break;
        }
        // A 128-key tile is two 64-token boxes per operand half; the second is
        // left out when it lies wholly past the valid keys (its block-table
        // entry may not exist).  Rows that are not loaded are masked (K) or
        // zeroed by the softmax group (V).
        const int pos0 = (tile_lo + j) * kBN;
        const int subs = pos0 + 64 < kv_end ? 2 : 1;
        int page[2], tok[2];
        for (int sub = 0; sub < subs; ++sub) {
          const int pos = pos0 + sub * 64;
          if (p.packed) {
            // rows past the tensor read as zeros; rows of the next request are
            // masked (K) or zeroed (V) like stale page slots
            tok[sub] = kv_start + pos;
            page[sub] = 0;
            continue;
          }
          const int page_idx = pos / p.page_size;
          page[sub] = p.block_table[static_cast<long long>(req) * p.pages_per_seq + page_idx];
          if (page[sub] < 0 || page[sub] >= p.num_pages) {
            report_status(p.status, FW_STATUS_BAD_PAGE);
            page[sub] = 0;
          }
          tok[sub] = pos - page_idx * p.page_size;
        }
        if constexpr (kFp8) {
          // one 64-token box of a head plane is [64][128 B] of fp8
          mbar_arrive_expect_tx(&bars->f8k_full, subs * 64 * 128);
          for (int sub = 0; sub < subs; ++sub)
            tma_load_4d(smem + kSmemF8K + sub * 8192, &map_kv, &bars->f8k_full, 0, 2 * h, tok[sub], page[sub]);
          k_armed = j + 1;
          if (!FW_WAIT(18, j, &bars->f8v_empty, (j & 1) ^ 1)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&bars->f8v_full, subs * 64 * 128);
          for (int sub = 0; sub < subs; ++sub)
            tma_load_4d(smem + kSmemF8V + sub * 8192, &map_kv, &bars->f8v_full, 0, 2 * h + 1, tok[sub], page[sub]);
          v_armed = j + 1;
          continue;
        }
        mbar_arrive_expect_tx(&bars->k_full[s], subs * 64 * D * 2);
        for (int sub = 0; sub < subs; ++sub)
          for (int half = 0; half < D / 64; ++half) {
            uint8_t* dst = smem + kSmemK + s * 32768 + half * 16384 + sub * 8192;
            if (p.packed) tma_load_3d(dst, &map_kv, &bars->k_full[s], half * 64, tok[sub], h);
            else tma_load_4d(dst, &map_kv, &bars->k_full[s], half * 64, 2 * h, tok[sub], page[sub]);
          }
        k_armed = j + 1;
        if (!FW_WAIT(18, j, &bars->v_empty[s], (round & 1) ^ 1)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&bars->v_full[s], subs * 64 * D * 2);
        for (int sub = 0; sub < subs; ++sub)
          for (int half = 0; half < D / 64; ++half) {
            uint8_t* dst = smem + kSmemV + s * 32768 + half * 16384 + sub * 8192;
            if (p.packed) tma_load_3d(dst, &map_v, &bars->v_full[s], half * 64, tok[sub], h);
            else tma_load_4d(dst, &map_kv, &bars->v_full[s], half * 64, 2 * h + 1, tok[sub], page[sub]);
          }
        v_armed = j + 1;
      }
      if (!ok) {
        // A wait gave up: record it, tell the other warps, and let the copies
        // that are still in flight land before this CTA's shared memory goes away.
        *abort_flag = 1;
        report_timeout(p.status);
        drain_wait(&bars->q_full, 0);
        if constexpr (kFp8) {
          if (k_armed > 0) drain_wait(&bars->f8k_full, (k_armed - 1) & 1);
          if (v_armed > 0) drain_wait(&bars->f8v_full, (v_armed - 1) & 1);
        } else {
          for (int j = max(0, k_armed - kKvStages); j < k_armed; ++j)
            drain_wait(&bars->k_full[j % kKvStages], (j / kKvStages) & 1);
          for (int j = max(0, v_armed - kKvStages); j < v_armed; ++j)
            drain_wait(&bars->v_full[j % kKvStages], (j / kKvStages) & 1);
        }
      }
    }
  } else if (n_tiles > 0 && warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Per stream the chain is QK(j) -> softmax(j) -> PV(j) -> QK(j+1): S has one
    // buffer per stream (P overwrites it), so the next QK follows the PV that
    // read P.  The two streams alternate, which keeps the tensor pipe busy with
    // one stream's MMAs while the other stream's softmax group works.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = instr_desc(kBN, false, kF16);
      constexpr uint32_t idesc_pv = instr_desc(D, true, kF16);
      const uint64_t q_desc0 = smem_desc(smem_u32(smem + kSmemQ), 16, 1024);
      const uint64_t k_desc0 = smem_desc(smem_u32(smem + kSmemK), 16, 1024);
      const uint64_t v_desc0 = smem_desc(smem_u32(smem + kSmemV), 16384, 1024);
      auto issue_qk = [&](int t, int j) {
        const uint64_t q_desc = q_desc0 + static_cast<uint32_t>(t * (32768 >> 4));
        const uint64_t k_desc = k_desc0 + static_cast<uint32_t>((j % kKvStages) * (32768 >> 4));
        const uint32_t d_addr = tmem_s(tmem, t);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;  // head_dim half, 16-element step
          tc_mma(d_addr, desc_advance(q_desc, off), desc_advance(k_desc, off), idesc_qk, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars->s_full[t]);
      };
      // with a rotary embedding, or f16 operands, the softmax warps rework their rows of Q first
      bool ok = p.rotary_cos != nullptr || kF16 ? FW_WAIT(19, 0, &bars->q_rotated, 0) : FW_WAIT(2, 0, &bars->q_full, 0);
      if (ok) ok = FW_WAIT(3, 0, &bars->k_full[0], 0);
      if (ok) {
        tc_fence_after();
        for (int t = 0; t < n_streams; ++t) issue_qk(t, 0);
        tc_commit(&bars->k_empty[0]);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kKvStages;
        const uint32_t round = j / kKvStages;
        const uint64_t v_desc = v_desc0 + static_cast<uint32_t>(s * (32768 >> 4));
        for (int t = 0; t < n_streams && ok; ++t) {
          ok = FW_WAIT(6 + t, j, &bars->p_full[t], j & 1);
          if (ok && t == 0) ok = FW_WAIT(5, j, &bars->v_full[s], round & 1);
          if (!ok) break;
          tc_fence_after();
          const uint32_t o_addr = tmem_o(tmem, t), p_addr = tmem_s(tmem, t);
          tc_mma_ts(o_addr, p_addr, v_desc, idesc_pv, j > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < 8; ++k)
            tc_mma_ts(o_addr, p_addr + k * 8, desc_advance(v_desc, k * 2048), idesc_pv, 1u);
          tc_commit(&bars->pv_done[t]);
          if (t == n_streams - 1) tc_commit(&bars->v_empty[s]);
          if (j + 1 < n_tiles) {
            if (t == 0) ok = FW_WAIT(4, j, &bars->k_full[(j + 1) % kKvStages], ((j + 1) / kKvStages) & 1);
            if (!ok) break;
            tc_fence_after();
            issue_qk(t, j + 1);
            if (t == n_streams - 1) tc_commit(&bars->k_empty[(j + 1) % kKvStages]);
          }
        }
      }
      if (!ok) {
        // The MMAs issued so far must have drained before tensor memory is freed.
        *abort_flag = 1;
        report_timeout(p.status);
        tc_commit(&bars->drain);
        drain_wait(&bars->drain, 0);
      }
    }
  } else if (kFp8 && warp >= 2 + kStreams * 4) {
    // ------------------------------------------------------------ fp8 -> bf16 converters
    // Each 16-byte chunk of a staged fp8 row (16 head_dim elements of one key)
    // becomes two 16-byte chunks of the bf16 operand tile: half d / 64, row =
    // key, chunk (d % 64) / 8 under the 128-byte swizzle, the layout a TMA copy
    // of a bf16 pool would have produced.
    if (n_tiles > 0) {
      const int ct = (warp - (2 + kStreams * 4)) * 32 + lane;  // 0 .. 63
      bool ok = true;
      // Thread ct always takes 16-byte chunk ct % 8 of keys ct / 8, ct / 8 + 8, ...:
      // the swizzle term (key & 7) is then a per-thread constant and a step is
      // 1024 bytes in both buffers.  Eight chunks are loaded before any is widened
      // so the conversions of different keys overlap.
      const int c8 = ct & 7, r0 = ct >> 3;
      const int src_off = r0 * 128 + ((c8 ^ r0) << 4);
      const int c = (c8 & 3) * 2;
      const int dst_off = (c8 >> 2) * 16384 + r0 * 128;
      const int dst_a = dst_off + ((c ^ r0) << 4), dst_b = dst_off + (((c + 1) ^ r0) << 4);
      auto widen_tile = [&](const uint8_t* staged, uint8_t* tile) {
#pragma unroll 1
        for (int n0 = 0; n0 < kBN / 8; n0 += 8) {
          uint4 raw[8];
#pragma unroll
          for (int n = 0; n < 8; ++n) raw[n] = *reinterpret_cast<const uint4*>(staged + src_off + (n0 + n) * 1024);
#pragma unroll
          for (int n = 0; n < 8; ++n) {
            const uint32_t w[4] = {raw[n].x, raw[n].y, raw[n].z, raw[n].w};
            uint32_t wide[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              // every fp8 value is an f16 value: one conversion per pair, no rounding
              wide[2 * i] = fp8_half_to_f16x2<KVT, false>(w[i]);
              wide[2 * i + 1] = fp8_half_to_f16x2<KVT, true>(w[i]);
            }
            *reinterpret_cast<uint4*>(tile + dst_a + (n0 + n) * 1024) = make_uint4(wide[0], wide[1], wide[2], wide[3]);
            *reinterpret_cast<uint4*>(tile + dst_b + (n0 + n) * 1024) = make_uint4(wide[4], wide[5], wide[6], wide[7]);
          }
        }
      };
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kKvStages;
        const uint32_t round = j / kKvStages;
        ok = FW_WAIT(24, j, &bars->f8k_full, j & 1);
        if (ok) ok = FW_WAIT(25, j, &bars->k_empty[s], (round & 1) ^ 1);
        if (!ok) break;
        widen_tile(smem + kSmemF8K, smem + kSmemK + s * 32768);
        fence_proxy_async_smem();  // the tensor core reads what these threads wrote
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->k_full[s]);
          mbar_arrive(&bars->f8k_empty);
        }
        ok = FW_WAIT(26, j, &bars->f8v_full, j & 1);
        if (ok) ok = FW_WAIT(27, j, &bars->v_empty[s], (round & 1) ^ 1);
        if (!ok) break;
        widen_tile(smem + kSmemF8V, smem + kSmemV + s * 32768);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->v_full[s]);
          mbar_arrive(&bars->f8v_empty);
        }
      }
      if (!ok && lane == 0) {
        *abort_flag = 1;
        report_timeout(p.status);
      }
    }
  } else if (warp >= 2 && (warp - 2) / 4 < n_streams) {
    // ------------------------------------------------------------ softmax groups
    const int t = (warp - 2) >> 2;           // stream of this warp group
    const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;     // row of the stream's 128-row tile
    const int g = row / p.tpb, tl = t * p.tpb + (row - g * p.tpb);  // head in group, token in item
    const bool row_ok = g < p.group && tl < q_valid;
    const int diag = diag_base + tl;
    const int diag_lo = diag_base + t * p.tpb, diag_hi = diag_lo + p.tpb - 1;  // this stream's diagonals
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_addr = tmem_s(tmem, t) + lane_addr, o_addr = tmem_o(tmem, t) + lane_addr;
    const float kd = p.k_descale ? *p.k_descale : 1.0f;
    const float c1 = p.softcap > 0.f ? p.scale * kd / p.softcap : p.scale * kd * kLog2e;
    const float c2 = p.softcap * kLog2e;
    const float mul = p.softcap > 0.f ? 1.0f : c1;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;

    if ((p.rotary_cos != nullptr || kF16) && n_tiles > 0) {
      // Rotary embedding, fused: this thread's softmax row is also its row of the
      // Q tile the TMA copy left in shared memory; rotate it in place at the
      // row's own key position (its diagonal) before the first QK MMA reads it.
      // With an fp8 pool the MMAs take f16 operands (the pool's values widen to
      // f16 exactly, with one conversion per pair), so the row becomes f16 here.
      ok = FW_WAIT(20 + t, 0, &bars->q_full, 0);
      if (ok) {
        if (p.rotary_cos != nullptr && row_ok && diag >= 0 && diag < p.rotary_len)
          rotate_q_row_in_smem<D>(smem + kSmemQ + t * 32768, 16384, row, diag, p);
        if constexpr (kF16) q_row_bf16_to_f16_in_smem<D>(smem + kSmemQ + t * 32768, 16384, row);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->q_rotated);
      }
    }

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % kKvStages;
      const int pos0 = (tile_lo + j) * kBN;
      if (!FW_WAIT(8 + t, j, &bars->s_full[t], j & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // keys every row of the stream sees without a right-side mask
      const int clear_end = p.right >= 0 ? min(diag_lo + p.right + 1, kv_end) : kv_end;
      const bool need_mask = pos0 + kBN > clear_end ||
                             (p.window_left >= 0 && pos0 < diag_hi - p.window_left);
      // One pass per 64-key half: load S, softcap / mask (warp-uniform code
      // variants), P = 2^(s * mul - base) against the CURRENT exponent base, and
      // the row max of the exponents.  The base only has to move when a score
      // outruns it by more than kRescaleThreshold (or on the first tile): then
      // the tile is redone against the new base and O is rescaled.  So the
      // common tile reads S once and needs no separate max pass.
      uint32_t packed[2][32];
      float sum, top;   // row sum of P; row max of the exponents (true-max variant only)
      bool over;        // some P above 2^kRescaleThreshold (cheap variant only)
      auto exponentiate = [&](float neg_base, auto want_true_max) {
        constexpr bool kTrueMax = decltype(want_true_max)::value;
        uint64_t sum2 = pack2(0.f, 0.f);
        const uint64_t mul2 = pack2(mul, mul), base2 = pack2(neg_base, neg_base);
        float top0 = -INFINITY, top1 = -INFINITY;
        uint32_t pmax = 0u;  // P >= 0, so +0 is the identity of the bf16 max
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t sr[2][32];
          tmem_ld32(s_addr + half * 64, sr[0]);
          tmem_ld32(s_addr + half * 64 + 32, sr[1]);
          tmem_wait_ld();
          const int hpos = pos0 + half * 64;
          if (p.softcap > 0.f) {
            if (need_mask) transform_row<true, true>(sr, c1, c2, hpos, kv_end, diag, p.right, p.window_left);
            else transform_row<true, false>(sr, c1, c2, hpos, kv_end, diag, p.right, p.window_left);
          } else if (need_mask) {
            transform_row<false, true>(sr, c1, c2, hpos, kv_end, diag, p.right, p.window_left);
          }
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const uint64_t y2 = fma2(pack2(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), mul2, base2);
              if constexpr (kTrueMax) {
                float y0, y1;
                unpack2(y2, y0, y1);
                top0 = fmaxf(top0, y0);
                top1 = fmaxf(top1, y1);
              }
              float p0, p1;
              uint32_t pk;
              if constexpr (FW_EXP2_BF16X2 != 0) {
                // both exponentials in one special-function op, on bf16 operands: P is
                // rounded to bf16 for the PV MMA anyway, and the row sum below adds the
                // rounded values, so l matches the P the MMA sees
                float y0, y1;
                unpack2(y2, y0, y1);
                pk = exp2_bf16x2(pack_bf16(y0, y1));
                p0 = __uint_as_float(pk << 16);
                p1 = __uint_as_float(pk & 0xffff0000u);
              } else {
                // the loop is fully unrolled, so this choice is made at compile time
                if (FW_EXP2_POLY_EVERY > 0 && ((i >> 1) % (FW_EXP2_POLY_EVERY > 0 ? FW_EXP2_POLY_EVERY : 1)) == 0)
                  exp2_pair<true>(y2, p0, p1);
                else
                  exp2_pair<false>(y2, p0, p1);
                pk = kF16 ? pack_f16(p0, p1) : pack_bf16(p0, p1);
              }
              sum2 = add2(sum2, pack2(p0, p1));
              if constexpr (!kTrueMax && FW_OVER_BY_SUM == 0) pmax = kF16 ? max_f16x2(pmax, pk) : max_bf16x2(pmax, pk);
              packed[half][c * 16 + (i >> 1)] = pk;
            }
        }
        float s0, s1;
        unpack2(sum2, s0, s1);
        sum = s0 + s1;
        top = fmaxf(top0, top1);  // row max minus the base (the row max itself when the base is 0)
        // bf16 bit patterns of non-negative values order like integers
        if constexpr (FW_OVER_BY_SUM != 0) over = sum > 256.0f;  // no P can be above 2^8 unless their sum is
        else over = max(pmax & 0xffffu, pmax >> 16) > (kF16 ? 0x5c00u : 0x4380u);  // 256.0 = 2^kRescaleThreshold as f16 / bf16
      };
      static_assert(kRescaleThreshold == 8.0f, "the bf16 constant above is 2^8");
      float alpha = 1.f;
      float neg_base = m_used == -INFINITY ? 0.f : -m_used;
      // Rows that have no base yet (first tile, or everything masked so far) need
      // the true row max; otherwise the cheap variant only tells whether some
      // exponent outran the base.
      const bool fresh = m_used == -INFINITY;
      const bool any_fresh = __any_sync(0xffffffffu, fresh);
      if (any_fresh) exponentiate(neg_base, std::true_type{});
      else exponentiate(neg_base, std::false_type{});
      const bool move_base = fresh ? top > -INFINITY : (any_fresh ? top > kRescaleThreshold : over);
      if (__any_sync(0xffffffffu, move_base)) {
        if (!any_fresh) exponentiate(neg_base, std::true_type{});  // rare: fetch the true max
        if (move_base) {
          const float mx = top - neg_base;
          alpha = fast_exp2(m_used - mx);  // 0 when there was no base yet
          m_used = mx;
          neg_base = -mx;
        }
        exponentiate(neg_base, std::false_type{});  // lanes whose base stayed put get the same P again
        if (j > 0) {
          // PV(j-1) of this stream precedes QK(j) in the tensor pipe, so it has
          // drained; the wait makes its writes to O visible here.
          if (!FW_WAIT(10 + t, j, &bars->pv_done[t], (j - 1) & 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr + c * 32, o);
          }
        }
      }
      // P over the start of S: two bf16 keys per 32-bit column, the A operand of
      // the PV MMA.  (All of this thread's S row has been read by now.)
      tmem_st32(s_addr, packed[0]);
      tmem_st32(s_addr + 32, packed[1]);
      l_run = l_run * alpha + sum;
      tmem_wait_st();
      // Last tile: keys past the valid length may hold anything (NaN included);
      // their P is 0, so their V rows must be finite: zero them.  Both streams
      // write the same zeros, so neither depends on the other.
      if (pos0 + kBN > kv_end) {
        if (!FW_WAIT(12 + t, j, &bars->v_full[s], (j / kKvStages) & 1)) {
          ok = false;
          break;
        }
        const int first_bad = kv_end - pos0;  // in [1, kBN - 1]
        uint8_t* vbase = smem + kSmemV + s * 32768;
        for (int idx = row; idx < (kBN - first_bad) * (D / 8); idx += 128) {
          const int r = first_bad + idx / (D / 8), c = idx % (D / 8);
          *reinterpret_cast<uint4*>(vbase + (c >> 3) * 16384 + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[t]);
    }

    // ---- epilogue: O / l -> bf16, lse
    if (ok && n_tiles > 0) ok = FW_WAIT(16 + t, n_tiles - 1, &bars->pv_done[t], (n_tiles - 1) & 1);
    if (ok) {
      tc_fence_after();
      const int hq = h * p.group + min(g, p.group - 1);
      const float sink2 = p.sinks ? p.sinks[p.sink_period > 0 ? hq % p.sink_period : hq] * kLog2e : -INFINITY;
      const float m_all = fmaxf(m_used, sink2);
      float out_scale = 0.f, lse = -INFINITY;
      if (m_all != -INFINITY) {
        const float w_keys = m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_all);
        const float den = l_run * w_keys + (sink2 == -INFINITY ? 0.f : fast_exp2(sink2 - m_all));
        if (den > 0.f) {
          out_scale = w_keys * (p.v_descale ? *p.v_descale : 1.0f) / den;
          lse = (m_all + log2f(den)) * kLn2;
        }
      }
      __nv_bfloat16* orow = p.out + (static_cast<long long>(q_row0) + tl) * p.tok_stride +
                            static_cast<long long>(hq) * p.head_stride;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld32(o_addr + c * 32, o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            v.x = pack_bf16(__uint_as_float(o[i]) * out_scale, __uint_as_float(o[i + 1]) * out_scale);
            v.y = pack_bf16(__uint_as_float(o[i + 2]) * out_scale, __uint_as_float(o[i + 3]) * out_scale);
            v.z = pack_bf16(__uint_as_float(o[i + 4]) * out_scale, __uint_as_float(o[i + 5]) * out_scale);
            v.w = pack_bf16(__uint_as_float(o[i + 6]) * out_scale, __uint_as_float(o[i + 7]) * out_scale);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = v;
          }
        }
      }
      if (row_ok && p.lse != nullptr) p.lse[static_cast<long long>(hq) * p.total_q + q_row0 + tl] = lse;
      tc_fence_before();
    } else if (lane == 0) {
      *abort_flag = 1;
      report_timeout(p.status);
    }
  }

  // ---- teardown: everyone meets here, then the allocating warp frees TMEM.
  __syncthreads();
  if (warp == 1 && n_tiles > 0) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

// ---------------------------------------------------------------- host
bool tcgen05_prefill_supported(const FwPrefillArgs* a) {
  if (a->head_dim == 256) return tcgen05_d256_supported(a);
  const bool packed_kv = a->block_table == nullptr && a->v_packed != nullptr;
  // fp8 pools are widened inside the kernel: paged, head_dim 128 (a head plane is one 128-byte row)
  if (a->kv_dtype != FW_DTYPE_BF16 && (packed_kv || a->head_dim != 128)) return false;
  if (a->head_dim != 128 && !(a->head_dim == 64 && packed_kv)) return false;
  if (a->nheads_k <= 0 || a->nheads % a->nheads_k) return false;
  const int group = a->nheads / a->nheads_k;
  // 128 rows hold (128 / group) tokens x group heads; a group that does not
  // divide 128 leaves the last rows idle.
  if (group > kBM) return false;
  const bool packed = a->block_table == nullptr && a->v_packed != nullptr;
  if (!packed && (a->page_size <= 0 || a->page_size % 64)) return false;  // a tile is two 64-token boxes
  if (a->batch > 2048) return false;
  if (!(a->softmax_scale > 0.f)) return false;  // the row max is taken before scaling
  return true;
}

static int tc05_max_items(const FwPrefillArgs* a) {
  const int qb = kStreams * (kBM / (a->nheads / a->nheads_k));  // query tokens per CTA
  return (a->total_q + qb - 1) / qb + a->batch;
}

uint64_t tcgen05_prefill_workspace_bytes(const FwPrefillArgs* a) {
  if (a->head_dim == 256) return tcgen05_d256_workspace_bytes(a);
  return 256 + static_cast<uint64_t>(tc05_max_items(a)) * 8 * sizeof(int);
}

int tcgen05_prefill(const FwPrefillArgs* a, cudaStream_t stream) {
  if (a->head_dim == 256) return tcgen05_d256_prefill(a, stream);
  const bool packed = a->block_table == nullptr && a->v_packed != nullptr;
  if (packed) {
    const bool slots = a->kv_request_stride > 0 && a->seqused_k != nullptr;  // fixed-size request slots
    if (a->q == nullptr || a->out == nullptr || a->kv_cache == nullptr || a->cu_seqlens_q == nullptr ||
        (a->cu_seqlens_k == nullptr && !slots) || a->total_k <= 0) {
      set_error("q, out, k, v, cu_seqlens_q and cu_seqlens_k must not be NULL and total_k positive.");
      return FW_ERR_BAD_SHAPE;
    }
    if (reinterpret_cast<uintptr_t>(a->v_packed) & 15) {
      set_error("v must be 16-byte aligned.");
      return FW_ERR_BAD_SHAPE;
    }
  } else if (a->q == nullptr || a->out == nullptr || a->kv_cache == nullptr || a->cu_seqlens_q == nullptr ||
             a->seqused_k == nullptr || a->block_table == nullptr) {
    set_error("q, out, kv_cache, cu_seqlens_q, seqused_k and block_table must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  const uint64_t need = tcgen05_prefill_workspace_bytes(a);
  if (a->workspace == nullptr || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 255)) {
    set_error("workspace must be 256-byte aligned and hold %llu bytes; got %llu.",
              static_cast<unsigned long long>(need), static_cast<unsigned long long>(a->workspace_bytes));
    return FW_ERR_WORKSPACE;
  }
  if ((reinterpret_cast<uintptr_t>(a->kv_cache) & 15) || (reinterpret_cast<uintptr_t>(a->q) & 15) ||
      (reinterpret_cast<uintptr_t>(a->out) & 15)) {
    set_error("q, out and the cache must be 16-byte aligned.");
    return FW_ERR_BAD_SHAPE;
  }
  const int group = a->nheads / a->nheads_k;
  const int tpb = kBM / group;
  const int max_items = tc05_max_items(a);
  Tc05Params p;
  p.items = reinterpret_cast<int*>(static_cast<uint8_t*>(a->workspace) + 256);
  p.block_table = a->block_table;
  p.k_descale = a->k_descale;
  p.v_descale = a->v_descale;
  p.sinks = a->sinks;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.status = static_cast<int*>(a->workspace);
  const int d = a->head_dim;
  if (a->token_major) {
    p.tok_stride = static_cast<long long>(a->nheads) * d;
    p.head_stride = d;
  } else {
    p.tok_stride = d;
    p.head_stride = static_cast<long long>(a->total_q) * d;
  }
  p.num_pages = a->num_pages;
  p.total_q = a->total_q;
  p.nheads = a->nheads;
  p.group = group;
  p.tpb = tpb;
  p.page_size = a->page_size;
  p.pages_per_seq = a->pages_per_seq;
  p.right = a->causal ? 0 : (packed && a->window_right > 0 ? a->window_right : -1);
  p.window_left = a->window_left;
  p.scale = a->softmax_scale;
  p.softcap = a->softcap;
  p.packed = packed;
  p.sink_period = a->sink_period;
  p.rotary_cos = a->rotary_cos;
  p.rotary_sin = a->rotary_sin;
  p.rotary_len = a->rotary_len;
  p.rotary_interleaved = a->rotary_interleaved;
  p.rotary_bf16 = a->rotary_bf16;

  int rc = launch_prefill_plan(a, kStreams * tpb, max_items, const_cast<int*>(p.items), p.tok_stride,
                               p.head_stride, p.status, stream);
  if (rc != FW_OK) return rc;

  // q viewed as (head_dim, tokens, heads); a box is 64 elements x tpb tokens of one head.
  CUtensorMap map_q, map_kv, map_v;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(d), static_cast<uint64_t>(a->total_q),
                              static_cast<uint64_t>(a->nheads)};
    const uint64_t strides[2] = {static_cast<uint64_t>(p.tok_stride) * 2, static_cast<uint64_t>(p.head_stride) * 2};
    const uint32_t box[3] = {64, static_cast<uint32_t>(tpb), 1};
    rc = encode_tensor_map_bf16(&map_q, 3, a->q, dims, strides, box);
    if (rc != FW_OK) return rc;
  }
  if (packed) {
    // K and V viewed as (head_dim, tokens, heads); a box is 64 elements x 64 tokens of one head.
    const uint64_t dims[3] = {static_cast<uint64_t>(d), static_cast<uint64_t>(a->total_k),
                              static_cast<uint64_t>(a->nheads_k)};
    const uint64_t row = static_cast<uint64_t>(d) * 2;
    const uint64_t tok = a->kv_token_major ? static_cast<uint64_t>(a->nheads_k) * row : row;
    const uint64_t head = a->kv_token_major ? row : static_cast<uint64_t>(a->total_k) * row;
    const uint64_t strides[2] = {tok, head};
    const uint32_t box[3] = {64, 64, 1};
    rc = encode_tensor_map_bf16(&map_kv, 3, a->kv_cache, dims, strides, box);
    if (rc != FW_OK) return rc;
    rc = encode_tensor_map_bf16(&map_v, 3, a->v_packed, dims, strides, box);
    if (rc != FW_OK) return rc;
  } else {
    // pool viewed as (head_dim, head planes [k0,v0,k1,v1,...], tokens in page, pages)
    if (a->kv_dtype == FW_DTYPE_BF16) {
      const uint64_t planes = 2ull * a->nheads_k;
      const uint64_t row_bytes = planes * 256;
      const uint64_t dims[4] = {128, planes, static_cast<uint64_t>(a->page_size), static_cast<uint64_t>(a->num_pages)};
      const uint64_t strides[3] = {256, row_bytes, row_bytes * a->page_size};
      const uint32_t box[4] = {64, 1, 64, 1};
      rc = encode_tensor_map_bf16(&map_kv, 4, a->kv_cache, dims, strides, box);
    } else {
      // fp8: bytes; a head plane of a token is one 128-byte row, an odd head count carries a pad head
      const uint64_t planes = 2ull * ((a->nheads_k + 1) / 2 * 2);
      const uint64_t row_bytes = planes * 128;
      const uint64_t dims[4] = {128, planes, static_cast<uint64_t>(a->page_size), static_cast<uint64_t>(a->num_pages)};
      const uint64_t strides[3] = {128, row_bytes, row_bytes * a->page_size};
      const uint32_t box[4] = {128, 1, 64, 1};
      rc = encode_tensor_map_u8_4d(&map_kv, a->kv_cache, dims, strides, box);
    }
    if (rc != FW_OK) return rc;
    map_v = map_kv;
  }
  using Kernel = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const Tc05Params);
  Kernel kernel = d == 64 ? prefill_tcgen05_kernel<64> : prefill_tcgen05_kernel<128>;
  int smem_bytes = kSmemBytes, threads = 64 + kStreams * 128;
  if (a->kv_dtype != FW_DTYPE_BF16) {
    kernel = a->kv_dtype == FW_DTYPE_E4M3 ? prefill_tcgen05_kernel<128, FW_DTYPE_E4M3>
                                          : prefill_tcgen05_kernel<128, FW_DTYPE_E5M2>;
    smem_bytes = kSmemBytesFp8;
    threads += kConverterWarps * 32;
  }
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (err != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%d bytes): %s", smem_bytes, cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  dim3 grid(a->nheads_k, max_items);
  cudaLaunchAttribute pdl{};
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, map_q, map_kv, map_v, p);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("tcgen05 prefill kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

}  // namespace fw
