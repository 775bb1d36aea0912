// head_dim 256 on the 5th-generation tensor cores: chunked prefill over the
// paged merged bf16 cache and attention over packed K/V, the same contract as
// prefill_tcgen05.cu (reference: flywheel_tpu/softmax_attention/prefill.py:437-661
// and kernels/fwd_paged.py:331-1019 of the reference project; its serving
// shapes use head_dim 256, docs/v7x.md:129-150).
//
// At 256 one 128-row output tile already takes 256 of the 512 tensor-memory
// columns, so a CTA holds ONE query tile (128 / group tokens x the group's
// heads) and instead keeps two S buffers: QK^T of tile j + 1 is issued before
// the softmax of tile j has finished, and the tensor pipe alternates QK(j + 1),
// PV(j) while the four softmax warps work through S(j).  Shared memory is what
// limits the KV tile to 64 keys: Q 64 KiB, K and V two stages of 32 KiB each.
//   warp 0: TMA producer, warp 1: tensor memory + MMA issue, warps 2-5: softmax
//   (one thread per row).  Tensor memory: O in columns [0, 256), S of even /
//   odd tiles in [256, 320) / [320, 384); P overwrites the start of its S.
#include "tcgen05.cuh"

namespace fw {
namespace d256 {

constexpr int kStages = 2;                 // K and V ring depth
constexpr int kTmemCols = 512;
constexpr int kThreads = 64 + 128;

// Shared-memory plan for head_dim D and BN keys per tile: operands are stored as
// 64-element (128-byte) column blocks, [block][rows][128 B].
template <int D, int BN>
struct Plan {
  static constexpr int kBlocks = D / 64;
  static constexpr int kKeyBlock = BN * 128;             // bytes of one column block of a K / V tile
  static constexpr int kQBytes = kBlocks * 16384;        // 128 query rows
  static constexpr int kTileBytes = kBlocks * kKeyBlock;
  static constexpr int kSmemQ = 0;
  static constexpr int kSmemK = kQBytes;
  static constexpr int kSmemV = kSmemK + kStages * kTileBytes;
  static constexpr int kSmemBar = kSmemV + kStages * kTileBytes;
  static constexpr int kSmemBytes = kSmemBar + 256;
  static_assert(D + 2 * BN <= kTmemCols, "O plus two S buffers must fit tensor memory");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct Bars {
  uint64_t q_full;
  uint64_t k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t s_full[2], p_full[2], pv_done;
  uint64_t drain;  // abort path: completion of the MMAs issued so far
  uint64_t q_rotated;  // rotary embedding: every softmax warp has rotated its rows of Q
  uint32_t tmem_base;
  int abort_flag;
};

template <int D, int BN>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tcgen05_d256_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const __grid_constant__ CUtensorMap map_v, const Tc05Params p) {
  using L = Plan<D, BN>;
  constexpr int kD = D, kBN = BN, kBlocks = L::kBlocks, kTileBytes = L::kTileBytes, kKeyBlock = L::kKeyBlock;
  constexpr int kSmemQ = L::kSmemQ, kSmemK = L::kSmemK, kSmemV = L::kSmemV, kSmemBar = L::kSmemBar;
  // tensor memory: O in columns [0, D), S of even / odd tiles behind it
  auto tmem_s = [](uint32_t base, int j) { return base + D + (j & 1) * BN; };
  extern __shared__ __align__(1024) uint8_t smem[];
  Bars* bars = reinterpret_cast<Bars*>(smem + kSmemBar);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.y, h = blockIdx.x;

  // An item is up to tpb query tokens of one request x the `group` heads of KV head h.
  // launched as a programmatic dependent of the plan kernel, which writes the item table
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int4 it = *reinterpret_cast<const int4*>(p.items + 8 * item);
  const int req = it.x, q_row0 = it.y, q_valid = it.z, anchor = it.w;
  const int kv_limit = p.items[8 * item + 4];
  const int kv_start = p.items[8 * item + 5];
  const int kv_end = p.right >= 0 ? min(anchor + p.right, kv_limit) : kv_limit;
  if (q_valid <= 0) return;
  if (launch_is_void(p.status)) return;
  const int diag_base = anchor - p.tpb;  // token t of the item sits on diagonal diag_base + t
  const int first_key = p.window_left >= 0 ? max(0, diag_base - p.window_left) : 0;
  const int tile_lo = first_key / kBN;
  const int tile_hi = kv_end > 0 ? (kv_end + kBN - 1) / kBN : 0;
  const int n_tiles = max(0, tile_hi - tile_lo);

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1);
      mbar_init(&bars->p_full[b], 4);
    }
    mbar_init(&bars->pv_done, 1);
    mbar_init(&bars->drain, 1);
    mbar_init(&bars->q_rotated, 4);
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
      mbar_arrive_expect_tx(&bars->q_full, p.group * p.tpb * kD * 2);
      for (int g = 0; g < p.group; ++g)
        for (int blk = 0; blk < kBlocks; ++blk)
          tma_load_3d(smem + kSmemQ + blk * 16384 + g * p.tpb * 128, &map_q, &bars->q_full, blk * 64, q_row0,
                      h * p.group + g);
      bool ok = true;
      int k_armed = 0, v_armed = 0;  // tiles whose K / V copies have been issued
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        const uint32_t round = j / kStages;
        // a tile is BN / 64 boxes of 64 tokens per column block; a box wholly past
        // the valid keys is left out (its block-table entry may not exist)
        const int pos0 = (tile_lo + j) * kBN;
        constexpr int kSubs = kBN / 64;
        int page[kSubs], tok[kSubs];
        int subs = 0;
        for (int sub = 0; sub < kSubs; ++sub) {
          const int pos = pos0 + sub * 64;
          if (sub > 0 && pos >= kv_end) break;
          ++subs;
          page[sub] = 0;
          if (p.packed) {
            tok[sub] = kv_start + pos;
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
        if (!FW_WAIT(1, j, &bars->k_empty[s], (round & 1) ^ 1)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&bars->k_full[s], subs * 64 * kD * 2);
        for (int sub = 0; sub < subs; ++sub)
          for (int blk = 0; blk < kBlocks; ++blk) {
            uint8_t* dst = smem + kSmemK + s * kTileBytes + blk * kKeyBlock + sub * 8192;
            if (p.packed) tma_load_3d(dst, &map_kv, &bars->k_full[s], blk * 64, tok[sub], h);
            else tma_load_4d(dst, &map_kv, &bars->k_full[s], blk * 64, 2 * h, tok[sub], page[sub]);
          }
        k_armed = j + 1;
        if (!FW_WAIT(18, j, &bars->v_empty[s], (round & 1) ^ 1)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&bars->v_full[s], subs * 64 * kD * 2);
        for (int sub = 0; sub < subs; ++sub)
          for (int blk = 0; blk < kBlocks; ++blk) {
            uint8_t* dst = smem + kSmemV + s * kTileBytes + blk * kKeyBlock + sub * 8192;
            if (p.packed) tma_load_3d(dst, &map_v, &bars->v_full[s], blk * 64, tok[sub], h);
            else tma_load_4d(dst, &map_kv, &bars->v_full[s], blk * 64, 2 * h + 1, tok[sub], page[sub]);
          }
        v_armed = j + 1;
      }
      if (!ok) {
        // A wait gave up: record it, tell the other warps, and let the copies
        // that are still in flight land before this CTA's shared memory goes away.
        *abort_flag = 1;
        report_timeout(p.status);
        drain_wait(&bars->q_full, 0);
        for (int j = max(0, k_armed - kStages); j < k_armed; ++j)
          drain_wait(&bars->k_full[j % kStages], (j / kStages) & 1);
        for (int j = max(0, v_armed - kStages); j < v_armed; ++j)
          drain_wait(&bars->v_full[j % kStages], (j / kStages) & 1);
      }
    }
  } else if (n_tiles > 0 && warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    // Issue order: QK(0); then per tile j: QK(j + 1), PV(j).  QK(j + 1) writes the
    // S buffer that P(j - 1) occupied; PV(j - 1) was issued before it and the
    // tensor pipe runs in order, so no wait is needed for that.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = instr_desc(kBN, false);
      constexpr uint32_t idesc_pv = instr_desc(kD, true);
      const uint64_t q_desc = smem_desc(smem_u32(smem + kSmemQ), 16, 1024);
      const uint64_t k_desc0 = smem_desc(smem_u32(smem + kSmemK), 16, 1024);
      const uint64_t v_desc0 = smem_desc(smem_u32(smem + kSmemV), kKeyBlock, 1024);
      auto issue_qk = [&](int j) {
        const uint64_t k_desc = k_desc0 + static_cast<uint32_t>((j % kStages) * (kTileBytes >> 4));
        const uint32_t d_addr = tmem_s(tmem, j);
#pragma unroll
        for (int k = 0; k < kD / 16; ++k)
          tc_mma(d_addr, desc_advance(q_desc, (k >> 2) * 16384 + (k & 3) * 32),
                 desc_advance(k_desc, (k >> 2) * kKeyBlock + (k & 3) * 32), idesc_qk, k > 0 ? 1u : 0u);
        tc_commit(&bars->s_full[j & 1]);
        tc_commit(&bars->k_empty[j % kStages]);
      };
      // with a rotary embedding the softmax warps rotate their rows of Q first
      bool ok = p.rotary_cos != nullptr ? FW_WAIT(19, 0, &bars->q_rotated, 0) : FW_WAIT(2, 0, &bars->q_full, 0);
      if (ok) ok = FW_WAIT(3, 0, &bars->k_full[0], 0);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kStages;
        if (j + 1 < n_tiles) {
          ok = FW_WAIT(4, j, &bars->k_full[(j + 1) % kStages], ((j + 1) / kStages) & 1);
          if (!ok) break;
          tc_fence_after();
          issue_qk(j + 1);
        }
        ok = FW_WAIT(5, j, &bars->v_full[s], (j / kStages) & 1);
        if (ok) ok = FW_WAIT(6, j, &bars->p_full[j & 1], (j >> 1) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint64_t v_desc = v_desc0 + static_cast<uint32_t>(s * (kTileBytes >> 4));
        const uint32_t p_addr = tmem_s(tmem, j);
        tc_mma_ts(tmem, p_addr, v_desc, idesc_pv, j > 0 ? 1u : 0u);
#pragma unroll
        for (int k = 1; k < kBN / 16; ++k)
          tc_mma_ts(tmem, p_addr + k * 8, desc_advance(v_desc, k * 2048), idesc_pv, 1u);
        tc_commit(&bars->pv_done);
        tc_commit(&bars->v_empty[s]);
      }
      if (!ok) {
        // The MMAs issued so far must have drained before tensor memory is freed.
        *abort_flag = 1;
        report_timeout(p.status);
        tc_commit(&bars->drain);
        drain_wait(&bars->drain, 0);
      }
    }
  } else if (warp >= 2) {
    // ------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;            // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;     // row of the 128-row tile
    const int g = row / p.tpb, tl = row - g * p.tpb;  // head in group, token in item
    const bool row_ok = g < p.group && tl < q_valid;
    const int diag = diag_base + tl;
    const int diag_lo = diag_base, diag_hi = diag_base + p.tpb - 1;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t o_addr = tmem + lane_addr;
    const float kd = p.k_descale ? *p.k_descale : 1.0f;
    const float c1 = p.softcap > 0.f ? p.scale * kd / p.softcap : p.scale * kd * kLog2e;
    const float c2 = p.softcap * kLog2e;
    const float mul = p.softcap > 0.f ? 1.0f : c1;
    float m_used = -INFINITY, l_run = 0.f;
    bool ok = true;

    if (p.rotary_cos != nullptr && n_tiles > 0) {
      // Rotary embedding, fused: rotate this thread's row of the Q tile in shared
      // memory at the row's own key position before the first QK MMA reads it.
      ok = FW_WAIT(20, 0, &bars->q_full, 0);
      if (ok) {
        if (row_ok && diag >= 0 && diag < p.rotary_len) rotate_q_row_in_smem<kD>(smem + kSmemQ, 16384, row, diag, p);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->q_rotated);
      }
    }

    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % kStages;
      const int pos0 = (tile_lo + j) * kBN;
      const uint32_t s_addr = tmem_s(tmem, j) + lane_addr;
      if (!FW_WAIT(8, j, &bars->s_full[j & 1], (j >> 1) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int clear_end = p.right >= 0 ? min(diag_lo + p.right + 1, kv_end) : kv_end;
      const bool need_mask = pos0 + kBN > clear_end || (p.window_left >= 0 && pos0 < diag_hi - p.window_left);
      constexpr int kHalves = kBN / 64;  // 64 keys per pass over a row
      uint32_t packed[kHalves][32];
      float sum, top;
      bool over;
      auto exponentiate = [&](float neg_base, auto want_true_max) {
        constexpr bool kTrueMax = decltype(want_true_max)::value;
        uint64_t sum2 = pack2(0.f, 0.f);
        const uint64_t mul2 = pack2(mul, mul), base2 = pack2(neg_base, neg_base);
        float top0 = -INFINITY, top1 = -INFINITY;
        uint32_t pmax = 0u;
#pragma unroll
        for (int half = 0; half < kHalves; ++half) {
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
                pk = pack_bf16(p0, p1);
              }
              sum2 = add2(sum2, pack2(p0, p1));
              if constexpr (!kTrueMax && FW_OVER_BY_SUM == 0) pmax = max_bf16x2(pmax, pk);
              packed[half][c * 16 + (i >> 1)] = pk;
            }
        }
        float s0, s1;
        unpack2(sum2, s0, s1);
        sum = s0 + s1;
        top = fmaxf(top0, top1);
        if constexpr (FW_OVER_BY_SUM != 0) over = sum > 256.0f;  // no P can be above 2^8 unless their sum is
        else over = max(pmax & 0xffffu, pmax >> 16) > 0x4380u;  // bf16(256.0) = 2^kRescaleThreshold
      };
      static_assert(kRescaleThreshold == 8.0f, "the bf16 constant above is 2^8");
      float alpha = 1.f;
      float neg_base = m_used == -INFINITY ? 0.f : -m_used;
      const bool fresh = m_used == -INFINITY;
      const bool any_fresh = __any_sync(0xffffffffu, fresh);
      if (any_fresh) exponentiate(neg_base, std::true_type{});
      else exponentiate(neg_base, std::false_type{});
      const bool move_base = fresh ? top > -INFINITY : (any_fresh ? top > kRescaleThreshold : over);
      if (__any_sync(0xffffffffu, move_base)) {
        if (!any_fresh) exponentiate(neg_base, std::true_type{});
        if (move_base) {
          const float mx = top - neg_base;
          alpha = fast_exp2(m_used - mx);
          m_used = mx;
          neg_base = -mx;
        }
        exponentiate(neg_base, std::false_type{});
        if (j > 0) {
          // PV(j - 1) is the last MMA that wrote O; PV(j) waits for this tile's P.
          if (!FW_WAIT(10, j, &bars->pv_done, (j - 1) & 1)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < kD / 32; ++c) {
            uint32_t o[32];
            tmem_ld32(o_addr + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st32(o_addr + c * 32, o);
          }
        }
      }
#pragma unroll
      for (int half = 0; half < kHalves; ++half)
        tmem_st32(s_addr + half * 32, packed[half]);  // P over the start of S: two bf16 keys per column
      l_run = l_run * alpha + sum;
      tmem_wait_st();
      // Last tile: zero the V rows past the valid keys (their P is 0, but 0 x NaN is not).
      if (pos0 + kBN > kv_end) {
        if (!FW_WAIT(12, j, &bars->v_full[s], (j / kStages) & 1)) {
          ok = false;
          break;
        }
        const int first_bad = kv_end - pos0;  // in [1, kBN - 1]
        uint8_t* vbase = smem + kSmemV + s * kTileBytes;
        for (int idx = row; idx < (kBN - first_bad) * (kD / 8); idx += 128) {
          const int r = first_bad + idx / (kD / 8), c = idx % (kD / 8);
          *reinterpret_cast<uint4*>(vbase + (c >> 3) * kKeyBlock + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
              make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[j & 1]);
    }

    // ---- epilogue: O / l -> bf16, lse
    if (ok && n_tiles > 0) ok = FW_WAIT(16, n_tiles - 1, &bars->pv_done, (n_tiles - 1) & 1);
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
      for (int c = 0; c < kD / 32; ++c) {
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

}  // namespace d256

// ---------------------------------------------------------------- host
bool tcgen05_d256_supported(const FwPrefillArgs* a) {
  const bool packed = a->block_table == nullptr && a->v_packed != nullptr;
  if (a->kv_dtype != FW_DTYPE_BF16 || a->head_dim != 256) return false;
  if (a->nheads_k <= 0 || a->nheads % a->nheads_k) return false;
  if (a->nheads / a->nheads_k > kBM) return false;
  if (!packed && (a->page_size <= 0 || a->page_size % 64)) return false;
  if (a->batch > 2048) return false;
  if (!(a->softmax_scale > 0.f)) return false;
  return true;
}

static int d256_max_items(const FwPrefillArgs* a) {
  const int qb = kBM / (a->nheads / a->nheads_k);  // query tokens per CTA
  return (a->total_q + qb - 1) / qb + a->batch;
}

uint64_t tcgen05_d256_workspace_bytes(const FwPrefillArgs* a) {
  return 256 + static_cast<uint64_t>(d256_max_items(a)) * 8 * sizeof(int);
}

template <int D, int BN>
static int launch_single_tile(const FwPrefillArgs* a, cudaStream_t stream) {
  using namespace d256;
  constexpr int kD = D;
  constexpr int kSmemBytes = Plan<D, BN>::kSmemBytes;
  auto kernel = prefill_tcgen05_d256_kernel<D, BN>;
  const bool packed = a->block_table == nullptr && a->v_packed != nullptr;
  if (packed) {
    const bool slots = a->kv_request_stride > 0 && a->seqused_k != nullptr;
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
  const uint64_t need = tcgen05_d256_workspace_bytes(a);
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
  const int max_items = d256_max_items(a);
  Tc05Params p;
  p.items = reinterpret_cast<int*>(static_cast<uint8_t*>(a->workspace) + 256);
  p.block_table = a->block_table;
  p.k_descale = a->k_descale;
  p.v_descale = a->v_descale;
  p.sinks = a->sinks;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.status = static_cast<int*>(a->workspace);
  if (a->token_major) {
    p.tok_stride = static_cast<long long>(a->nheads) * kD;
    p.head_stride = kD;
  } else {
    p.tok_stride = kD;
    p.head_stride = static_cast<long long>(a->total_q) * kD;
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

  int rc = launch_prefill_plan(a, tpb, max_items, const_cast<int*>(p.items), p.tok_stride, p.head_stride, p.status,
                               stream);
  if (rc != FW_OK) return rc;

  CUtensorMap map_q, map_kv, map_v;
  {
    const uint64_t dims[3] = {kD, static_cast<uint64_t>(a->total_q), static_cast<uint64_t>(a->nheads)};
    const uint64_t strides[2] = {static_cast<uint64_t>(p.tok_stride) * 2, static_cast<uint64_t>(p.head_stride) * 2};
    const uint32_t box[3] = {64, static_cast<uint32_t>(tpb), 1};
    rc = encode_tensor_map_bf16(&map_q, 3, a->q, dims, strides, box);
    if (rc != FW_OK) return rc;
  }
  if (packed) {
    const uint64_t dims[3] = {kD, static_cast<uint64_t>(a->total_k), static_cast<uint64_t>(a->nheads_k)};
    const uint64_t row = kD * 2;
    const uint64_t tok = a->kv_token_major ? static_cast<uint64_t>(a->nheads_k) * row : row;
    const uint64_t head = a->kv_token_major ? row : static_cast<uint64_t>(a->total_k) * row;
    const uint64_t strides[2] = {tok, head};
    const uint32_t box[3] = {64, 64, 1};
    rc = encode_tensor_map_bf16(&map_kv, 3, a->kv_cache, dims, strides, box);
    if (rc != FW_OK) return rc;
    rc = encode_tensor_map_bf16(&map_v, 3, a->v_packed, dims, strides, box);
    if (rc != FW_OK) return rc;
  } else {
    const uint64_t planes = 2ull * a->nheads_k;
    const uint64_t row_bytes = planes * kD * 2;
    const uint64_t dims[4] = {kD, planes, static_cast<uint64_t>(a->page_size), static_cast<uint64_t>(a->num_pages)};
    const uint64_t strides[3] = {kD * 2, row_bytes, row_bytes * a->page_size};
    const uint32_t box[4] = {64, 1, 64, 1};
    rc = encode_tensor_map_bf16(&map_kv, 4, a->kv_cache, dims, strides, box);
    if (rc != FW_OK) return rc;
    map_v = map_kv;
  }
  cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (err != cudaSuccess) {
    set_error("cudaFuncSetAttribute(%d bytes): %s", kSmemBytes, cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  dim3 grid(a->nheads_k, max_items);
  cudaLaunchAttribute pdl{};
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kernel, map_q, map_kv, map_v, p);
  err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("tcgen05 head_dim 256 kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

// The kernel is written for any (head_dim, keys per tile) whose O and two S
// buffers fit tensor memory; <128, 128> was measured against the two-stream
// kernel of prefill_tcgen05.cu and lost (849 vs 1008 TFLOP/s on the chunked
// prefill benchmark), so only <256, 64> is built.
int tcgen05_d256_prefill(const FwPrefillArgs* a, cudaStream_t stream) {
  return launch_single_tile<256, 64>(a, stream);
}

}  // namespace fw
