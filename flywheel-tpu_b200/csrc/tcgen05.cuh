// Building blocks shared by the tcgen05 attention kernels: the launch
// parameters, tcgen05 / tensor-memory PTX wrappers, shared-memory and
// instruction descriptors, packed f32x2 arithmetic and the softmax passes.
#pragma once

#include <climits>
#include <type_traits>

#include "common.cuh"

namespace fw {

constexpr int kBM = 128;                   // query rows of one MMA tile (TMEM lanes)
constexpr float kRescaleThreshold = 8.0f;  // log2 units a row max may drift before O is rescaled

struct Tc05Params {
  const int* items;  // 8 ints per query block: request, first q row, valid tokens, diagonal anchor, kv length
  const int* block_table;
  const float* k_descale;
  const float* v_descale;
  const float* sinks;
  __nv_bfloat16* out;
  float* lse;
  int* status;
  long long tok_stride, head_stride;  // elements, shared by q and out
  long long num_pages;
  int total_q, nheads, group, tpb, page_size, pages_per_seq;
  int right, window_left;  // keys up to `right` past a row's diagonal are visible (0 = causal); -1 = no bound
  float scale, softcap;
  int packed;       // K and V are packed tensors addressed by token (no block table)
  int sink_period;  // head h uses sinks[h % sink_period]; 0 = one sink per head
  // Rotary embedding of Q inside the kernel (rotary.py:27-215 of the reference
  // rotates Q in its attention kernel too): NULL, or (rotary_len, head_dim / 2)
  // cos / sin tables, f32 or bf16.  A query row on diagonal `pos` is rotated at
  // position pos in f32 and rounded once to bf16; positions past the table stay
  // as they are.
  const void* rotary_cos;
  const void* rotary_sin;
  int rotary_len, rotary_interleaved, rotary_bf16;
};

__device__ __forceinline__ float rotary_entry(const void* table, long long index, int is_bf16) {
  return is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(table)[index])
                 : static_cast<const float*>(table)[index];
}

// Rotates one query row that a TMA copy left in shared memory as D / 64 blocks
// of [rows][128 B] with the 128-byte swizzle (16-byte chunk c of row r sits at
// r * 128 + ((c ^ (r & 7)) << 4) inside its block; `block_bytes` apart).  The
// caller owns the row; it must fence the generic-proxy writes before the tensor
// core reads them.
template <int D>
__device__ __forceinline__ void rotate_q_row_in_smem(uint8_t* q_tile, int block_bytes, int row, int pos,
                                                     const Tc05Params& p) {
  constexpr int kHalf = D / 2;
  auto chunk_ptr = [&](int element) {  // the 16-byte chunk holding `element` (a multiple of 8) of this row
    const int block = element >> 6, c = (element & 63) >> 3;
    return reinterpret_cast<uint4*>(q_tile + block * block_bytes + row * 128 + ((c ^ (row & 7)) << 4));
  };
  const long long base = static_cast<long long>(pos) * kHalf;
  if (!p.rotary_interleaved) {
    // element i pairs with element i + D / 2
#pragma unroll
    for (int i0 = 0; i0 < kHalf; i0 += 8) {
      uint4* pa = chunk_ptr(i0);
      uint4* pb = chunk_ptr(i0 + kHalf);
      uint4 a = *pa, b = *pb;
      __nv_bfloat16* x1 = reinterpret_cast<__nv_bfloat16*>(&a);
      __nv_bfloat16* x2 = reinterpret_cast<__nv_bfloat16*>(&b);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = rotary_entry(p.rotary_cos, base + i0 + i, p.rotary_bf16);
        const float sn = rotary_entry(p.rotary_sin, base + i0 + i, p.rotary_bf16);
        const float u = __bfloat162float(x1[i]), w = __bfloat162float(x2[i]);
        x1[i] = __float2bfloat16_rn(u * c - w * sn);
        x2[i] = __float2bfloat16_rn(u * sn + w * c);
      }
      *pa = a;
      *pb = b;
    }
  } else {
    // elements (2 i, 2 i + 1) form pair i
#pragma unroll
    for (int e0 = 0; e0 < D; e0 += 8) {
      uint4* pa = chunk_ptr(e0);
      uint4 a = *pa;
      __nv_bfloat16* x = reinterpret_cast<__nv_bfloat16*>(&a);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float c = rotary_entry(p.rotary_cos, base + (e0 >> 1) + i, p.rotary_bf16);
        const float sn = rotary_entry(p.rotary_sin, base + (e0 >> 1) + i, p.rotary_bf16);
        const float u = __bfloat162float(x[2 * i]), w = __bfloat162float(x[2 * i + 1]);
        x[2 * i] = __float2bfloat16_rn(u * c - w * sn);
        x[2 * i + 1] = __float2bfloat16_rn(u * sn + w * c);
      }
      *pa = a;
    }
  }
}

// ---------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// The MMAs are issued by one thread, so every instruction between two of them
// is on the tensor pipe's critical path: descriptors are built once per tile
// and advanced by adding a constant to their address field (low 32 bits never
// carry: shared addresses stay below 2^18), and the accumulate predicate is
// only materialised where it is not a constant.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }

// D(tmem) (+)= A(tmem) * B(smem): A is 128 lanes x (K/2) 32-bit columns of packed bf16.
__device__ __forceinline__ void tc_mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D(tmem) (+)= A(smem) * B(smem), bf16 operands, f32 accumulate.
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31,%32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
      "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
      "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
      "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle, sm_100 version bits.
// K-major operand: rows of 128 B, 8-row groups 1024 B apart (SBO); LBO unused.
// MN-major operand: 64-element (128 B) runs along MN, next run LBO bytes away,
// next group of 8 K-rows SBO bytes away.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3fff);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}

// kind::f16 instruction descriptor: f32 accumulate, A and B both bf16 (format 1)
// or both f16 (format 0), M = 128.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn_major, bool f16_operands = false) {
  return (1u << 4) | (f16_operands ? 0u : (1u << 7) | (1u << 10)) | (b_mn_major ? (1u << 16) : 0u) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(kBM >> 4) << 24);
}

// One row of a Q tile in shared memory (128-byte swizzle, 64-element blocks
// `block_bytes` apart) converted in place from bf16 to f16, finite values kept
// finite.  Element positions do not change, so the swizzle does not matter.
template <int D>
__device__ __forceinline__ void q_row_bf16_to_f16_in_smem(uint8_t* q_tile, int block_bytes, int row) {
#pragma unroll
  for (int block = 0; block < D / 64; ++block)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4* ptr = reinterpret_cast<uint4*>(q_tile + block * block_bytes + row * 128 + (c << 4));
      uint4 v = *ptr;
      auto convert = [](uint32_t two_bf16) {
        return pack_f16_sat(__uint_as_float(two_bf16 << 16), __uint_as_float(two_bf16 & 0xffff0000u));
      };
      v.x = convert(v.x);
      v.y = convert(v.y);
      v.z = convert(v.z);
      v.w = convert(v.w);
      *ptr = v;
    }
}

// 2^y for two scores, on the special-function unit (two ex2.approx) or, with
// kPoly, on the FMA pipe: y is split into its nearest integer n (adding
// 1.5 * 2^23 leaves n in the low mantissa bits) and f = y - n in [-0.5, 0.5],
// 2^f is a cubic (maximum relative error 7.5e-5, far below the bf16 rounding P
// gets next), and n goes into the exponent field by an integer add.  y is
// clamped to [-126, 126]: the low end gives a subnormal that rounds to nothing,
// 126 still trips the rescale check.
// FW_EXP2_POLY_EVERY = n sends every n-th pair of scores down the FMA-pipe form.
// It is off: measured on B200 on the chunked-prefill benchmark workload (rounds
// of 0.5 s, power-capped clocks) the kernel ran 877 TFLOP/s with none, 795 with
// every 4th pair, 775 with every 3rd, 723 with every 2nd - the softmax warps are
// short of issue slots, not of special-function throughput.
#ifndef FW_EXP2_POLY_EVERY
#define FW_EXP2_POLY_EVERY 0
#endif
// Experiment switches of the softmax inner loop (see the measurements beside the
// defaults): FW_EXP2_BF16X2 computes both exponentials of a pair with one
// ex2.approx.ftz.bf16x2; FW_OVER_BY_SUM detects a score that outran the exponent
// base from the row sum instead of a running bf16 max of P.
#ifndef FW_EXP2_BF16X2
#define FW_EXP2_BF16X2 0
#endif
#ifndef FW_OVER_BY_SUM
#define FW_OVER_BY_SUM 0
#endif
__device__ __forceinline__ uint32_t exp2_bf16x2(uint32_t y) {
  uint32_t r;
  asm("ex2.approx.ftz.bf16x2 %0, %1;" : "=r"(r) : "r"(y));
  return r;
}

template <bool kPoly>
__device__ __forceinline__ void exp2_pair(uint64_t y2, float& p0, float& p1) {
  float y0, y1;
  unpack2(y2, y0, y1);
  if constexpr (!kPoly) {
    p0 = fast_exp2(y0);
    p1 = fast_exp2(y1);
  } else {
    const uint64_t yc = pack2(fminf(fmaxf(y0, -126.f), 126.f), fminf(fmaxf(y1, -126.f), 126.f));
    const uint64_t t = add2(yc, pack2(12582912.f, 12582912.f));
    const uint64_t nf = add2(t, pack2(-12582912.f, -12582912.f));
    const uint64_t f = fma2(nf, pack2(-1.f, -1.f), yc);
    uint64_t poly = fma2(pack2(0.0551716685f, 0.0551716685f), f, pack2(0.2426111251f, 0.2426111251f));
    poly = fma2(poly, f, pack2(0.6932609677f, 0.6932609677f));
    poly = fma2(poly, f, pack2(0.9999280572f, 0.9999280572f));
    float t0, t1, q0, q1;
    unpack2(t, t0, t1);
    unpack2(poly, q0, q1);
    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
  }
}

// Pass 1 of the softmax over one 64-key row: optional softcap (scores become
// log2-unit logits in place), optional mask (-inf in place), returns the row
// max of what is left in `sr` (raw scores without a softcap).
template <bool kSoftcap, bool kMask>
__device__ __forceinline__ float transform_row(uint32_t (&sr)[2][32], float c1, float c2, int pos0, int kv_end,
                                               int diag, int right, int window_left) {
  float mx0 = -INFINITY, mx1 = -INFINITY;
  const int hi = right >= 0 ? min(kv_end - 1, diag + right) : kv_end - 1;  // last visible key
  const int lo = window_left >= 0 ? diag - window_left : INT_MIN;    // first visible key
#pragma unroll
  for (int c = 0; c < 2; ++c)
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float x0 = __uint_as_float(sr[c][i]), x1 = __uint_as_float(sr[c][i + 1]);
      if constexpr (kSoftcap) {
        x0 = accurate_tanh(x0 * c1) * c2;
        x1 = accurate_tanh(x1 * c1) * c2;
      }
      if constexpr (kMask) {
        const int key = pos0 + c * 32 + i;
        if (key < lo || key > hi) x0 = -INFINITY;
        if (key + 1 < lo || key + 1 > hi) x1 = -INFINITY;
      }
      if constexpr (kSoftcap || kMask) {
        sr[c][i] = __float_as_uint(x0);
        sr[c][i + 1] = __float_as_uint(x1);
      }
      mx0 = fmaxf(mx0, x0);
      mx1 = fmaxf(mx1, x1);
    }
  return fmaxf(mx0, mx1);
}

// First waiter that gives up leaves where it was: status[1] = wait site,
// status[2] = tile index, status[3] = item | kv head << 20.
__device__ __forceinline__ void record_timeout(int* status, int site, int j) {
  if (status != nullptr && atomicCAS(status + 1, 0, site) == 0) {
    status[2] = j;
    status[3] = static_cast<int>(blockIdx.y | (blockIdx.x << 20));
  }
}

// Abort path only: a short bounded wait that lets copies or MMAs that are
// already in flight land before the CTA gives its shared and tensor memory up.
__device__ __forceinline__ void drain_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t spin = 0; spin < (1u << 16) && !mbar_try_wait(bar, parity); ++spin) __nanosleep(64);
}

#define FW_WAIT(site, j, bar, parity) \
  (mbar_wait_bounded(bar, parity, abort_flag) || (record_timeout(p.status, site, j), false))

}  // namespace fw
