// Shared device helpers for the sm_100a paged-KV attention kernels: mbarrier,
// TMA (non-multicast tiled bulk tensor copies), ldmatrix / mma.sync wrappers,
// bounded waits that report through a status word instead of spinning forever.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "flywheel_b200.h"

namespace fw {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Iteration cap of every device-side wait.  Each failed try_wait already
// blocks for a hardware-defined slice; with the back-off below the cap is on
// the order of a second, after which the waiter records FW_STATUS_WAIT_TIMEOUT
// and the kernel drains and returns.
constexpr uint32_t kWaitSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Non-blocking test of a phase (never suspends the thread).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred P1;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P1, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P1;\n\t"
      "}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false after `limit` failed polls or as soon as
// *abort_flag (shared memory) is set by another waiter of the same CTA.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag,
                                                  uint32_t limit = kWaitSpinLimit) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    // A sleeping warp leaves its issue slots to the warps that compute.
    // try_wait already parks the thread for a hardware time slice; back off
    // further only when the wait is clearly a long one.
    if (spin > 512) {
      if ((spin & 63) == 0 && *abort_flag) return false;
      __nanosleep(spin > 8192 ? 256 : 32);
    }
  }
  return false;
}

// ---------------------------------------------------------------- TMA
// Tiled 4-D bulk tensor load global -> this CTA's shared memory (no multicast).
// c0 is the innermost coordinate and must address a 16-byte boundary.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cta.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---------------------------------------------------------------- ldmatrix / mma.sync
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                            uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16) * B(16x8); bf16 or f16 operands.
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                        uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// tanh through exp2: 1 - 2 / (2^(2x*log2e) + 1); relative error ~1e-6, well
// inside what a softcap needs (tanh.approx would cost ~2^-11 absolute).
__device__ __forceinline__ float accurate_tanh(float x) {
  float e = fast_exp2(fminf(x * (2.0f * kLog2e), 80.0f));
  return 1.0f - 2.0f * fast_rcp(e + 1.0f);
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// Two fp8 values (low byte first) -> f16x2.
template <int KVT>
__device__ __forceinline__ uint32_t fp8x2_to_f16x2(uint16_t v) {
  uint32_t r;
  if constexpr (KVT == FW_DTYPE_E4M3) {
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  } else {
    asm("cvt.rn.f16x2.e5m2x2 %0, %1;" : "=r"(r) : "h"(v));
  }
  return r;
}
// The two fp8 values in the low (kHigh = false) or high half of a 32-bit word
// -> f16x2.  e5m2 is the top byte of an f16 (same sign, exponent and bias, two
// mantissa bits), so widening it is a byte placement: one prmt, no conversion,
// NaN and infinity patterns included.
template <int KVT, bool kHigh>
__device__ __forceinline__ uint32_t fp8_half_to_f16x2(uint32_t word) {
  if constexpr (KVT == FW_DTYPE_E5M2) {
    // result bytes (low to high): 0, b0, 0, b1 (or b2, b3); selector 4 picks a zero byte of the second operand
    return __byte_perm(word, 0u, kHigh ? 0x3424 : 0x1404);
  } else {
    return fp8x2_to_f16x2<KVT>(static_cast<uint16_t>(kHigh ? word >> 16 : word & 0xffffu));
  }
}

// Packed f32x2 arithmetic (two lanes per instruction on sm_100) and packed
// bf16x2 max: they halve the issue slots the softmax spends around each exp2.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint32_t max_f16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// Two f32 -> f16x2, out-of-range values clamped to the largest finite f16.
__device__ __forceinline__ uint32_t pack_f16_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}

// Records a failure in the device status word.  The codes are distinct bits and
// the word is their OR, so a clamped page id reported by an earlier launch does
// not hide a later timeout.  The word stays set until the host reads it.
__device__ __forceinline__ void report_status(int* status, int code) {
  if (status != nullptr) atomicOr(status, code);
}
// Word 4 of the status block says "the launch in flight is void": a bounded
// wait of this launch gave up, so CTAs that have not started yet may leave at
// once.  Unlike word 0 it is cleared at the head of every launch that uses it,
// so nothing an earlier launch reported can switch a later one off.
constexpr int kStatusLaunchVoidWord = 4;
__device__ __forceinline__ void report_timeout(int* status) {
  if (status == nullptr) return;
  atomicOr(status, FW_STATUS_WAIT_TIMEOUT);
  *reinterpret_cast<volatile int*>(status + kStatusLaunchVoidWord) = 1;
}
__device__ __forceinline__ bool launch_is_void(const int* status) {
  return status != nullptr && *reinterpret_cast<const volatile int*>(status + kStatusLaunchVoidWord) != 0;
}

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);
int sm_count();
// Encodes a byte-typed 4-D tiled tensor map with 128-byte swizzle; dims/box are
// innermost first, strides are for dims 1..3 in bytes.  Returns FW_OK or
// FW_ERR_LAUNCH with fw_last_error set.
int encode_tensor_map_u8_4d(CUtensorMap* map, const void* base, const uint64_t dims[4],
                            const uint64_t strides[3], const uint32_t box[4]);

// bf16-typed tiled tensor map of rank 3 or 4 with 128-byte swizzle; strides are
// for dims 1..rank-1 in bytes.
int encode_tensor_map_bf16(CUtensorMap* map, int rank, const void* base, const uint64_t* dims,
                           const uint64_t* strides, const uint32_t* box);

// Query-block table for chunked prefill (decode.cu): cuts every active request
// into blocks of qb tokens, writes 8 ints per block into items[0..max_items),
// clears the packed rows no active request owns and clears the "launch is void"
// word of the status block for the attention kernel that follows.
int launch_prefill_plan(const FwPrefillArgs* args, int qb, int max_items, int* items, long long tok_stride,
                        long long head_stride, int* status, cudaStream_t stream);

// Chunked prefill on tcgen05 tensor cores (prefill_tcgen05.cu).
bool tcgen05_prefill_supported(const FwPrefillArgs* args);
uint64_t tcgen05_prefill_workspace_bytes(const FwPrefillArgs* args);
int tcgen05_prefill(const FwPrefillArgs* args, cudaStream_t stream);

// The same at head_dim 256 (prefill_tcgen05_d256.cu); the three entry points
// above hand over to these when head_dim is 256.
bool tcgen05_d256_supported(const FwPrefillArgs* args);
uint64_t tcgen05_d256_workspace_bytes(const FwPrefillArgs* args);
int tcgen05_d256_prefill(const FwPrefillArgs* args, cudaStream_t stream);

// fw_decode_kvcache reporting to `status` instead of the head of its workspace (decode.cu).
int decode_with_status(const FwDecodeArgs* args, int* status, cudaStream_t stream);

// Chunked prefill through the split-KV decode kernel (decode.cu).
uint64_t splitkv_prefill_workspace_bytes(const FwPrefillArgs* args);
int splitkv_prefill(const FwPrefillArgs* args, cudaStream_t stream);

}  // namespace fw
