// Cross-GPU exchange of per-rank attention states: what the sending side (the
// decode launch's combine kernel, or the stand-alone scatter kernel) and the
// merging side share.
//
// Every float travels as an 8-byte pair {value, epoch}, written with one store,
// so the data is its own flag: the receiver polls the pairs it needs until they
// carry the epoch of the step, and neither side issues a system-scope fence or
// raises a separate flag.  (An 8-byte aligned store is delivered whole; two
// pairs go out as one 16-byte vector store and both epochs are checked.)
//
// Layout of a rank's exchange buffer (the same on every rank):
//   [0, 4096)     this rank's own bookkeeping: word 0 = epoch of the last
//                 completed step, word 1 = merge blocks done
//   [4096, ...)   2 x world slots of slot_pairs pairs: rows * head_dim pairs of
//                 o, then rows pairs of lse; indexed [epoch parity][source rank]
// Two parities, because a rank may run one step ahead of a peer that is still
// merging the previous one; it cannot run two ahead, since its own merge of
// step e + 1 needs that peer's state of step e + 1, which the peer sends only
// after its merge of step e.
#pragma once

#include "common.cuh"

namespace fw {

constexpr int kMaxRanks = 16;
constexpr uint64_t kExchangeHeader = 4096;
constexpr uint32_t kExchangePollLimit = 1u << 20;  // polls of a row before giving up (about a second)

struct PeerSlots {
  uint8_t* peers[kMaxRanks];  // every rank's exchange buffer as mapped in this process (own included)
  int world, rank;            // world == 0: no exchange
  uint64_t slot_pairs;        // rows * (head_dim + 1), rounded up to an even count
};

// Pairs of one (o, lse) slot; even, so every slot starts on a 16-byte boundary.
__host__ __device__ inline uint64_t slot_pairs_of(int rows, int head_dim) {
  return (static_cast<uint64_t>(rows) * (head_dim + 1) + 1) & ~1ull;
}

__device__ __forceinline__ uint2* slot_of(uint8_t* buffer, uint32_t epoch, int world, int source,
                                          uint64_t slot_pairs) {
  return reinterpret_cast<uint2*>(buffer + kExchangeHeader) +
         (static_cast<uint64_t>(epoch & 1) * world + source) * slot_pairs;
}

// The epoch of the step being enqueued: one past the last step this rank's
// merge completed (kernels of a step run after that merge in stream order).
__device__ __forceinline__ uint32_t step_epoch(const uint8_t* own_buffer) {
  return *reinterpret_cast<const volatile uint32_t*>(own_buffer) + 1;
}

// Two pairs (16-byte aligned) / one pair.
__device__ __forceinline__ void store_pairs2(uint2* dst, float a, float b, uint32_t epoch) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(epoch),
               "r"(__float_as_uint(b)), "r"(epoch)
               : "memory");
}
__device__ __forceinline__ void store_pair(uint2* dst, float a, uint32_t epoch) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(epoch) : "memory");
}
// True when both pairs carry `epoch`.
__device__ __forceinline__ bool load_pairs2(const uint2* src, uint32_t epoch, float& a, float& b) {
  uint32_t va, ea, vb, eb;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(va), "=r"(ea), "=r"(vb), "=r"(eb)
               : "l"(src)
               : "memory");
  a = __uint_as_float(va);
  b = __uint_as_float(vb);
  return ea == epoch && eb == epoch;
}
__device__ __forceinline__ bool load_pair(const uint2* src, uint32_t epoch, float& a) {
  uint32_t va, ea;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(va), "=r"(ea) : "l"(src) : "memory");
  a = __uint_as_float(va);
  return ea == epoch;
}

// Merge side, enqueued as a programmatic dependent of the sending kernel.
struct MergeParams {
  PeerSlots slots;
  const float* sinks;
  __nv_bfloat16* out;
  float* lse;
  int* status;
  int rows, nheads, head_dim;
  int lse_head_stride, lse_token_stride;
  // round-robin bookkeeping advanced once the step is merged (NULL: none)
  int* global_len;
  int* local_len;
  int* append_enable;
  int page_size, advance;
};
int launch_gather_merge(const MergeParams& p, cudaStream_t stream);

// Tokens of the first `len` positions that fall in pages p with p % world == rank.
__host__ __device__ inline int round_robin_local_length(int len, int page_size, int world, int rank) {
  const int full_pages = len / page_size, tail = len - full_pages * page_size;
  // full pages owned: those p < full_pages with p % world == rank
  const int owned_full = full_pages > rank ? (full_pages - rank + world - 1) / world : 0;
  return owned_full * page_size + (full_pages % world == rank ? tail : 0);
}

}  // namespace fw
