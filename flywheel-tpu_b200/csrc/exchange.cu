// Cross-GPU exchange of per-rank attention states for one long request whose KV
// pages are split over the GPUs of a node, fused with the merge: every rank
// stores its sink-free (o, lse) state straight into each peer's memory over
// NVLink (plain peer stores, no multicast), raises a per-rank epoch flag there,
// and the merge kernel waits - with an iteration limit - for the flags of all
// ranks before it reads the gathered states from its own memory.  It replaces
// an NCCL all-gather of 33 KB plus a merge launch.
//
// The merge itself is _merge_states of the reference project
// (patches/tpu-inference.patch:7174-7186); the reference has no multi-device
// code in its library, the exchange is this build's.
//
// Layout of a rank's exchange buffer (same on every rank, cudaMalloc'ed here so
// its IPC handle can be opened by the peers):
//   [0, 256)            this rank's own bookkeeping: step counter, merge blocks done,
//                       scatter blocks done per peer
//   [256, 256 + 4 W)    flags[r]: last epoch rank r has delivered
//   [4096, ...)         2 x W slots of rows * (head_dim + 1) floats: [o | lse],
//                       indexed [epoch parity][source rank]
// Two parities, because a rank may run one step ahead of a peer that is still
// merging the previous one; it cannot run two ahead, since its own merge of
// step e + 1 needs that peer's state of step e + 1.
#include <cstring>

#include "common.cuh"

namespace fw {

constexpr int kMaxRanks = 16;
constexpr uint64_t kExchangeHeader = 4096;
constexpr uint32_t kExchangePollLimit = 1u << 21;  // polls of a peer's flag before giving up (about a second)

struct ExchangeParams {
  uint8_t* peers[kMaxRanks];  // every rank's exchange buffer as mapped in this process (own included)
  const float* state_out;     // (rows, head_dim) this rank's normalised partial output
  const float* state_lse;     // (rows,)
  const float* sinks;
  __nv_bfloat16* out;
  float* lse;
  int* status;
  int world, rank, rows, nheads, head_dim;
  int lse_head_stride, lse_token_stride;
  uint64_t slot_floats;  // rows * (head_dim + 1), rounded up to a multiple of 4
};

__device__ __forceinline__ void store_release_sys(uint32_t* addr, uint32_t value) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* addr) {
  uint32_t value;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(addr) : "memory");
  return value;
}

__device__ __forceinline__ float* slot_of(uint8_t* buffer, uint32_t epoch, int world, int source,
                                          uint64_t slot_floats) {
  return reinterpret_cast<float*>(buffer + kExchangeHeader) +
         (static_cast<uint64_t>(epoch & 1) * world + source) * slot_floats;
}

constexpr int kScatterBlocks = 8;  // blocks that share the copy to one peer

// Blocks (p, 0 .. kScatterBlocks) deliver this rank's state to rank p; the last
// of them to finish raises this rank's flag there.
__global__ void __launch_bounds__(128) scatter_state_kernel(const ExchangeParams p) {
  const int peer = blockIdx.x;
  uint32_t* header = reinterpret_cast<uint32_t*>(p.peers[p.rank]);
  // Launched as a programmatic dependent of the kernel that writes the state
  // (and, through it, of the previous step's merge, which advances the epoch).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t epoch = header[0] + 1;
  float* dst = slot_of(p.peers[peer], epoch, p.world, p.rank, p.slot_floats);
  const int n_out = p.rows * p.head_dim;
  const int first = (blockIdx.y * blockDim.x + threadIdx.x) * 4, stride = gridDim.y * blockDim.x * 4;
  for (int i = first; i < n_out; i += stride)
    *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(p.state_out + i);
  if (blockIdx.y == 0)
    for (int i = threadIdx.x; i < p.rows; i += blockDim.x) dst[n_out + i] = p.state_lse[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();  // this block's stores are out before it is counted
    uint32_t* arrived = header + 2 + peer;
    if (atomicAdd(arrived, 1u) == gridDim.y - 1) {
      *arrived = 0;
      __threadfence_system();
      store_release_sys(reinterpret_cast<uint32_t*>(p.peers[peer] + 256) + p.rank, epoch);
    }
  }
}

// One warp per row, after every rank's flag shows this step's epoch.  The last
// block to finish advances the step counter.
__global__ void __launch_bounds__(128) gather_merge_kernel(const ExchangeParams p) {
  __shared__ int failed;
  uint8_t* mine = p.peers[p.rank];
  uint32_t* header = reinterpret_cast<uint32_t*>(mine);
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the scatter kernel of this rank is done
  const uint32_t epoch = header[0] + 1;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const uint32_t* flag = reinterpret_cast<const uint32_t*>(mine + 256) + threadIdx.x;
    bool seen = false;
    for (uint32_t poll = 0; poll < kExchangePollLimit; ++poll) {
      // epochs only grow; the signed difference survives a wrap of the counter
      if (static_cast<int32_t>(load_acquire_sys(flag) - epoch) >= 0) {
        seen = true;
        break;
      }
      if (poll > 64) __nanosleep(poll > 4096 ? 512 : 64);
    }
    if (!seen) {
      failed = 1;
      report_status(p.status, FW_STATUS_WAIT_TIMEOUT);
    }
  }
  __syncthreads();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (!failed && row < p.rows) {
    const int head = row % p.nheads, tok = row / p.nheads;
    const int n_out = p.rows * p.head_dim;
    const float sink = p.sinks ? p.sinks[head] : -INFINITY;
    float top = sink;
    for (int r = 0; r < p.world; ++r)
      top = fmaxf(top, slot_of(mine, epoch, p.world, r, p.slot_floats)[n_out + row]);
    const int blocks = p.head_dim / 128;
    float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
    float den = 0.f;
    if (top != -INFINITY) {
      for (int r = 0; r < p.world; ++r) {
        const float* slot = slot_of(mine, epoch, p.world, r, p.slot_floats);
        const float l = slot[n_out + row];
        if (l == -INFINITY) continue;
        const float w = __expf(l - top);
        den += w;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          if (nb >= blocks) break;
          const float4 o = *reinterpret_cast<const float4*>(slot + static_cast<long long>(row) * p.head_dim +
                                                            nb * 128 + lane * 4);
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
  // the step is over once every block has read the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&header[1], 1u) == gridDim.x - 1) {
      header[1] = 0;
      __threadfence();
      header[0] = epoch;
    }
  }
}

// Floats of one (o, lse) slot, padded so every slot starts on a 16-byte boundary.
static uint64_t slot_floats_of(int rows, int head_dim) {
  return (static_cast<uint64_t>(rows) * (head_dim + 1) + 3) & ~3ull;
}

}  // namespace fw

using namespace fw;

extern "C" uint64_t fw_exchange_buffer_bytes(int32_t world, int32_t rows, int32_t head_dim) {
  if (world <= 0 || world > kMaxRanks || rows <= 0 || (head_dim != 128 && head_dim != 256)) {
    set_error("exchange buffer: world must be in [1, %d], rows positive, head_dim 128 or 256.", kMaxRanks);
    return 0;
  }
  return kExchangeHeader + 2ull * world * slot_floats_of(rows, head_dim) * sizeof(float);
}

extern "C" int fw_peer_alloc(uint64_t bytes, void** ptr, void* handle64) {
  if (ptr == nullptr || handle64 == nullptr || bytes == 0) {
    set_error("fw_peer_alloc: ptr and handle must not be NULL and bytes positive.");
    return FW_ERR_BAD_SHAPE;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed around as 64 bytes");
  cudaError_t err = cudaMalloc(ptr, bytes);
  if (err == cudaSuccess) err = cudaMemset(*ptr, 0, bytes);
  if (err == cudaSuccess) err = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), *ptr);
  if (err != cudaSuccess) {
    set_error("fw_peer_alloc(%llu bytes): %s", static_cast<unsigned long long>(bytes), cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_peer_open(const void* handle64, void** ptr) {
  if (ptr == nullptr || handle64 == nullptr) {
    set_error("fw_peer_open: ptr and handle must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  cudaIpcMemHandle_t handle;
  memcpy(&handle, handle64, sizeof(handle));
  cudaError_t err = cudaIpcOpenMemHandle(ptr, handle, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) {
    set_error("fw_peer_open: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_peer_close(void* ptr) {
  cudaError_t err = cudaIpcCloseMemHandle(ptr);
  if (err != cudaSuccess) {
    set_error("fw_peer_close: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_peer_free(void* ptr) {
  cudaError_t err = cudaFree(ptr);
  if (err != cudaSuccess) {
    set_error("fw_peer_free: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_state_exchange_merge(const FwExchangeArgs* a, void* stream_ptr) {
  if (a == nullptr || a->peer_buffers == nullptr || a->state_out == nullptr || a->state_lse == nullptr ||
      a->out == nullptr) {
    set_error("peer_buffers, state_out, state_lse and out must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->world <= 0 || a->world > kMaxRanks || a->rank < 0 || a->rank >= a->world) {
    set_error("world must be in [1, %d] and rank inside it; got world %d rank %d.", kMaxRanks, a->world, a->rank);
    return FW_ERR_BAD_SHAPE;
  }
  if (a->head_dim != 128 && a->head_dim != 256) {
    set_error("head_dim %d is not built; this library serves head_dim 128 and 256.", a->head_dim);
    return FW_ERR_UNSUPPORTED;
  }
  if (a->rows <= 0 || a->nheads <= 0) {
    set_error("rows and nheads must be positive.");
    return FW_ERR_BAD_SHAPE;
  }
  ExchangeParams p{};
  for (int r = 0; r < a->world; ++r) {
    if (a->peer_buffers[r] == nullptr) {
      set_error("peer_buffers[%d] is NULL.", r);
      return FW_ERR_BAD_SHAPE;
    }
    p.peers[r] = static_cast<uint8_t*>(a->peer_buffers[r]);
  }
  p.state_out = a->state_out;
  p.state_lse = a->state_lse;
  p.sinks = a->sinks;
  p.out = static_cast<__nv_bfloat16*>(a->out);
  p.lse = a->lse;
  p.status = a->status;
  p.world = a->world;
  p.rank = a->rank;
  p.rows = a->rows;
  p.nheads = a->nheads;
  p.head_dim = a->head_dim;
  p.lse_head_stride = a->lse_head_stride;
  p.lse_token_stride = a->lse_token_stride;
  p.slot_floats = slot_floats_of(a->rows, a->head_dim);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  // Both kernels are programmatic dependents of the kernel before them in the
  // stream: their launch latency hides under it, and each starts with
  // griddepcontrol.wait before it reads anything.
  cudaLaunchAttribute pdl{};
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3(a->world, kScatterBlocks);
  cfg.blockDim = dim3(128);
  cudaError_t err = cudaLaunchKernelEx(&cfg, scatter_state_kernel, p);
  if (err == cudaSuccess) {
    cfg.gridDim = dim3((a->rows + 3) / 4);
    err = cudaLaunchKernelEx(&cfg, gather_merge_kernel, p);
  }
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("exchange kernels launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

// ---------------------------------------------------------------- round-robin page ownership
namespace fw {

// Tokens of the first `len` positions that fall in pages p with p % world == rank.
__host__ __device__ inline int round_robin_local_length(int len, int page_size, int world, int rank) {
  const int full_pages = len / page_size, tail = len - full_pages * page_size;
  // full pages owned: those p < full_pages with p % world == rank
  const int owned_full = full_pages > rank ? (full_pages - rank + world - 1) / world : 0;
  return owned_full * page_size + (full_pages % world == rank ? tail : 0);
}

__global__ void shard_step_kernel(const FwShardStepArgs a) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int len = max(*a.global_len, 0);
  *a.local_len = round_robin_local_length(len, a.page_size, a.world, a.rank);
  *a.append_enable = (len / a.page_size) % a.world == a.rank ? 1 : 0;
  *a.global_len = len + a.advance;
}

}  // namespace fw

extern "C" int fw_shard_step(const FwShardStepArgs* a, void* stream_ptr) {
  if (a == nullptr || a->global_len == nullptr || a->local_len == nullptr || a->append_enable == nullptr) {
    fw::set_error("global_len, local_len and append_enable must be device pointers, not NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if (a->page_size <= 0 || a->world <= 0 || a->rank < 0 || a->rank >= a->world || a->advance < 0) {
    fw::set_error("page_size and world must be positive, 0 <= rank < world, advance >= 0; got %d, %d, %d, %d.",
                  a->page_size, a->world, a->rank, a->advance);
    return FW_ERR_BAD_SHAPE;
  }
  fw::shard_step_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream_ptr)>>>(*a);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    fw::set_error("shard step launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}
