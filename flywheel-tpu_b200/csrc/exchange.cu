// Cross-GPU exchange of per-rank attention states for one long request whose KV
// pages are split over the GPUs of a node, fused with the merge.  The sending
// side stores its sink-free (o, lse) state straight into each peer's memory
// over NVLink (plain peer stores, no multicast) as {value, epoch} pairs
// (exchange.cuh); the merge kernel polls - with an iteration limit - the pairs
// it needs in its own memory until they carry the step's epoch, so a step has
// no flag, no system-scope fence and no collective-library call.  The sender is
// normally the decode launch's own combine kernel (fw_sharded_decode_step,
// decode.cu); scatter_state_kernel below serves callers that already hold the
// state in a buffer.
//
// The merge itself is _merge_states of the reference project
// (patches/tpu-inference.patch:7174-7186); the reference has no multi-device
// code in its library, the exchange is this build's.
#include <cstring>

#include "exchange.cuh"

namespace fw {

struct ScatterParams {
  PeerSlots slots;
  const float* state_out;  // (rows, head_dim) this rank's normalised partial output
  const float* state_lse;  // (rows,)
  int rows, head_dim;
};

constexpr int kScatterBlocks = 8;  // blocks that share the copy to one peer

// Blocks (p, 0 .. kScatterBlocks) deliver this rank's state to rank p.
__global__ void __launch_bounds__(128) scatter_state_kernel(const ScatterParams p) {
  const int peer = blockIdx.x;
  // Launched as a programmatic dependent of the kernel that writes the state
  // (and, through it, of the previous step's merge, which advances the epoch).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const uint32_t epoch = step_epoch(p.slots.peers[p.slots.rank]);
  uint2* dst = slot_of(p.slots.peers[peer], epoch, p.slots.world, p.slots.rank, p.slots.slot_pairs);
  const int n_out = p.rows * p.head_dim;
  const int first = (blockIdx.y * blockDim.x + threadIdx.x) * 4, stride = gridDim.y * blockDim.x * 4;
  for (int i = first; i < n_out; i += stride) {
    const float4 v = *reinterpret_cast<const float4*>(p.state_out + i);
    store_pairs2(dst + i, v.x, v.y, epoch);
    store_pairs2(dst + i + 2, v.z, v.w, epoch);
  }
  if (blockIdx.y == 0)
    for (int i = threadIdx.x; i < p.rows; i += blockDim.x) store_pair(dst + n_out + i, p.state_lse[i], epoch);
}

// One warp per row: waits until every rank's pairs of that row carry this
// step's epoch, merges them, and the last block to finish advances the epoch
// (and the round-robin bookkeeping, when given).
__global__ void __launch_bounds__(128) gather_merge_kernel(const MergeParams p) {
  uint8_t* mine = p.slots.peers[p.slots.rank];
  uint32_t* header = reinterpret_cast<uint32_t*>(mine);
  // No griddepcontrol.wait: the pairs carry their own validity, so the blocks may
  // start polling while this rank's sending kernel still runs.  (That kernel
  // releases its dependents only after the decode grid is complete; the epoch
  // below was advanced by the previous step's merge, long done; and the last
  // block's bookkeeping runs only after every row of every rank - this rank's
  // sender included - has been delivered.)
  const uint32_t epoch = step_epoch(mine);
  const int world = p.slots.world;
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row < p.rows) {
    const int head = row % p.nheads, tok = row / p.nheads;
    const int n_out = p.rows * p.head_dim;
    const int blocks = p.head_dim / 128;
    const float sink = p.sinks ? p.sinks[head] : -INFINITY;
    // Running (max, sum, acc) over the ranks, in rank order, so every rank
    // computes bit-identical results.
    float top = -INFINITY, den = 0.f;
    float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
    bool failed = false;
    for (int r = 0; r < world && !failed; ++r) {
      const uint2* slot = slot_of(mine, epoch, world, r, p.slots.slot_pairs);
      const uint2* o_pairs = slot + static_cast<long long>(row) * p.head_dim + lane * 4;
      float4 o[2];
      float l = 0.f;
      bool seen = false;
      for (uint32_t poll = 0; poll < kExchangePollLimit; ++poll) {
        bool ok = load_pair(slot + n_out + row, epoch, l);
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          if (nb >= blocks) break;
          ok &= load_pairs2(o_pairs + nb * 128, epoch, o[nb].x, o[nb].y);
          ok &= load_pairs2(o_pairs + nb * 128 + 2, epoch, o[nb].z, o[nb].w);
        }
        if (__all_sync(0xffffffffu, ok)) {
          seen = true;
          break;
        }
        if (poll > 64) __nanosleep(poll > 4096 ? 512 : 64);
      }
      if (!seen) {
        failed = true;
        if (lane == 0) report_status(p.status, FW_STATUS_WAIT_TIMEOUT);
        break;
      }
      if (l == -INFINITY) continue;
      const float m_new = fmaxf(top, l);
      const float keep = __expf(top - m_new), w = __expf(l - m_new);  // e^-inf = 0
      den = den * keep + w;
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        if (nb >= blocks) break;
        acc[nb].x = acc[nb].x * keep + o[nb].x * w;
        acc[nb].y = acc[nb].y * keep + o[nb].y * w;
        acc[nb].z = acc[nb].z * keep + o[nb].z * w;
        acc[nb].w = acc[nb].w * keep + o[nb].w * w;
      }
      top = m_new;
    }
    if (sink != -INFINITY && !failed) {
      const float m_new = fmaxf(top, sink);
      const float keep = __expf(top - m_new);
      den = den * keep + __expf(sink - m_new);
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        acc[nb].x *= keep;
        acc[nb].y *= keep;
        acc[nb].z *= keep;
        acc[nb].w *= keep;
      }
      top = m_new;
    }
    const float inv = den > 0.f && !failed ? 1.f / den : 0.f;
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
          den > 0.f && !failed ? top + logf(den) : -INFINITY;
  }
  // the step is over once every block has read the epoch
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&header[1], 1u) == gridDim.x - 1) {
      header[1] = 0;
      if (p.global_len != nullptr) {
        // what fw_shard_step does ahead of a step, done for the next one
        const int len = max(*p.global_len, 0) + p.advance;
        *p.global_len = len;
        *p.local_len = round_robin_local_length(len, p.page_size, world, p.slots.rank);
        *p.append_enable = (len / p.page_size) % world == p.slots.rank ? 1 : 0;
      }
      __threadfence();
      header[0] = epoch;
    }
  }
}

int launch_gather_merge(const MergeParams& p, cudaStream_t stream) {
  cudaLaunchAttribute pdl{};
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg{};
  cfg.stream = stream;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cfg.gridDim = dim3((p.rows + 3) / 4);
  cfg.blockDim = dim3(128);
  cudaError_t err = cudaLaunchKernelEx(&cfg, gather_merge_kernel, p);
  if (err == cudaSuccess) err = cudaGetLastError();
  if (err != cudaSuccess) {
    set_error("merge kernel launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

}  // namespace fw

using namespace fw;

extern "C" uint64_t fw_exchange_buffer_bytes(int32_t world, int32_t rows, int32_t head_dim) {
  if (world <= 0 || world > kMaxRanks || rows <= 0 || (head_dim != 128 && head_dim != 256)) {
    set_error("exchange buffer: world must be in [1, %d], rows positive, head_dim 128 or 256.", kMaxRanks);
    return 0;
  }
  return kExchangeHeader + 2ull * world * slot_pairs_of(rows, head_dim) * sizeof(uint2);
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
  if (a == nullptr || a->peer_buffers == nullptr || a->out == nullptr) {
    set_error("peer_buffers and out must not be NULL.");
    return FW_ERR_BAD_SHAPE;
  }
  if ((a->state_out == nullptr) != (a->state_lse == nullptr)) {
    set_error("state_out and state_lse must be passed together (or both NULL: merge only).");
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
  if (a->global_len != nullptr &&
      (a->local_len == nullptr || a->append_enable == nullptr || a->page_size <= 0 || a->advance < 0)) {
    set_error("global_len needs local_len, append_enable, a positive page_size and advance >= 0.");
    return FW_ERR_BAD_SHAPE;
  }
  MergeParams m{};
  for (int r = 0; r < a->world; ++r) {
    if (a->peer_buffers[r] == nullptr) {
      set_error("peer_buffers[%d] is NULL.", r);
      return FW_ERR_BAD_SHAPE;
    }
    m.slots.peers[r] = static_cast<uint8_t*>(a->peer_buffers[r]);
  }
  m.slots.world = a->world;
  m.slots.rank = a->rank;
  m.slots.slot_pairs = slot_pairs_of(a->rows, a->head_dim);
  m.sinks = a->sinks;
  m.out = static_cast<__nv_bfloat16*>(a->out);
  m.lse = a->lse;
  m.status = a->status;
  m.rows = a->rows;
  m.nheads = a->nheads;
  m.head_dim = a->head_dim;
  m.lse_head_stride = a->lse_head_stride;
  m.lse_token_stride = a->lse_token_stride;
  m.global_len = a->global_len;
  m.local_len = a->local_len;
  m.append_enable = a->append_enable;
  m.page_size = a->page_size;
  m.advance = a->advance;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_ptr);
  if (a->state_out != nullptr) {
    // A programmatic dependent of the kernel before it in the stream: its launch
    // latency hides under that kernel, and it starts with griddepcontrol.wait.
    ScatterParams s{};
    s.slots = m.slots;
    s.state_out = a->state_out;
    s.state_lse = a->state_lse;
    s.rows = a->rows;
    s.head_dim = a->head_dim;
    cudaLaunchAttribute pdl{};
    pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl.val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg{};
    cfg.stream = stream;
    cfg.attrs = &pdl;
    cfg.numAttrs = 1;
    cfg.gridDim = dim3(a->world, kScatterBlocks);
    cfg.blockDim = dim3(128);
    cudaError_t err = cudaLaunchKernelEx(&cfg, scatter_state_kernel, s);
    if (err == cudaSuccess) err = cudaGetLastError();
    if (err != cudaSuccess) {
      set_error("scatter kernel launch: %s", cudaGetErrorString(err));
      return FW_ERR_LAUNCH;
    }
  }
  return launch_gather_merge(m, stream);
}

// ---------------------------------------------------------------- round-robin page ownership
namespace fw {

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
