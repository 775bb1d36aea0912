// Host-side plumbing of the C ABI: thread-local error text, device queries,
// tensor-map encoding through the driver entry point (no link-time dependency
// on libcuda), status read-back.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace fw {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int sm_count() {
  // Read once per device; the table is write-once data, so concurrent callers
  // at worst repeat the query.
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  });
  return fn;
}

int encode_tensor_map_u8_4d(CUtensorMap* map, const void* base, const uint64_t dims[4],
                            const uint64_t strides[3], const uint32_t box[4]) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver.");
    return FW_ERR_LAUNCH;
  }
  cuuint64_t gdims[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstrides[3] = {strides[0], strides[1], strides[2]};
  cuuint32_t gbox[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t estrides[4] = {1, 1, 1, 1};
  CUresult res = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), gdims, gstrides, gbox,
                    estrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (dims %llu,%llu,%llu,%llu strides %llu,%llu,%llu "
              "box %u,%u,%u,%u)",
              static_cast<int>(res), (unsigned long long)dims[0], (unsigned long long)dims[1],
              (unsigned long long)dims[2], (unsigned long long)dims[3], (unsigned long long)strides[0],
              (unsigned long long)strides[1], (unsigned long long)strides[2], box[0], box[1], box[2], box[3]);
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

int encode_tensor_map_bf16(CUtensorMap* map, int rank, const void* base, const uint64_t* dims,
                           const uint64_t* strides, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) {
    set_error("cuTensorMapEncodeTiled is not available from this driver.");
    return FW_ERR_LAUNCH;
  }
  cuuint64_t gdims[5], gstrides[4];
  cuuint32_t gbox[5], estrides[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estrides[i] = 1;
    if (i + 1 < rank) gstrides[i] = strides[i];
  }
  CUresult res = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdims, gstrides, gbox,
                    estrides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled (bf16, rank %d) failed with CUresult %d", rank, static_cast<int>(res));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

}  // namespace fw

extern "C" const char* fw_last_error(void) { return fw::g_error; }

extern "C" int fw_version(void) { return 8; }

namespace fw {
// A CTA that waits on a barrier nobody will ever arrive on: the wait must give
// up after `limit` polls, record FW_STATUS_WAIT_TIMEOUT and return, leaving the
// context usable.  This is the path every kernel's waits take when a producer
// or a peer never shows up.
__global__ void wait_timeout_probe_kernel(int* status, uint32_t limit) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !mbar_wait_bounded(&bar, 0, &abort_flag, limit)) {
    abort_flag = 1;
    report_status(status, FW_STATUS_WAIT_TIMEOUT);
  }
}
}  // namespace fw

extern "C" int fw_selftest_wait_timeout(void* workspace, uint32_t spin_limit, void* stream) {
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & 3)) {
    fw::set_error("workspace must be a 4-byte aligned device pointer.");
    return FW_ERR_WORKSPACE;
  }
  if (spin_limit > (1u << 20)) spin_limit = 1u << 20;  // a fraction of a second at most
  fw::wait_timeout_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<int*>(workspace), spin_limit);
  cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    fw::set_error("probe launch: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  return FW_OK;
}

extern "C" int fw_read_status(const void* workspace, void* stream, int32_t* status) {
  if (workspace == nullptr || status == nullptr) {
    fw::set_error("workspace and status must not be NULL.");
    return FW_ERR_WORKSPACE;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t err = cudaMemcpyAsync(status, workspace, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess) {
    fw::set_error("reading the status word: %s", cudaGetErrorString(err));
    return FW_ERR_LAUNCH;
  }
  if (*status != FW_STATUS_OK) {
    // The word is sticky on the device; clear it once it has been reported.
    cudaMemsetAsync(const_cast<void*>(workspace), 0, sizeof(int32_t), s);
    cudaStreamSynchronize(s);
  }
  return FW_OK;
}
