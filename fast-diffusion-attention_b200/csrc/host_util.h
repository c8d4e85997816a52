// Host-side helpers shared by the launchers: CUDA error capture, TMA tensor-map encoding through the driver
// entry point (so the library links only the CUDA runtime and still loads on a machine without a driver),
// and cached device properties. The reference does the equivalent work inside CuTe's make_tma_copy
// (csrc/fda/flash_fwd_launch_template.h:63-92 there).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../include/fda.h"

namespace fda {

inline char* cuda_error_buf() {
  static thread_local char buf[256] = {0};
  return buf;
}

inline int note_cuda_error(cudaError_t e, const char* what) {
  snprintf(cuda_error_buf(), 256, "%s: %s", what, cudaGetErrorString(e));
  return FDA_ERR_CUDA;
}

#define FDA_CUDA_TRY(expr)                                         \
  do {                                                             \
    cudaError_t _e = (expr);                                       \
    if (_e != cudaSuccess) return ::fda::note_cuda_error(_e, #expr); \
  } while (0)

inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      p = nullptr;
    }
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

// Tensor map over a (batch, rows, heads, dim) view with element strides; boxes are [box_rows][box_cols]
// elements of one (head, batch), written to shared memory as rows of box_cols elements with the 128-byte
// swizzle (box_cols * elem_bytes must be 128). Out-of-range elements read as zero.
inline int encode_tile_map(CUtensorMap* map, const void* ptr, int elem_bytes, bool is_fp8, bool is_fp16,
                           int64_t dim, int64_t rows, int64_t heads, int64_t batch, int64_t row_stride,
                           int64_t head_stride, int64_t batch_stride, int box_cols, int box_rows) {
  auto enc = tensor_map_encoder();
  if (!enc) {
    snprintf(cuda_error_buf(), 256, "cuTensorMapEncodeTiled entry point not available");
    return FDA_ERR_CUDA;
  }
  if (batch <= 1) batch_stride = rows * row_stride;  // unused dimension, any valid stride
  if (heads <= 1 && head_stride == 0) head_stride = dim;
  cuuint64_t gdim[4] = {(cuuint64_t)dim, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)(batch < 1 ? 1 : batch)};
  cuuint64_t gstride[3] = {(cuuint64_t)(row_stride * elem_bytes), (cuuint64_t)(head_stride * elem_bytes),
                           (cuuint64_t)(batch_stride * elem_bytes)};
  for (int i = 0; i < 3; ++i) {
    if (gstride[i] % 16 != 0 || gstride[i] == 0) return FDA_ERR_STRIDE;
  }
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return FDA_ERR_STRIDE;
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estride[4] = {1, 1, 1, 1};
  CUtensorMapDataType dt = is_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                  : (is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
  CUresult r = enc(map, dt, 4, const_cast<void*>(ptr), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(cuda_error_buf(), 256, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FDA_ERR_CUDA;
  }
  return FDA_OK;
}

// Per-device caches are indexed by the CUDA device ordinal up to this limit; beyond it nothing is cached (every call
// does the full work), so no ordinal is ever refused or silently skipped. A cudaDeviceReset() clears the function
// attributes the flags stand for: a process that resets a device must not call the library on it afterwards.
constexpr int kMaxCachedDevices = 64;

struct PerDeviceFlags {
  std::atomic<bool> done[kMaxCachedDevices];
};

// Raise a kernel's dynamic shared-memory limit once per device (the attribute is per device and per function).
template <typename Kernel>
int set_dynamic_smem(Kernel kernel, int bytes, PerDeviceFlags& flags) {
  int dev = 0;
  FDA_CUDA_TRY(cudaGetDevice(&dev));
  const bool cached = dev >= 0 && dev < kMaxCachedDevices;
  if (cached && flags.done[dev].load(std::memory_order_acquire)) return FDA_OK;
  FDA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (cached) flags.done[dev].store(true, std::memory_order_release);
  return FDA_OK;
}

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0;
};

inline int current_device_info(DeviceInfo* out) {
  static thread_local DeviceInfo cache[kMaxCachedDevices];
  int dev = 0;
  FDA_CUDA_TRY(cudaGetDevice(&dev));
  const bool cached = dev >= 0 && dev < kMaxCachedDevices;
  if (cached && cache[dev].device == dev) {
    *out = cache[dev];
    return FDA_OK;
  }
  DeviceInfo d;
  d.device = dev;
  FDA_CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
  FDA_CUDA_TRY(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
  if (cached) cache[dev] = d;
  *out = d;
  return FDA_OK;
}

// Launchers implemented next to their kernels.
int launch_fwd(const FdaFwdArgs& a, cudaStream_t stream);
int launch_bwd(const FdaBwdArgs& a, cudaStream_t stream, unsigned stage_mask);
int launch_bwd_noalloc(const FdaBwdArgs& a, cudaStream_t stream);
int launch_selftest_umma(int mode, const void* a, const void* b, float* c, int n, int k, cudaStream_t stream);
int launch_selftest_wait(long long limit_cycles, cudaStream_t stream);
int read_status_fwd(int32_t* out4);
int read_status_bwd(int32_t* out4);
int read_status_bwd_fused(int32_t* out4);
int read_status_selftest(int32_t* out4);

}  // namespace fda
