// Tensor-core self test: one 128-row GEMM through exactly the operand paths the attention kernels use
// (TMA boxes with the 128-byte swizzle -> shared-memory descriptors -> tcgen05.mma -> tensor memory ->
// tcgen05.ld). It exists so that a wrong descriptor shows up as a wrong number in a unit test and not as a
// wrong attention output. No counterpart in the reference (its WGMMA plumbing comes from CuTe).
#include "host_util.h"
#include "ptx.cuh"

namespace fda {
namespace {

struct SelfTestParams {
  CUtensorMap tm_a;
  CUtensorMap tm_b;
  const __nv_bfloat16* a;
  float* c;
  int n;
  int k;
  int mode;
};

constexpr int kPanelBytes = 128 * 128;  // [128 rows][64 bf16]

__global__ void __launch_bounds__(128, 1) selftest_umma_kernel(const __grid_constant__ SelfTestParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                    // up to 2 panels
  uint8_t* sB = smem + 2 * kPanelBytes;  // up to 4 panels (mode 1: [k rows][64 cols] x n/64; mode 0: [n rows][64] x k/64)
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(&bar_load, 1);
    ptx::mbar_init(&bar_mma, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_s, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const uint32_t tmem_c = tmem;        // accumulator: n columns (<= 256)
  const uint32_t tmem_a = tmem + 256;  // A operand for mode 1: k/2 columns

  const int kpanels = p.k / 64;
  const int npanels = p.n / 64;
  if (threadIdx.x == 0) {
    uint32_t bytes = 0;
    if (p.mode == 0) {
      bytes = kpanels * kPanelBytes + kpanels * (p.n * 128);
      ptx::mbar_expect_tx(&bar_load, bytes);
      for (int c = 0; c < kpanels; ++c) {
        ptx::tma_load_4d(sA + c * kPanelBytes, &p.tm_a, &bar_load, c * 64, 0, 0, 0);
        ptx::tma_load_4d(sB + c * (p.n * 128), &p.tm_b, &bar_load, c * 64, 0, 0, 0);
      }
    } else {
      // mode 2 also brings A in as [k rows][128 columns]: two 64-column panels of k rows
      bytes = npanels * (p.k * 128) + (p.mode == 2 ? 2 * (p.k * 128) : 0);
      ptx::mbar_expect_tx(&bar_load, bytes);
      for (int c = 0; c < npanels; ++c) {
        ptx::tma_load_4d(sB + c * (p.k * 128), &p.tm_b, &bar_load, c * 64, 0, 0, 0);
      }
      if (p.mode == 2) {
        for (int c = 0; c < 2; ++c) ptx::tma_load_4d(sA + c * (p.k * 128), &p.tm_a, &bar_load, c * 64, 0, 0, 0);
      }
    }
  }
  if (p.mode == 1) {
    // A (128 x k) row-major in global memory -> tensor memory, two bf16 per 32-bit column, row = lane.
    const int row = warp * 32 + lane;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(p.a + static_cast<size_t>(row) * p.k);
    for (int c0 = 0; c0 < p.k / 2; c0 += 16) {
      uint32_t r[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) r[i] = src[c0 + i];
      ptx::tmem_st16(tmem_a + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
    }
    ptx::tmem_wait_st();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();

  if (threadIdx.x == 0) {
    bool ok = ptx::mbar_wait(&bar_load, 0, &abort_flag, 101);
    if (ok) {
      ptx::tc_fence_after();
      if (p.mode == 0) {
        const uint32_t idesc = ptx::make_idesc(128, p.n, 1, false, false);
        for (int kk = 0; kk < p.k / 16; ++kk) {
          const uint32_t a_addr = ptx::smem_u32(sA) + (kk / 4) * kPanelBytes + (kk % 4) * 32;
          const uint32_t b_addr = ptx::smem_u32(sB) + (kk / 4) * (p.n * 128) + (kk % 4) * 32;
          ptx::umma_ss_f16(tmem_c, ptx::make_smem_desc(a_addr, 16, 1024), ptx::make_smem_desc(b_addr, 16, 1024),
                           idesc, kk > 0);
        }
      } else if (p.mode == 2) {
        // both operands MN-major: the reduction dimension walks down the 128-byte rows (16 rows per instruction)
        const uint32_t idesc = ptx::make_idesc(128, p.n, 1, true, true);
        for (int kk = 0; kk < p.k / 16; ++kk) {
          const uint32_t a_addr = ptx::smem_u32(sA) + kk * 2048;
          const uint32_t b_addr = ptx::smem_u32(sB) + kk * 2048;
          ptx::umma_ss_f16(tmem_c, ptx::make_smem_desc(a_addr, p.k * 128, 1024),
                           ptx::make_smem_desc(b_addr, p.k * 128, 1024), idesc, kk > 0);
        }
      } else {
        const uint32_t idesc = ptx::make_idesc(128, p.n, 1, false, true);
        for (int kk = 0; kk < p.k / 16; ++kk) {
          const uint32_t b_addr = ptx::smem_u32(sB) + kk * 2048;
          ptx::umma_ts_f16(tmem_c, tmem_a + kk * 8, ptx::make_smem_desc(b_addr, p.k * 128, 1024), idesc, kk > 0);
        }
      }
    }
    ptx::umma_commit(&bar_mma);
  }
  ptx::mbar_wait(&bar_mma, 0, &abort_flag, 102);
  ptx::tc_fence_after();
  {
    const int row = warp * 32 + lane;
    for (int c0 = 0; c0 < p.n; c0 += 32) {
      uint32_t r[32];
      ptx::tmem_ld32(tmem_c + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
      ptx::tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) p.c[static_cast<size_t>(row) * p.n + c0 + i] = __uint_as_float(r[i]);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem, 512);
}


// A wait that nobody ends: one block allocates tensor memory the way the attention kernels do, one thread waits on a
// barrier no one arrives at with a SHORT limit, the others see the abort flag in their own wait, and everybody takes
// the kernels' exit path (drain, free the tensor memory, return). Exercises ptx::mbar_wait's give-up branch, which
// in the attention kernels is two seconds away.
__global__ void __launch_bounds__(128, 1) selftest_wait_kernel(long long limit_cycles) {
  __shared__ uint64_t never;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(&never, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_base_s, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  // thread 0 gives up after limit_cycles and raises the flag; the others wait with the production limit and leave
  // as soon as they see the flag
  const bool ok = ptx::mbar_wait(&never, 0, &abort_flag, 110, threadIdx.x == 0 ? limit_cycles : ptx::kWaitLimitCycles);
  (void)ok;
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem, 512);
}

}  // namespace

int launch_selftest_wait(long long limit_cycles, cudaStream_t stream) {
  if (limit_cycles < 1000 || limit_cycles > 100000000LL) return FDA_ERR_SHAPE;   // at most ~50 ms
  DeviceInfo info;
  int rc = current_device_info(&info);
  if (rc) return rc;
  if (info.cc_major != 10) return FDA_ERR_ARCH;
  selftest_wait_kernel<<<1, 128, 0, stream>>>(limit_cycles);
  FDA_CUDA_TRY(cudaGetLastError());
  return FDA_OK;
}

int launch_selftest_umma(int mode, const void* a, const void* b, float* c, int n, int k, cudaStream_t stream) {
  if (!a || !b || !c) return FDA_ERR_NULL;
  if (mode < 0 || mode > 2 || n % 64 || k % 64 || n < 64 || n > 256 || k < 64 || k > 128) return FDA_ERR_SHAPE;
  DeviceInfo info;
  int rc = current_device_info(&info);
  if (rc) return rc;
  if (info.cc_major != 10) return FDA_ERR_ARCH;
  SelfTestParams p;
  memset(&p, 0, sizeof(p));
  p.a = static_cast<const __nv_bfloat16*>(a);
  p.c = c;
  p.n = n;
  p.k = k;
  p.mode = mode;
  if (mode == 2) {
    // A: (k, 128) row-major (the transpose of the left operand), boxes [k][64]
    rc = encode_tile_map(&p.tm_a, a, 2, false, false, 128, k, 1, 1, 128, 128, 128 * (int64_t)k, 64, k);
  } else {
    // A: (128, k) row-major, boxes [128][64]
    rc = encode_tile_map(&p.tm_a, a, 2, false, false, k, 128, 1, 1, k, k, 128 * (int64_t)k, 64, 128);
  }
  if (rc) return rc;
  if (mode == 0) {
    rc = encode_tile_map(&p.tm_b, b, 2, false, false, k, n, 1, 1, k, k, n * (int64_t)k, 64, n);
  } else {
    rc = encode_tile_map(&p.tm_b, b, 2, false, false, n, k, 1, 1, n, n, n * (int64_t)k, 64, k);
  }
  if (rc) return rc;
  const int smem = 6 * kPanelBytes + 1024;
  static PerDeviceFlags smem_set;
  rc = set_dynamic_smem(selftest_umma_kernel, smem, smem_set);
  if (rc) return rc;
  selftest_umma_kernel<<<1, 128, smem, stream>>>(p);
  FDA_CUDA_TRY(cudaGetLastError());
  return FDA_OK;
}


int read_status_selftest(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}

}  // namespace fda
