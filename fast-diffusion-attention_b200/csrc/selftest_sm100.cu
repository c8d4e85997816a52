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
#ifdef FDA_UMMA_TIMING
__device__ long long g_umma_timing[8];
#endif

__global__ void __launch_bounds__(128, 1) selftest_umma_kernel(const __grid_constant__ SelfTestParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                    // up to 2 panels
  uint8_t* sB = smem + 2 * kPanelBytes;  // up to 4 panels (mode 1: [k rows][64 cols] x n/64; mode 0: [n rows][64] x k/64)
  __shared__ uint64_t bar_load, bar_mma;
#ifdef FDA_UMMA_TIMING
  __shared__ uint64_t bar_time, bar_mma2, bar_w1;
  __shared__ int go_flag;
#endif
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(&bar_load, 1);
    ptx::mbar_init(&bar_mma, 1);
#ifdef FDA_UMMA_TIMING
    ptx::mbar_init(&bar_time, 1);
    ptx::mbar_init(&bar_w1, 1);
    go_flag = 0;
    ptx::mbar_init(&bar_mma2, 1);
#endif
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
      bytes = npanels * (p.k * 128);
      ptx::mbar_expect_tx(&bar_load, bytes);
      for (int c = 0; c < npanels; ++c) {
        ptx::tma_load_4d(sB + c * (p.k * 128), &p.tm_b, &bar_load, c * 64, 0, 0, 0);
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
      } else {
        const uint32_t idesc = ptx::make_idesc(128, p.n, 1, false, true);
        for (int kk = 0; kk < p.k / 16; ++kk) {
          const uint32_t b_addr = ptx::smem_u32(sB) + kk * 2048;
          ptx::umma_ts_f16(tmem_c, tmem_a + kk * 8, ptx::make_smem_desc(b_addr, p.k * 128, 1024), idesc, kk > 0);
        }
      }
    }
    ptx::umma_commit(&bar_mma);
#ifdef FDA_UMMA_TIMING
    // Debug build only: issue cost and execution time of a burst of identical MMAs (the accumulator is junk after).
    ptx::mbar_wait(&bar_mma, 0, &abort_flag, 103);
    {
      constexpr int kBurst = 256;
      const uint32_t a_lo = ptx::smem_desc_lo(ptx::smem_u32(sA), 16);
      const uint32_t b_lo = ptx::smem_desc_lo(ptx::smem_u32(sB), p.mode == 0 ? 16 : p.k * 128);
      const uint32_t idesc = ptx::make_idesc(128, p.n, 1, false, p.mode != 0);
      const uint32_t idesc_ss128 = ptx::make_idesc(128, 128, 1, false, false);
      const long long t0 = clock64();
      for (int i = 0; i < kBurst; ++i) {
        if (p.mode == 0) ptx::umma_ss_f16_lh(tmem_c, a_lo + (i & 3) * 2, b_lo + (i & 3) * 2, ptx::smem_desc_hi(1024), idesc, 1);
        else ptx::umma_ts_f16_lh(tmem_c, tmem_a + (i & 3) * 8, b_lo + (i & 3) * 128, ptx::smem_desc_hi(1024), idesc, 1);
      }
      const long long t1 = clock64();
      ptx::umma_commit(&bar_time);
      ptx::mbar_wait(&bar_time, 0, &abort_flag, 104);
      const long long t2 = clock64();
      g_umma_timing[0] = kBurst;
      g_umma_timing[1] = t1 - t0;
      g_umma_timing[2] = t2 - t0;
      // unrolled burst without per-iteration branches
      const uint32_t hi = ptx::smem_desc_hi(1024);
      const long long u0 = clock64();
      if (p.mode == 0) {
#pragma unroll 1
        for (int i = 0; i < kBurst; i += 8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) ptx::umma_ss_f16_lh(tmem_c, a_lo + (j & 3) * 2, b_lo + (j & 3) * 2, hi, idesc, 1);
        }
      } else {
#pragma unroll 1
        for (int i = 0; i < kBurst; i += 8) {
#pragma unroll
          for (int j = 0; j < 8; ++j) ptx::umma_ts_f16_lh(tmem_c, tmem_a + (j & 3) * 8, b_lo + (j & 3) * 128, hi, idesc, 1);
        }
      }
      const long long u1 = clock64();
      ptx::umma_commit(&bar_time);
      ptx::mbar_wait(&bar_time, 1, &abort_flag, 107);
      g_umma_timing[4] = u1 - u0;
      g_umma_timing[5] = clock64() - u0;
      // two issuing threads: signal warp 1 to issue the same burst into other columns at the same time
      *reinterpret_cast<volatile int*>(&go_flag) = 1;
      const long long w0 = clock64();
#pragma unroll 1
      for (int i = 0; i < kBurst; i += 8) {
#pragma unroll
        for (int j = 0; j < 8; ++j) ptx::umma_ss_f16_lh(tmem_c, a_lo + (j & 3) * 2, b_lo + (j & 3) * 2, hi, idesc_ss128, 1);
      }
      ptx::umma_commit(&bar_time);
      ptx::mbar_wait(&bar_time, 0, &abort_flag, 108);
      ptx::mbar_wait(&bar_w1, 0, &abort_flag, 109);
      g_umma_timing[6] = clock64() - w0;
      // latency of one MMA + commit + wait round trip
      const long long t3 = clock64();
      if (p.mode == 0) ptx::umma_ss_f16_lh(tmem_c, a_lo, b_lo, ptx::smem_desc_hi(1024), idesc, 1);
      else ptx::umma_ts_f16_lh(tmem_c, tmem_a, b_lo, ptx::smem_desc_hi(1024), idesc, 1);
      ptx::umma_commit(&bar_time);
      ptx::mbar_wait(&bar_time, 1, &abort_flag, 105);
      g_umma_timing[3] = clock64() - t3;
      ptx::umma_commit(&bar_mma2);
    }
#endif
  }
#ifdef FDA_UMMA_TIMING
  if (threadIdx.x == 32) {
    long long spin0 = clock64();
    while (*reinterpret_cast<volatile int*>(&go_flag) == 0 && clock64() - spin0 < 2000000000LL) {}
    const uint32_t a_lo = ptx::smem_desc_lo(ptx::smem_u32(sA), 16);
    const uint32_t b_lo = ptx::smem_desc_lo(ptx::smem_u32(sB), 16);
    const uint32_t idesc_ss128 = ptx::make_idesc(128, 128, 1, false, false);
    const uint32_t hi = ptx::smem_desc_hi(1024);
#pragma unroll 1
    for (int i = 0; i < 256; i += 8) {
#pragma unroll
      for (int j = 0; j < 8; ++j) ptx::umma_ss_f16_lh(tmem + 384, a_lo + (j & 3) * 2, b_lo + (j & 3) * 2, hi, idesc_ss128, 1);
    }
    ptx::umma_commit(&bar_w1);
  }
#endif
  ptx::mbar_wait(&bar_mma, 0, &abort_flag, 102);
#ifdef FDA_UMMA_TIMING
  ptx::mbar_wait(&bar_mma2, 0, &abort_flag, 106);
#endif
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

#ifdef FDA_UMMA_TIMING
// Debug build only: cost of a burst of MMAs issued by one thread of warp 16 while warps 0-15 make "noise" of one
// kind: 0 idle (parked on a barrier), 1 polling an mbarrier that never completes, 2 FMA + ex2 arithmetic,
// 3 shared-memory loads. out[noise] = cycles per MMA for SS N=128, out[4 + noise] for SS N=64, out[8 + noise] TS.
__device__ long long g_contention[192];
__device__ __align__(128) uint8_t g_copy_src[32768];
__global__ void __launch_bounds__(544, 1) umma_contention_kernel(int noise, int random_fill, int out_base) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar_never, bar_done, bar_copy, bar_x, bar_y;
  __shared__ uint32_t tmem_base_s;
  long long copies = 0;
  __shared__ int stop_flag, abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    stop_flag = 0; abort_flag = 0;
    ptx::mbar_init(&bar_never, 1);
    ptx::mbar_init(&bar_done, 1);
    ptx::mbar_init(&bar_copy, 1);
    ptx::mbar_init(&bar_x, 1);
    ptx::mbar_init(&bar_y, 1);
    ptx::fence_mbar_init();
  }
  if (warp == 16) { ptx::tmem_alloc(&tmem_base_s, 512); ptx::tmem_relinquish(); }
  if (random_fill) {
    // bf16 values in (-1, 1) with busy mantissas, so that the tensor pipe toggles as it does on real data
    uint32_t x = 0x9E3779B9u * (threadIdx.x + 1) + blockIdx.x;
    for (int i = threadIdx.x; i < 196608 / 4; i += blockDim.x) {
      x = x * 1664525u + 1013904223u;
      const uint32_t lo16 = 0x3C00u + ((x >> 8) & 0x03FFu) + ((x >> 3) & 0x8000u);
      const uint32_t hi16 = 0x3C00u + ((x >> 18) & 0x03FFu) + ((x >> 1) & 0x8000u);
      reinterpret_cast<uint32_t*>(smem)[i] = lo16 | (hi16 << 16);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  volatile int* stop = &stop_flag;
  if (warp < 16) {
    float acc = static_cast<float>(threadIdx.x);
    if (noise == 1) {
      while (!*stop) { if (ptx::mbar_try_wait(&bar_never, 0)) break; }
    } else if (noise == 2) {
      while (!*stop) {
#pragma unroll
        for (int i = 0; i < 16; ++i) acc = ptx::ex2(fmaf(acc, 0.5f, -1.f)) + acc * 0.25f;
      }
    } else if (noise == 3) {
      const float4* src = reinterpret_cast<const float4*>(smem) + (threadIdx.x & 255);
      while (!*stop) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { const float4 v = src[i * 512]; acc += v.x + v.w; }
      }
    }
    else if (noise == 4 || noise == 5) {
      const uint32_t taddr = tmem + 384 + (static_cast<uint32_t>((warp & 3) * 32) << 16);
      uint32_t r[32];
      while (!*stop) {
        ptx::tmem_ld32(taddr, r);
        ptx::tmem_wait_ld();
        if (noise == 5) { ptx::tmem_st32(taddr + 32, r); ptx::tmem_wait_st(); }
        acc += __uint_as_float(r[lane]);
      }
    }
    else if (noise == 6 && threadIdx.x == 0) {
      // bulk copies from global memory into a shared region the MMAs do not read, 32 KB per round
      uint32_t par = 0;
      long long t_start = clock64();
      while (!*stop && clock64() - t_start < 400000000LL) {
        ptx::mbar_expect_tx(&bar_copy, 32768);
        ptx::bulk_load_1d(smem + 131072, g_copy_src, 16384, &bar_copy);
        ptx::bulk_load_1d(smem + 131072 + 16384, g_copy_src + 16384, 16384, &bar_copy);
        if (!ptx::mbar_wait(&bar_copy, par, &abort_flag, 111)) break;
        par ^= 1;
        ++copies;
      }
      if (blockIdx.x == 0) g_contention[out_base + 62] = copies;
      if (blockIdx.x == 0) g_contention[out_base + 63] = clock64() - t_start;
    }
    if (acc == 123.456f) g_contention[191] = 1;
  } else if (lane == 0) {
    constexpr int kBurst = 256;
    const uint32_t hi = ptx::smem_desc_hi(1024);
    const uint32_t a_lo = ptx::smem_desc_lo(ptx::smem_u32(smem), 16);
    const uint32_t b_lo = ptx::smem_desc_lo(ptx::smem_u32(smem + 32768), 16);
    const uint32_t b_mn = ptx::smem_desc_lo(ptx::smem_u32(smem + 32768), 16384);
    for (int variant = 0; variant < 3; ++variant) {
      const uint32_t idesc = variant == 0 ? ptx::make_idesc(128, 128, 1, false, false)
                                          : (variant == 1 ? ptx::make_idesc(128, 64, 1, false, false)
                                                          : ptx::make_idesc(128, 128, 1, false, true));
      const long long t0 = clock64();
#pragma unroll 1
      for (int i = 0; i < kBurst; i += 8) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (variant < 2) ptx::umma_ss_f16_lh(tmem, a_lo + (j & 3) * 2, b_lo + (j & 3) * 2, hi, idesc, 1);
          else ptx::umma_ts_f16_lh(tmem, tmem + 256 + (j & 3) * 8, b_mn + (j & 3) * 128, hi, idesc, 1);
        }
      }
      ptx::umma_commit(&bar_done);
      ptx::mbar_wait(&bar_done, variant & 1, &abort_flag, 110);
      if (blockIdx.x == 0) g_contention[out_base + variant * 8 + noise] = (clock64() - t0) / kBurst;
    }
    // Sequences of the backward kernels, operands stepping through the tiles as there. Variant 3: 16 SS N=64 (two
    // chains over 8 k-steps) then 8 TS N=128 with an MN-major B; variant 4: 16 SS N=128 then 8 TS N=128.
    for (int sync_pattern = 0; sync_pattern < 2; ++sync_pattern)
    for (int variant = 3; variant < 5; ++variant) {
      const uint32_t idesc_s = ptx::make_idesc(128, variant == 3 ? 64 : 128, 1, false, false);
      const uint32_t idesc_g = ptx::make_idesc(128, 128, 1, false, true);
      const uint32_t a2_lo = ptx::smem_desc_lo(ptx::smem_u32(smem + 65536), 16);
      const uint32_t bpanel = variant == 3 ? 8192 : 16384;
      const uint32_t b2_lo = ptx::smem_desc_lo(ptx::smem_u32(smem + 32768), 16);
      const uint32_t b2_mn = ptx::smem_desc_lo(ptx::smem_u32(smem + 32768), bpanel);
      constexpr int kRounds = 32;
      const long long t0 = clock64();
#pragma unroll 1
      for (int i = 0; i < kRounds; ++i) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a_off = ((kk / 4) * 16384 + (kk % 4) * 32) >> 4;
          const uint32_t b_off = ((kk / 4) * bpanel + (kk % 4) * 32) >> 4;
          ptx::umma_ss_f16_lh(tmem, a_lo + a_off, b2_lo + b_off, hi, idesc_s, kk > 0);
          ptx::umma_ss_f16_lh(tmem + 128, a2_lo + a_off, b2_lo + b_off + ((variant == 3 ? 16384 : 32768) >> 4), hi, idesc_s, kk > 0);
        }
        const int nk = variant == 3 ? 4 : 8;
        if (sync_pattern) {
          ptx::umma_commit(&bar_x);
          (void)ptx::mbar_try_wait(&bar_never, 0);
          ptx::tc_fence_after();
        }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (kk < nk) {
            ptx::umma_ts_f16_lh(tmem + 256, tmem + kk * 8, b2_mn + kk * (2048 >> 4), hi, idesc_g, 1);
            if (variant == 3) ptx::umma_ts_f16_lh(tmem + 384, tmem + 128 + kk * 8, b2_mn + (16384 >> 4) + kk * (2048 >> 4), hi, idesc_g, 1);
          }
        }
        if (sync_pattern) {
          ptx::umma_commit(&bar_y);
          (void)ptx::mbar_try_wait(&bar_never, 0);
          ptx::tc_fence_after();
        }
      }
      ptx::umma_commit(&bar_done);
      ptx::mbar_wait(&bar_done, variant & 1, &abort_flag, 110);
      if (blockIdx.x == 0) g_contention[out_base + (sync_pattern ? 48 : 24) + (variant - 3) * 8 + noise] = (clock64() - t0) / kRounds;
    }
    *stop = 1;
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 16) ptx::tmem_dealloc(tmem, 512);
}
#endif

}  // namespace

#ifdef FDA_UMMA_TIMING
extern "C" int fda_debug_umma_contention(long long* out192) {
  cudaFuncSetAttribute(umma_contention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  // one CTA on stale shared memory; one CTA on random data; one CTA per SM on random data
  const int grids[3] = {1, 1, 148}, fills[3] = {0, 1, 1};
  for (int cfg = 0; cfg < 3; ++cfg) {
    for (int noise = 0; noise < 7; ++noise) {
      if (cfg > 0 && noise != 0 && noise != 5) continue;
      umma_contention_kernel<<<grids[cfg], 544, 200 * 1024>>>(noise, fills[cfg], cfg * 64);
      if (cudaDeviceSynchronize() != cudaSuccess) return 1;
    }
  }
  return cudaMemcpyFromSymbol(out192, g_contention, sizeof(long long) * 192) == cudaSuccess ? 0 : 1;
}
#endif

int launch_selftest_umma(int mode, const void* a, const void* b, float* c, int n, int k, cudaStream_t stream) {
  if (!a || !b || !c) return FDA_ERR_NULL;
  if (mode < 0 || mode > 1 || n % 64 || k % 64 || n < 64 || n > 256 || k < 64 || k > 128) return FDA_ERR_SHAPE;
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
  // A: (128, k) row-major, boxes [128][64]
  rc = encode_tile_map(&p.tm_a, a, 2, false, false, k, 128, 1, 1, k, k, 128 * (int64_t)k, 64, 128);
  if (rc) return rc;
  if (mode == 0) {
    rc = encode_tile_map(&p.tm_b, b, 2, false, false, k, n, 1, 1, k, k, n * (int64_t)k, 64, n);
  } else {
    rc = encode_tile_map(&p.tm_b, b, 2, false, false, n, k, 1, 1, n, n, n * (int64_t)k, 64, k);
  }
  if (rc) return rc;
  const int smem = 6 * kPanelBytes + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    FDA_CUDA_TRY(cudaFuncSetAttribute(selftest_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr_set = true;
  }
  selftest_umma_kernel<<<1, 128, smem, stream>>>(p);
  FDA_CUDA_TRY(cudaGetLastError());
  return FDA_OK;
}

#ifdef FDA_UMMA_TIMING
extern "C" int fda_debug_umma_timing(long long* out8) {
  return cudaMemcpyFromSymbol(out8, g_umma_timing, sizeof(long long) * 8) == cudaSuccess ? 0 : 1;
}
#endif

int read_status_selftest(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}

}  // namespace fda
