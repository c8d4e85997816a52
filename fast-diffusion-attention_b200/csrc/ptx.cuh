// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA tile loads, tcgen05 (tensor memory allocation,
// MMA issue, commit, tensor-memory loads/stores) and the descriptors they take. These replace the sm90
// mechanics of the reference (WGMMA wrappers, named barriers, TMA pipeline: csrc/fda/utils.h:123-192,
// csrc/fda/named_barrier.hpp, csrc/fda/sm90_pipeline_no_cluster.hpp there); nothing is ported from them.
#pragma once

#include <cstdint>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace fda {

// ---------------------------------------------------------------------------------------------------------
// Device status word. A wait that gives up records (code, block, detail) here instead of trapping; the
// kernel then drains and returns so the context stays usable. Host side: fda_device_status().
// ---------------------------------------------------------------------------------------------------------
static __device__ int g_fda_status[4];

namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier -------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Make generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma operands).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for the whole warp, made by lane 0 after every lane has reached this point (each lane has done its
// own tcgen05 wait + fence before calling). 128 separate arrivals on one barrier serialise; 4 do not.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort_flag` lives in shared memory; once any thread of the CTA gives up, every later wait
// returns at once so the CTA can drain, free its tensor memory and exit. Returns false when aborted.
constexpr long long kWaitLimitCycles = 4000000000LL;  // about two seconds at the boost clock

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int code,
                                          long long limit_cycles = kWaitLimitCycles) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 127u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit_cycles) {
        *abort_flag = code;
        if (atomicCAS(&g_fda_status[0], 0, code) == 0) {
          g_fda_status[1] = static_cast<int>(blockIdx.x);
          g_fda_status[2] = static_cast<int>(threadIdx.x);
          g_fda_status[3] = static_cast<int>(parity);
        }
        return false;
      }
    }
  }
  return true;
}


// ---- TMA tile loads (no cluster fan-out: every CTA fetches its own tiles) ----------------------------------
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "r"(c2), "r"(c3)
      : "memory");
}

// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---- tile stores through shared memory ----------------------------------------------------------------------
// The tile lies in shared memory in the layout of the map (128-byte swizzle for the maps of this library); the
// copy clips at the tensor's bounds. Generic-proxy writes to the tile need fence_proxy_async_smem() and a barrier
// before the store is issued; the issuing thread commits a group and waits for it before the tile is reused.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2,
                                             int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all committed groups of this thread have finished READING shared memory (the tile may be overwritten)
__device__ __forceinline__ void bulk_wait_group_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
// at most kPending of this thread's committed groups may still be reading shared memory
template <int kPending>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
// Untiled bulk reduction shared -> global: adds `bytes` (a multiple of 16) of fp32 values to global memory; both
// addresses 16-byte aligned. Part of the issuing thread's current bulk group.
__device__ __forceinline__ void bulk_reduce_add_f32(float* gmem_dst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(gmem_dst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
// all committed groups of this thread are complete
__device__ __forceinline__ void bulk_wait_group0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void st_shared_v4(void* smem_dst, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(smem_u32(smem_dst)), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
// Row `row` of a [rows][128 bytes] tile in the 128-byte swizzle: 16-byte chunk c of the row sits at chunk
// c ^ (row & 7). `w` holds the row's 32 words (64 16-bit values).
__device__ __forceinline__ void st_shared_row128_sw(uint8_t* tile, int row, const uint32_t* w) {
  uint8_t* base = tile + row * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    st_shared_v4(base + ((c ^ (row & 7)) << 4), w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
  }
}

// ---- register reallocation between warpgroups -------------------------------------------------------------
// Every warp of a warpgroup (four consecutive warps, the first a multiple of four) must execute the call; kRegs
// is a multiple of 8 in [24, 256]. A kernel that uses these is launched with whole warpgroups only, and the
// per-warpgroup counts it sets must add up to at most the 64K registers of the SM.
template <uint32_t kRegs>
__device__ __forceinline__ void reg_release_to() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegs));
}
template <uint32_t kRegs>
__device__ __forceinline__ void reg_acquire_to() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegs));
}

// ---- tensor memory ----------------------------------------------------------------------------------------
// Whole-warp calls. `ncols` is a power of two >= 32; the address of the allocation is written to *smem_dst.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---- MMA issue (one thread) -------------------------------------------------------------------------------
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void umma_ss_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc]
__device__ __forceinline__ void umma_ts_f16(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ss_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_f8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ---- descriptors ------------------------------------------------------------------------------------------
// Instruction descriptor of tcgen05.mma kind::f16 / kind::f8f6f4 with fp32 accumulation.
//   bits 4-5 accumulator format (1 = f32), 7-9 A format, 10-12 B format (f16 kind: 0 = f16, 1 = bf16;
//   f8f6f4 kind: 0 = e4m3), 15 A major (0 = K-major, 1 = MN-major), 16 B major, 17-22 N/8, 24-28 M/16.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, int ab_format, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | (static_cast<uint32_t>(ab_format) << 7) | (static_cast<uint32_t>(ab_format) << 10) |
         (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor for tiles stored as [rows][128 bytes] with the 128-byte swizzle (what a TMA
// box of 128 bytes x rows with CU_TENSOR_MAP_SWIZZLE_128B writes); the tile base is 1024-byte aligned.
//   bits 0-13 address/16, 16-29 leading byte offset/16, 32-45 stride byte offset/16, 46-47 version (1),
//   61-63 layout (2 = 128-byte swizzle).
// K-major operand (the 128-byte rows run along the reduction dimension): stride offset = 1024 (eight rows),
// leading offset unused. MN-major operand (rows run along M/N, the reduction dimension walks down the rows):
// stride offset = 1024 (eight reduction rows), leading offset = distance between 64-element column panels.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t leading_bytes,
                                                   uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// The same descriptor split in two 32-bit words so that the MMA-issuing thread does one integer add per MMA:
// the high word (stride offset, version, swizzle mode) is a compile-time constant, the low word is
// (address / 16) | (leading offset / 16) << 16 and advances by (byte offset / 16).
__host__ __device__ constexpr uint32_t smem_desc_hi(uint32_t stride_bytes) {
  return ((stride_bytes >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr, uint32_t leading_bytes) {
  return ((smem_addr & 0x3FFFFu) >> 4) | (((leading_bytes >> 4) & 0x3FFFu) << 16);
}
__device__ __forceinline__ void umma_ss_f16_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_f16_lh(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_ss_f8_lh(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_ts_f8_lh(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t hi, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %4, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- tensor-memory loads / stores: 32 lanes x 32-bit, N consecutive columns per thread -------------------------
// Warp w of a warpgroup may only touch lanes 32*(w%4) .. +31; lane field = bits 31-16 of the address.
#define FDA_R4(a, i) "=r"(a[i]), "=r"(a[i + 1]), "=r"(a[i + 2]), "=r"(a[i + 3])
#define FDA_W4(a, i) "r"(a[i]), "r"(a[i + 1]), "r"(a[i + 2]), "r"(a[i + 3])

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : FDA_R4(r, 0), FDA_R4(r, 4), FDA_R4(r, 8), FDA_R4(r, 12), FDA_R4(r, 16), FDA_R4(r, 20), FDA_R4(r, 24),
        FDA_R4(r, 28)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : FDA_R4(r, 0), FDA_R4(r, 4), FDA_R4(r, 8), FDA_R4(r, 12)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      ::FDA_W4(r, 0), FDA_W4(r, 4), FDA_W4(r, 8), FDA_W4(r, 12), FDA_W4(r, 16), FDA_W4(r, 20), FDA_W4(r, 24),
      FDA_W4(r, 28), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      ::FDA_W4(r, 0), FDA_W4(r, 4), FDA_W4(r, 8), FDA_W4(r, 12), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%8], {%0, %1, %2, %3, %4, %5, %6, %7};" ::FDA_W4(r, 0),
               FDA_W4(r, 4), "r"(taddr)
               : "memory");
}
#undef FDA_R4
#undef FDA_W4

// 256-bit global store (one full 32-byte sector per thread); the address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t* r) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// ---- small math helpers --------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two fp32 operations per instruction (sm_100 has packed fp32 FMA / ADD / MUL on register pairs) and the
// three-input maximum: the softmax loops are bound by instruction latency with two or four warps per scheduler, so
// fewer instructions per element is what makes them faster.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1, float c0, float c1) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1), "f"(c0), "f"(c1));
}
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "add.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void mul2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
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
// four floats -> four e4m3 bytes, a in the lowest byte (round to nearest, saturating)
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}
template <bool kBf16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  return kBf16 ? pack_bf16(lo, hi) : pack_f16(lo, hi);
}

// Store 32 fp32 accumulator values of one row as 16-bit after scaling: columns [col0, col0 + 32) of a row of
// `head_dim` (a multiple of 8) elements. `wide` = the row pointer and head_dim allow 32-byte stores.
template <bool kBf16>
__device__ __forceinline__ void store_row32(uint16_t* row_ptr, int col0, const uint32_t* acc, float scale,
                                            int head_dim, bool wide) {
  uint32_t w[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    w[i] = pack2<kBf16>(__uint_as_float(acc[2 * i]) * scale, __uint_as_float(acc[2 * i + 1]) * scale);
  }
  if (wide) {
#pragma unroll
    for (int i = 0; i < 32; i += 16) {
      if (col0 + i < head_dim) st_global_v8(row_ptr + col0 + i, w + i / 2);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      if (col0 + i < head_dim) {
        *reinterpret_cast<uint4*>(row_ptr + col0 + i) = make_uint4(w[i / 2], w[i / 2 + 1], w[i / 2 + 2], w[i / 2 + 3]);
      }
    }
  }
}

// The same 32 columns, but stored so that four neighbouring lanes write 64 contiguous bytes of ONE row: the four
// lanes of a group first swap their 16-byte pieces (a 4 x 4 transpose by two exchanges of shuffles), then lane j
// stores piece j of each of the group's four rows. A warp instruction then touches 8 rows instead of 32, which is
// what the load/store unit's cost goes by. Every lane of the warp must call this (shuffles); lane l holds row l
// of the warp's 32 rows, of which the first `rows_valid` are written. `row_ptr` is the lane's own row, rows are
// `row_stride` elements apart, and everything is 16-byte aligned.
// `w` holds the row's 32 columns already scaled and packed to 16 bits (16 words); it is overwritten.
__device__ __forceinline__ void store_rows32_grouped_packed(uint16_t* row_ptr, int64_t row_stride, int rows_valid,
                                                            int col0, uint32_t* w, int head_dim) {
  const int lane = threadIdx.x & 31;
  const int j = lane & 3;
  // first exchange, partner lane ^ 1: even lanes give pieces 1 and 3, odd lanes pieces 0 and 2
#pragma unroll
  for (int k = 0; k < 4; k += 2) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t send = (j & 1) ? w[4 * k + q] : w[4 * (k + 1) + q];
      const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
      if (j & 1) w[4 * k + q] = recv; else w[4 * (k + 1) + q] = recv;
    }
  }
  // second exchange, partner lane ^ 2: lanes 0, 1 give pieces 2 and 3, lanes 2, 3 pieces 0 and 1
#pragma unroll
  for (int k = 0; k < 2; ++k) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t send = (j & 2) ? w[4 * k + q] : w[4 * (k + 2) + q];
      const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 2);
      if (j & 2) w[4 * k + q] = recv; else w[4 * (k + 2) + q] = recv;
    }
  }
  // now w[4 * i ..] is piece j (columns col0 + 8 j .. + 8) of row (lane & ~3) + i
  const int col = col0 + 8 * j;
  if (col < head_dim) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = (lane & ~3) + i;
      if (r < rows_valid) {
        uint16_t* dst = row_ptr + static_cast<int64_t>(i - j) * row_stride + col;
        *reinterpret_cast<uint4*>(dst) = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
      }
    }
  }
}

template <bool kBf16>
__device__ __forceinline__ void pack_row32(const uint32_t* acc, float scale, uint32_t* w) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    w[i] = pack2<kBf16>(__uint_as_float(acc[2 * i]) * scale, __uint_as_float(acc[2 * i + 1]) * scale);
  }
}

template <bool kBf16>
__device__ __forceinline__ void store_rows32_grouped(uint16_t* row_ptr, int64_t row_stride, int rows_valid, int col0,
                                                     const uint32_t* acc, float scale, int head_dim) {
  uint32_t w[16];
  pack_row32<kBf16>(acc, scale, w);
  store_rows32_grouped_packed(row_ptr, row_stride, rows_valid, col0, w, head_dim);
}

}  // namespace ptx
}  // namespace fda
