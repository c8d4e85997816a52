// Backward pass of block-diffusion attention for sm_100a.
//
// The reference runs up to six launches (csrc/fda/flash_bwd_launch_template.h:26-284 there): a preprocess
// (flash_bwd_preprocess_kernel.h:106-208), an optional noisy-diagonal kernel, the dK/dV-stationary main kernel
// with an fp32 dQ accumulator reduced through global memory (mainloop_bwd_sm90_tma_gmma_ws.hpp:413-1014,
// epilogue_bwd.hpp:25-441), and convert passes (flash_bwd_postprocess_kernel.h:160-264). On B200 the tensor
// memory budget (512 columns) and the cost of a global fp32 reduction lead to a different split:
//
//   1. bwd_preprocess : delta = rowsum(dO * O) and LSE * log2(e), written to a padded per-(sample, head, half)
//                       layout whose padding rows carry LSE2 = +inf (so padded query rows get P = 0).
//   2. bwd_dkdv       : one CTA per (128-key tile, KV head, sample, half); K, V stay in shared memory, the
//                       visible query tiles of every query head of the group stream through. S^T = K Q^T and
//                       dP^T = V dO^T land in tensor memory (keys on lanes); P^T and dS^T go back to tensor
//                       memory as 16-bit A operands of dV += P^T dO and dK += dS^T Q. GQA sums over the group
//                       inside the CTA: no fp32 dK/dV accumulators in global memory.
//   3. bwd_dq         : forward-shaped, one CTA per 128-row query tile: S = Q K^T, dP = dO V^T, dS to tensor
//                       memory, dQ += dS K. No cross-CTA reduction at all, so dQ needs no atomics, no fp32
//                       accumulator, no zero-fill and no convert pass.
//
// Seven GEMMs per tile pair instead of five, in exchange for zero global reductions; every gradient has a
// fixed accumulation order, so the result is bitwise reproducible whether or not `deterministic` is set.
// Numerics kept from the reference: P = exp2(S*c - LSE2) from the saved LSE, dS = P * (dP - delta)
// [* (1 - tanh^2) with softcap, before masking], P and dS rounded to the input dtype before the second GEMMs,
// dK and dQ scaled by softmax_scale once at the end (mainloop_bwd...hpp:836-893, :1009).
#include "geometry.h"
#include "host_util.h"
#include "ptx.cuh"
#include "sched.cuh"

#ifndef FDA_ABL
#define FDA_ABL 0   // debug builds only: 1 skips the softmax-backward arithmetic, 2 also the tensor-memory traffic
#endif

#ifdef FDA_TRACE
__device__ long long g_fda_trace[8 * 256];
extern "C" int fda_debug_trace(long long* out) {
  return cudaMemcpyFromSymbol(out, g_fda_trace, sizeof(long long) * 8 * 256) == cudaSuccess ? 0 : 1;
}
#define FDA_TRACE_PUT(row, idx) do { if (blockIdx.x == 0 && (idx) < 256u) g_fda_trace[(row) * 256 + (idx)] = clock64(); } while (0)
#else
#define FDA_TRACE_PUT(row, idx) do { } while (0)
#endif
// FDA_TRACE=1 traces the dK/dV kernel, FDA_TRACE=2 the dQ kernel
#if defined(FDA_TRACE) && FDA_TRACE == 1
#define FDA_TRACE_AT(row, idx) FDA_TRACE_PUT(row, idx)
#else
#define FDA_TRACE_AT(row, idx) do { } while (0)
#endif
#if defined(FDA_TRACE) && FDA_TRACE == 2
#define FDA_TRACE_Q(row, idx) FDA_TRACE_PUT(row, idx)
#else
#define FDA_TRACE_Q(row, idx) do { } while (0)
#endif
#if defined(FDA_TRACE) && FDA_TRACE == 5   // phases of a compute warp in the dK/dV kernel
#define FDA_TRACE_KC(row, idx) FDA_TRACE_PUT(row, idx)
#else
#define FDA_TRACE_KC(row, idx) do { } while (0)
#endif
#if defined(FDA_TRACE) && FDA_TRACE == 4   // item boundaries of the dK/dV kernel
#define FDA_TRACE_KI(row, idx) FDA_TRACE_PUT(row, idx)
#else
#define FDA_TRACE_KI(row, idx) do { } while (0)
#endif
#if defined(FDA_TRACE) && FDA_TRACE == 3   // item boundaries of the dQ kernel
#define FDA_TRACE_QI(row, idx) FDA_TRACE_PUT(row, idx)
#else
#define FDA_TRACE_QI(row, idx) do { } while (0)
#endif
#ifdef FDA_CTA_TIMES
__device__ unsigned long long g_fda_cta_times_b[2 * 2 * 160];   // [kernel][start / end][CTA]
extern "C" int fda_debug_cta_times_bwd(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_fda_cta_times_b, sizeof(unsigned long long) * 640) == cudaSuccess ? 0 : 1;
}
#define FDA_CTA_STAMP(kernel, which) do { if (threadIdx.x == 0 && blockIdx.x < 160) { unsigned long long t_; \
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_fda_cta_times_b[(kernel) * 320 + (which) * 160 + blockIdx.x] = t_; } } while (0)
#else
#define FDA_CTA_STAMP(kernel, which) do { } while (0)
#endif
#ifdef FDA_CLOCKRATE
__device__ unsigned long long g_fda_clockrate[2];
extern "C" int fda_debug_clockrate(unsigned long long* out2) {
  return cudaMemcpyFromSymbol(out2, g_fda_clockrate, 16) == cudaSuccess ? 0 : 1;
}
#endif

#ifndef FDA_SHORT8_KV
#define FDA_SHORT8_KV 4   // eighths of a (sample, head)'s items that count as short: dK/dV kernel
#endif
#ifndef FDA_SHORT8_Q
#define FDA_SHORT8_Q 1    // the same for the dQ kernel
#endif

namespace fda {
namespace {

constexpr int kTile = 128;  // rows of every query / key tile
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  CUtensorMap tm_q, tm_k, tm_v, tm_do;
  CUtensorMap tm_q64, tm_do64;  // same tensors, 64-row boxes (dK/dV kernel)
  CUtensorMap tm_k64, tm_v64;   // 64-row boxes of K / V (dQ kernel for head dimensions above 128)
  const void* out;
  const void* dout;
  void* dq;
  void* dk;
  void* dv;
  int64_t o_bs, o_rs, o_hs;
  int64_t do_bs, do_rs, do_hs;
  int64_t dq_bs, dq_rs, dq_hs;
  int64_t dk_bs, dk_rs, dk_hs;
  int64_t dv_bs, dv_rs, dv_hs;
  const float* lse;
  float* delta_pad;  // (batch, heads, 2, n_pad)
  float* lse2_pad;   // (batch, heads, 2, n_pad)
  const int32_t* cu_seqlens;
  int batch, seqlen, total, heads, heads_k, head_dim, block_size;
  int n_pad;           // round_up(max n, 128)
  int tiles_per_half;  // n_pad / 128
  int n_long_kv, n_long_q;  // of the 2 * tiles_per_half items of a (sample, head): how many count as long
  int* ticket_kv;      // work counters of the two persistent kernels, zeroed before each launch
  int* ticket_q;
  int wide_store;      // dq/dk/dv rows allow 32-byte stores
  float scale_log2, softcap_pre, softmax_scale;
};

struct Sample {
  int n, row0, bcoord;
};

__device__ __forceinline__ Sample sample_of(const BwdParams& p, int b) {
  Sample s;
  if (p.cu_seqlens != nullptr) {
    const int lo = p.cu_seqlens[b];
    s.n = (p.cu_seqlens[b + 1] - lo) / 2;
    s.row0 = lo;
    s.bcoord = 0;
  } else {
    s.n = p.seqlen / 2;
    s.row0 = 0;
    s.bcoord = b;
  }
  return s;
}

__device__ __forceinline__ int64_t stat_segment(const BwdParams& p, int b, int h, int half) {
  return ((static_cast<int64_t>(b) * p.heads + h) * 2 + half) * p.n_pad;
}

// ------------------------------------------------------------------------------------------------------------
// 1. preprocess
// ------------------------------------------------------------------------------------------------------------
constexpr int kPreUnroll = 4;   // rows per thread group: more loads in flight, fewer and longer blocks

template <bool kBf16, int kLanes>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const __grid_constant__ BwdParams p) {
  constexpr int kRowsPerWarp = 32 / kLanes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / kLanes, l = lane % kLanes;
  const int hh = blockIdx.y;
  const int h = hh >> 1, half = hh & 1;
  const int b = blockIdx.z;
  const Sample sm = sample_of(p, b);
  const int64_t seg = stat_segment(p, b, h, half);
  // row u of this thread group: position in the half (rows >= n, up to n_pad, only get their padding values)
  const int r0 = ((blockIdx.x * 8 + warp) * kPreUnroll) * kRowsPerWarp + sub;
  float acc[kPreUnroll];
  // head dimensions up to 8 * kLanes take one 16-byte piece of O and of dO per lane: all loads of the kPreUnroll rows
  // are issued before the first use
  uint4 ov[kPreUnroll], gv[kPreUnroll];
#pragma unroll
  for (int u = 0; u < kPreUnroll; ++u) {
    const int r = r0 + u * kRowsPerWarp;
    acc[u] = 0.f;
    ov[u] = make_uint4(0, 0, 0, 0);
    gv[u] = make_uint4(0, 0, 0, 0);
    if (r < sm.n && l * 8 < p.head_dim) {
      const int64_t srow = static_cast<int64_t>(sm.row0) + half * sm.n + r;
      const uint16_t* o = static_cast<const uint16_t*>(p.out) + sm.bcoord * p.o_bs + srow * p.o_rs + h * p.o_hs;
      const uint16_t* g = static_cast<const uint16_t*>(p.dout) + sm.bcoord * p.do_bs + srow * p.do_rs + h * p.do_hs;
      ov[u] = *reinterpret_cast<const uint4*>(o + l * 8);
      gv[u] = *reinterpret_cast<const uint4*>(g + l * 8);
    }
  }
#pragma unroll
  for (int u = 0; u < kPreUnroll; ++u) {
    const uint32_t aw[4] = {ov[u].x, ov[u].y, ov[u].z, ov[u].w};
    const uint32_t dw[4] = {gv[u].x, gv[u].y, gv[u].z, gv[u].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 fa, fd;
      if (kBf16) {
        fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&aw[i]));
        fd = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dw[i]));
      } else {
        fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
        fd = __half22float2(*reinterpret_cast<const __half2*>(&dw[i]));
      }
      acc[u] = fmaf(fa.x, fd.x, acc[u]);
      acc[u] = fmaf(fa.y, fd.y, acc[u]);
    }
#pragma unroll
    for (int off = kLanes / 2; off > 0; off >>= 1) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], off);
  }
  if (l == 0) {
#pragma unroll
    for (int u = 0; u < kPreUnroll; ++u) {
      const int r = r0 + u * kRowsPerWarp;
      if (r >= p.n_pad) continue;
      const bool valid = r < sm.n;
      float lse2 = INFINITY;
      if (valid) {
        const int64_t srow = static_cast<int64_t>(sm.row0) + half * sm.n + r;
        const int64_t li = (p.cu_seqlens != nullptr)
                               ? static_cast<int64_t>(h) * p.total + srow
                               : (static_cast<int64_t>(b) * p.heads + h) * p.seqlen + (half * sm.n + r);
        const float lse = p.lse[li];
        lse2 = (lse == -INFINITY) ? 0.f : lse * kLog2e;
      }
      p.delta_pad[seg + r] = valid ? acc[u] : 0.f;
      p.lse2_pad[seg + r] = lse2;
    }
  }
}

// Shared-memory layout helpers ------------------------------------------------------------------------------------
template <int kHeadDim>
struct TileCfg {
  static constexpr int kTileBytes = kTile * kHeadDim * 2;
  static constexpr int kPanels = kHeadDim / 64;
  static constexpr int kPanelBytes = 128 * 128;
};

template <int kHeadDim>
__device__ __forceinline__ void load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar, int row, int head,
                                          int bcoord) {
#pragma unroll
  for (int c = 0; c < TileCfg<kHeadDim>::kPanels; ++c) {
    ptx::tma_load_4d(dst + c * TileCfg<kHeadDim>::kPanelBytes, tm, bar, c * 64, row, head, bcoord);
  }
}

// Compute warpgroups of the two backward kernels: each owns kCols of the 128 columns of S / dP (all 128 lanes).
constexpr int kCmpWG = 4;
constexpr int kCols = kTile / kCmpWG;             // 32 columns per warpgroup
constexpr int kCmpThreads = 128 * kCmpWG;         // 512
constexpr int kBwdThreads = kCmpThreads + 128;    // + a warpgroup of TMA warp, two MMA warps and an idle warp
// 640 threads start with 96 registers each; that pool is all the block ever has (asking for more would block a
// warpgroup for ever): 4 * 128 * 104 + 128 * 64 = 640 * 96.
constexpr uint32_t kComputeRegs = 104, kProducerRegs = 64;
static_assert(kCmpThreads * kComputeRegs + 128 * kProducerRegs <= kBwdThreads * 96, "register pool");
// The dK/dV kernel has a sixth warpgroup that only writes the finished accumulators out, so that the compute
// warps go straight on to the next item: 768 threads start with 80 registers each.
constexpr int kDkdvThreads = kBwdThreads + 128;
constexpr int kEpiWarp0 = 4 * kCmpWG + 4;
constexpr uint32_t kDkdvComputeRegs = 88, kDkdvProducerRegs = 64, kDkdvEpilogueRegs = 64;
static_assert(kCmpThreads * kDkdvComputeRegs + 128 * kDkdvProducerRegs + 128 * kDkdvEpilogueRegs <= kDkdvThreads * 80,
              "register pool");
constexpr int kLoadWarpB = 4 * kCmpWG;
constexpr int kMmaWarpB = 4 * kCmpWG + 1;
static_assert(kCols == 32, "one 32-column tensor-memory load per operand and warp");

// P and dS of kN columns for one thread. `s`/`dp` hold the raw accumulators; the results are packed 16-bit.
// lse2 / delta are per column (kPerColumn, read from shared memory) or per thread. kMasked is a template
// parameter so that the common fully-visible tile carries no per-element compare/select at all.
template <int kN, bool kBf16, bool kSoftcap, bool kPerColumn, bool kMasked, bool kNeedP>
__device__ __forceinline__ void softmax_backward_cols(const uint32_t* s, const uint32_t* dp, const float* lse2_col,
                                                      const float* delta_col, float lse2_row, float delta_row,
                                                      float scale_log2, float softcap_pre, int lo, int hi,
                                                      uint32_t* pk_p, uint32_t* pk_ds) {
#pragma unroll
  for (int c = 0; c < kN; c += 2) {
    float pv[2], dsv[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int col = c + e;
      float x = __uint_as_float(s[col]);
      float dt = 1.f;
      if (kSoftcap) {
        x = ptx::tanh_fast(x * softcap_pre);
        dt = 1.f - x * x;
      }
      const float l2 = kPerColumn ? lse2_col[col] : lse2_row;
      const float dl = kPerColumn ? delta_col[col] : delta_row;
      float pr = ptx::ex2(fmaf(x, scale_log2, -l2));
      float d = pr * (__uint_as_float(dp[col]) - dl);
      if (kSoftcap) d *= dt;
      if (kMasked && (col < lo || col >= hi)) {
        pr = 0.f;
        d = 0.f;
      }
      pv[e] = pr;
      dsv[e] = d;
    }
    if (kNeedP) pk_p[c / 2] = ptx::pack2<kBf16>(pv[0], pv[1]);
    pk_ds[c / 2] = ptx::pack2<kBf16>(dsv[0], dsv[1]);
  }
}

// ------------------------------------------------------------------------------------------------------------
// 2. dK / dV
// ------------------------------------------------------------------------------------------------------------
struct KvItem {
  int b, hk, kh, k0, k1, n, row0, bcoord;
  bool valid;
};

__device__ __forceinline__ KvItem decode_kv_item(const BwdParams& p, int idx) {
  // (sample, KV head)-major: the CTAs running at the same time stream the Q / dO tiles of a few heads, which then
  // stay in L2. Inside a head: clean key tiles first, early ones first (they are seen by the most queries), then
  // the noisy key tiles (one block of queries each) as filler.
  KvItem it;
  const int per_bh = 2 * p.tiles_per_half;
  int bh, rem;
  two_phase_order(idx, per_bh, p.n_long_kv, p.batch * p.heads_k, bh, rem);
  it.kh = rem < p.tiles_per_half ? 1 : 0;
  const int kt = rem < p.tiles_per_half ? rem : rem - p.tiles_per_half;
  it.b = bh / p.heads_k;
  it.hk = bh - it.b * p.heads_k;
  const Sample sm = sample_of(p, it.b);
  it.n = sm.n;
  it.row0 = sm.row0;
  it.bcoord = sm.bcoord;
  it.k0 = kt * kTile;
  it.valid = it.k0 < it.n;
  it.k1 = imin(it.k0 + kTile, it.n);
  return it;
}

// Query spans of the item's key tile: [0] for query tiles of the same half, [1] for noisy query tiles seeing
// clean keys. Built once per item; classifying a query tile is then compares only.
struct KvSpans {
  Span same, cross;
  bool partial_keys;
  __device__ __forceinline__ int classify(int qh, int kh, int qa, int qb) const {
    int c = (qh == kh ? same : cross).classify(qa, qb - qa);
    if (c == kTileFull && partial_keys) c = kTileMasked;
    return c;
  }
};

__device__ __forceinline__ KvSpans make_kv_spans(const KvItem& it, int bs) {
  KvSpans sp;
  sp.same = query_span(it.kh, it.kh, it.k0, it.k1, it.n, bs);
  sp.cross = it.kh == 1 ? query_span(0, 1, it.k0, it.k1, it.n, bs) : Span{0, 0, 0, 0};
  sp.partial_keys = (it.k1 - it.k0) < kTile;
  return sp;
}

// The query side streams in sub-tiles of kSub = 64 rows so that S^T / dP^T (64 columns each) can be double
// buffered in tensor memory next to the dK / dV accumulators: while the compute warps turn buffer u into
// P^T / dS^T, the tensor pipe runs dV / dK of the previous sub-tile and S^T / dP^T of the next one.
constexpr int kSub = 64;
constexpr int kSubCols = kSub / kCmpWG;  // 16 query columns per compute warpgroup

template <int kHeadDim, int kStages>
struct DkdvCfg {
  using T = TileCfg<kHeadDim>;
  static constexpr int kSubTileBytes = kSub * kHeadDim * 2;     // Q or dO sub-tile
  static constexpr int kSubPanelBytes = kSub * 128;             // one 64-column panel of a sub-tile
  static constexpr int kStageBytes = 2 * kSubTileBytes + 1024;  // Q sub-tile, dO sub-tile, lse2[64], delta[64], header
  static constexpr int kHeaderOffset = 2 * kSubTileBytes + 512;
  static constexpr int kSmemBytes = 2 * T::kTileBytes + kStages * kStageBytes + 1024 + 512;
  static constexpr int kThreads = kDkdvThreads;
  // buffer u: S^T at u*128, dP^T at u*128 + 64; accumulators behind
  // head dimensions above 128 do not leave room for both accumulators next to the S^T / dP^T buffers: the key
  // tile is then processed in kPasses passes, each producing kAccDim columns of dK and dV
  static constexpr int kAccDim = kHeadDim > 128 ? 128 : kHeadDim;
  static constexpr int kPasses = kHeadDim / kAccDim;
  static constexpr int kLookahead = kStages >= 2 ? 2 : 1;  // S^T / dP^T sub-steps issued ahead of dV / dK
  static constexpr int kTmemDK = 256, kTmemDV = 256 + kAccDim;
  static_assert(256 + 2 * kAccDim <= 512, "tensor memory budget");
  static_assert(kStageBytes % 1024 == 0, "sub-tiles must stay 1024-byte aligned for the 128-byte swizzle");
};

// Sub-steps of one item: query heads of the group x visible 128-row query tiles x two 64-row halves; a half
// with no visible row is skipped. All roles walk this sequence identically.
struct SubStep {
  int h, qh, sa, sb, cls;
};

template <int kHeadDim, int kStages, bool kBf16, bool kSoftcap>
__global__ void __launch_bounds__(kDkdvThreads, 1) bwd_dkdv_kernel(const __grid_constant__ BwdParams p) {
  using Cfg = DkdvCfg<kHeadDim, kStages>;
  using T = TileCfg<kHeadDim>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + T::kTileBytes;
  uint8_t* sStage = smem + 2 * T::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStage + kStages * Cfg::kStageBytes);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + 1;
  uint64_t* st_full = bars + 2;
  uint64_t* st_empty = st_full + kStages;
  uint64_t* sdp_full = st_empty + kStages;   // [2]
  uint64_t* pds_full = sdp_full + 2;         // [2]
  uint64_t* acc_full = pds_full + 2;
  uint64_t* buf_free = acc_full + 1;         // [2]
  uint64_t* acc_free = buf_free + 2;         // the epilogue warps have the accumulators in registers
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  SchedMailbox* mbox = reinterpret_cast<SchedMailbox*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  FDA_CTA_STAMP(0, 0);
#ifdef FDA_CLOCKRATE
  long long cr_c0 = 0; unsigned long long cr_t0 = 0;
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    cr_c0 = clock64();
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(cr_t0));
  }
#endif
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    sched_init(mbox, 4 * kCmpWG + 2 + 4);   // compute warps, two MMA issuers, four epilogue warps
    ptx::mbar_init(kv_full, 1);
    ptx::mbar_init(kv_empty, 1);
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&st_full[i], 1);
      ptx::mbar_init(&st_empty[i], 1);
    }
    for (int u = 0; u < 2; ++u) {
      ptx::mbar_init(&sdp_full[u], 1);
      ptx::mbar_init(&pds_full[u], 4 * kCmpWG);
      ptx::mbar_init(&buf_free[u], 1);
    }
    ptx::mbar_init(acc_full, 1);
    ptx::mbar_init(acc_free, 4);
    ptx::fence_mbar_init();
  }
  if (warp == kLoadWarpB) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int bs = p.block_size;
  const int group = p.heads / p.heads_k;
  const int total_items = p.tiles_per_half * 2 * p.heads_k * p.batch * Cfg::kPasses;

  // Calls fn(SubStep) for every non-skipped sub-step of the item, in order; stops early when fn returns false.
  auto for_each_substep = [&](const KvItem& it, const QueryPlan& plan, const KvSpans& spans, auto&& fn) -> bool {
    for (int g = 0; g < group; ++g) {
      for (int s = 0; s < plan.steps(); ++s) {
        int qh, qt;
        plan.step(s, it.kh, qh, qt);
        const int qa = qt * kTile, qb = imin(qa + kTile, it.n);
        if (spans.classify(qh, it.kh, qa, qb) == kTileSkip) continue;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          SubStep st;
          st.sa = qa + half * kSub;
          if (st.sa >= qb) continue;
          st.sb = imin(st.sa + kSub, qb);
          st.cls = spans.classify(qh, it.kh, st.sa, st.sb);
          if (st.cls == kTileSkip) continue;
          st.h = it.hk * group + g;
          st.qh = qh;
          if (!fn(st)) return false;
        }
      }
    }
    return true;
  };

  // Whole warpgroups: four of compute warps, one of the TMA warp, the two MMA warps and an idle warp. The fifth
  // hands registers to the other four. The counts are set inside the role branches, so that the compiler never
  // has to assume the smaller one where the branches meet.
  if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------------------------------------ epilogue
    // Four warps, one per quarter of the tensor-memory lanes: dK and dV of a finished item go out to global memory
    // while the other roles are already at work on the next item.
    ptx::reg_release_to<kDkdvEpilogueRegs>();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t n_item = 0;
    for (uint32_t n_sched = 0;; ++n_sched) {
      const int idx = sched_consume<true>(mbox, n_sched, abort_flag);
      if (idx < 0 || idx >= total_items) break;
      const KvItem it = decode_kv_item(p, idx / Cfg::kPasses);
      if (!it.valid) continue;
      const int pass_col0 = (idx % Cfg::kPasses) * Cfg::kAccDim;
      const int kj = it.k0 + row;
      const int rows_valid = imax(0, imin(32, it.n - (it.k0 + quad * 32)));  // of this warp's 32 key rows
      const int64_t srow = static_cast<int64_t>(it.row0) + it.kh * it.n + kj;
      uint16_t* dk_row = static_cast<uint16_t*>(p.dk) + it.bcoord * p.dk_bs + srow * p.dk_rs + it.hk * p.dk_hs;
      uint16_t* dv_row = static_cast<uint16_t*>(p.dv) + it.bcoord * p.dv_bs + srow * p.dv_rs + it.hk * p.dv_hs;
      if (!ptx::mbar_wait(acc_full, n_item & 1, abort_flag, 62)) break;
      ++n_item;
      ptx::tc_fence_after();
      // dK and dV sit side by side in tensor memory: 2 * d / 32 chunks of 32 columns
      constexpr int kChunks = 2 * Cfg::kAccDim / 32;
#pragma unroll 1
      for (int gidx = 0; gidx < kChunks; ++gidx) {
        const bool is_dv = gidx * 32 >= Cfg::kAccDim;
        const int col0 = pass_col0 + gidx * 32 - (is_dv ? Cfg::kAccDim : 0);
        uint32_t accv[32];
        ptx::tmem_ld32(tmem + Cfg::kTmemDK + lane_addr + gidx * 32, accv);
        ptx::tmem_wait_ld();
        if (gidx == kChunks - 1) {
          // everything is in registers: the first dV / dK products of the next item may overwrite the accumulators
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(acc_free);
        }
        // Plain row stores: these four warps are in nobody's way, what counts is that the accumulators are free
        // again before the next item's first dV / dK product is due (a few thousand cycles).
        if (lane < rows_valid) {
          ptx::store_row32<kBf16>(is_dv ? dv_row : dk_row, col0, accv, is_dv ? 1.f : p.softmax_scale, p.head_dim,
                                  p.wide_store != 0);
        }
      }
    }
  } else if (warp >= 4 * kCmpWG) {
  ptx::reg_release_to<kDkdvProducerRegs>();
  if (warp == kLoadWarpB) {
    // ------------------------------------------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t n_item = 0, gc = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_produce(mbox, n_sched, p.ticket_kv, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const KvItem it = decode_kv_item(p, idx / Cfg::kPasses);
        if (!it.valid) continue;
        const QueryPlan plan = make_query_plan(it.kh, it.k0, it.k1, it.n, bs, kTile);
        const KvSpans spans = make_kv_spans(it, bs);
        if (!ptx::mbar_wait(kv_empty, (n_item & 1) ^ 1, abort_flag, 41)) break;
        ptx::mbar_expect_tx(kv_full, 2 * T::kTileBytes);
        const int k_row = it.row0 + it.kh * it.n + it.k0;
        load_tile<kHeadDim>(sK, &p.tm_k, kv_full, k_row, it.hk, it.bcoord);
        load_tile<kHeadDim>(sV, &p.tm_v, kv_full, k_row, it.hk, it.bcoord);
        // The loader alone walks the item's geometry. Each stage carries a two-word header for the other roles:
        // {bit 0 last sub-step of the item, bit 1 partially masked, bit 2 queries of the keys' own half; first row}.
        // A sub-step is sent when its successor is known, so that the last one can be marked.
        auto emit = [&](const SubStep& st, bool last) -> bool {
          const uint32_t stage = gc % kStages;
          if (!ptx::mbar_wait(&st_empty[stage], ((gc / kStages) & 1) ^ 1, abort_flag, 42)) return false;
          uint8_t* base = sStage + stage * Cfg::kStageBytes;
          volatile int* hdr = reinterpret_cast<volatile int*>(base + Cfg::kHeaderOffset);
          hdr[0] = (last ? 1 : 0) | (st.cls == kTileMasked ? 2 : 0) | (st.qh == it.kh ? 4 : 0);
          hdr[1] = st.sa;
#if FDA_ABL >= 3
          ptx::mbar_expect_tx(&st_full[stage], 512);
#else
          ptx::mbar_expect_tx(&st_full[stage], 2 * Cfg::kSubTileBytes + 512);
#endif
          const int q_row = it.row0 + st.qh * it.n + st.sa;
#if FDA_ABL < 3
#pragma unroll
          for (int c = 0; c < T::kPanels; ++c) {
            ptx::tma_load_4d(base + c * Cfg::kSubPanelBytes, &p.tm_q64, &st_full[stage], c * 64, q_row, st.h, it.bcoord);
            ptx::tma_load_4d(base + Cfg::kSubTileBytes + c * Cfg::kSubPanelBytes, &p.tm_do64, &st_full[stage], c * 64,
                             q_row, st.h, it.bcoord);
          }
#endif
          const int64_t seg = stat_segment(p, it.b, st.h, st.qh) + st.sa;
          ptx::bulk_load_1d(base + 2 * Cfg::kSubTileBytes, p.lse2_pad + seg, 256, &st_full[stage]);
          ptx::bulk_load_1d(base + 2 * Cfg::kSubTileBytes + 256, p.delta_pad + seg, 256, &st_full[stage]);
          ++gc;
          return true;
        };
        SubStep pend{};
        bool have = false;
        alive = for_each_substep(it, plan, spans, [&](const SubStep& st) -> bool {
          if (have && !emit(pend, false)) return false;
          pend = st;
          have = true;
          return true;
        });
        // every valid key tile is seen at least by the queries of its own rows, so there is a last sub-step
        if (alive && have) alive = emit(pend, true);
        ++n_item;
      }
      if (*abort_flag) __nanosleep(100000);
    }
  } else if (warp == kMmaWarpB) {
    // ------------------------------------------------------------------- MMA issuer 1: S^T = K Q^T, dP^T = V dO^T
    // Two threads issue the MMAs of this kernel. The tensor pipe's queue is short, so whatever else an issuing
    // thread does (barrier waits, commits) leaves the pipe idle; with two issuers one's bookkeeping overlaps the
    // other's MMAs. Their only mutual dependency is the S^T / dP^T buffer: sub-step g may overwrite buffer g & 1
    // once dV / dK of sub-step g - 2 have read it (buf_free).
    if (lane == 0) {
      constexpr int kFmt = kBf16 ? 1 : 0;
      const uint32_t idesc_s = ptx::make_idesc(kTile, kSub, kFmt, false, false);
      constexpr uint32_t kHi = ptx::smem_desc_hi(1024);
      const uint32_t k_lo = ptx::smem_desc_lo(ptx::smem_u32(sK), 16);
      const uint32_t v_lo = ptx::smem_desc_lo(ptx::smem_u32(sV), 16);
      const uint32_t st_lo_k = ptx::smem_desc_lo(ptx::smem_u32(sStage), 16);
      uint32_t n_item = 0, g = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_consume<false>(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const KvItem it = decode_kv_item(p, idx / Cfg::kPasses);
        if (!it.valid) continue;
        if (!ptx::mbar_wait(kv_full, n_item & 1, abort_flag, 51)) break;
        for (bool last = false; alive && !last; ++g) {
          const uint32_t u = g & 1u, stage = g % kStages;
          if (!ptx::mbar_wait(&st_full[stage], (g / kStages) & 1u, abort_flag, 52)) { alive = false; break; }
          last = (*reinterpret_cast<const volatile int*>(sStage + stage * Cfg::kStageBytes + Cfg::kHeaderOffset) & 1) != 0;
          if (!ptx::mbar_wait(&buf_free[u], ((g >> 1) & 1u) ^ 1u, abort_flag, 54)) { alive = false; break; }
          FDA_TRACE_AT(3, g);
          ptx::tc_fence_after();
          const uint32_t q_off = stage * (Cfg::kStageBytes >> 4);
          const uint32_t do_off = q_off + (Cfg::kSubTileBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk) {
            const uint32_t a_off = ((kk / 4) * T::kPanelBytes + (kk % 4) * 32) >> 4;
            const uint32_t b_off = ((kk / 4) * Cfg::kSubPanelBytes + (kk % 4) * 32) >> 4;
            ptx::umma_ss_f16_lh(tmem + u * 128, k_lo + a_off, st_lo_k + q_off + b_off, kHi, idesc_s, kk > 0);
            ptx::umma_ss_f16_lh(tmem + u * 128 + 64, v_lo + a_off, st_lo_k + do_off + b_off, kHi, idesc_s, kk > 0);
          }
          ptx::umma_commit(&sdp_full[u]);
          FDA_TRACE_AT(4, g);
        }
        // K and V are read by these products only: the next item's tiles may load while the last dV / dK products
        // and the epilogue of this item still run
        if (alive) ptx::umma_commit(kv_empty);
        ++n_item;
      }
    }
  } else if (warp == kMmaWarpB + 1) {
    // ------------------------------------------------------------------- MMA issuer 2: dV += P^T dO, dK += dS^T Q
    if (lane == 0) {
      constexpr int kFmt = kBf16 ? 1 : 0;
      const uint32_t idesc_g = ptx::make_idesc(kTile, Cfg::kAccDim, kFmt, false, true);
      constexpr uint32_t kHi = ptx::smem_desc_hi(1024);
      const uint32_t st_lo_mn = ptx::smem_desc_lo(ptx::smem_u32(sStage), Cfg::kSubPanelBytes);    // MN-major use
      uint32_t g = 0, n_item_b = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_consume<false>(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const KvItem it = decode_kv_item(p, idx / Cfg::kPasses);
        if (!it.valid) continue;
        // descriptor offset of the first 64-column panel of this pass in a sub-tile
        const uint32_t pass_panel_off = (idx % Cfg::kPasses) * (Cfg::kAccDim / 64) * (Cfg::kSubPanelBytes >> 4);
        bool acc = false;
        // the first products of an item overwrite the accumulators: the epilogue warps must have read the last item's
        if (!ptx::mbar_wait(acc_free, (n_item_b & 1u) ^ 1u, abort_flag, 57)) break;
        ++n_item_b;
        for (bool last = false; alive && !last; ++g) {
          const uint32_t u = g & 1u, stage = g % kStages;
          // the stage barrier orders the header and, through the other issuer's wait on it, nothing else here:
          // the tiles themselves are read by the MMAs, after P^T / dS^T (pds_full) which follow S^T / dP^T
          if (!ptx::mbar_wait(&st_full[stage], (g / kStages) & 1u, abort_flag, 55)) { alive = false; break; }
          last = (*reinterpret_cast<const volatile int*>(sStage + stage * Cfg::kStageBytes + Cfg::kHeaderOffset) & 1) != 0;
          FDA_TRACE_AT(0, g);
          if (!ptx::mbar_wait(&pds_full[u], (g >> 1) & 1u, abort_flag, 53)) { alive = false; break; }
          FDA_TRACE_AT(1, g);
          ptx::tc_fence_after();
          const uint32_t q_off = stage * (Cfg::kStageBytes >> 4);
          const uint32_t do_off = q_off + (Cfg::kSubTileBytes >> 4);
          const uint32_t st_t = tmem + u * 128, dpt_t = tmem + u * 128 + 64;
#pragma unroll
          for (int kk = 0; kk < kSub / 16; ++kk) {
            ptx::umma_ts_f16_lh(tmem + Cfg::kTmemDV, st_t + kk * kSubCols,
                                st_lo_mn + do_off + pass_panel_off + kk * (2048 >> 4), kHi, idesc_g,
                                (acc || kk > 0) ? 1u : 0u);
            ptx::umma_ts_f16_lh(tmem + Cfg::kTmemDK, dpt_t + kk * kSubCols,
                                st_lo_mn + q_off + pass_panel_off + kk * (2048 >> 4), kHi, idesc_g,
                                (acc || kk > 0) ? 1u : 0u);
          }
          acc = true;
          ptx::umma_commit(&buf_free[u]);
          ptx::umma_commit(&st_empty[stage]);
          FDA_TRACE_AT(2, g);
        }
        if (!alive) break;
        ptx::umma_commit(acc_full);
      }
    }
  }
  } else {
    ptx::reg_acquire_to<kDkdvComputeRegs>();
    // -------------------------------------------------------------------------------------- softmax backward
    const int wg = warp >> 2;                  // which kSubCols query columns of a sub-tile
    const int quad = warp & 3;
    const int row = quad * 32 + lane;          // key row inside the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t n_item = 0, gc = 0;
    bool alive = true;
    for (uint32_t n_sched = 0; alive; ++n_sched) {
      if (threadIdx.x == 0) FDA_TRACE_KI(2, n_item);
      const int idx = sched_consume<true>(mbox, n_sched, abort_flag);
      if (idx < 0 || idx >= total_items) break;
      if (threadIdx.x == 0) FDA_TRACE_KI(3, n_item);
      const KvItem it = decode_kv_item(p, idx / Cfg::kPasses);
      const int pass_col0 = (idx % Cfg::kPasses) * Cfg::kAccDim;
      if (!it.valid) continue;
      const int kj = it.k0 + row;
      // queries that see this thread's key: same-half tiles and (clean keys only) noisy tiles of later blocks
      int same_lo, same_hi, cross_lo, cross_hi;
      query_interval(it.kh, it.kh, kj, it.n, bs, same_lo, same_hi);
      query_interval(0, 1, kj, it.n, bs, cross_lo, cross_hi);
      if (threadIdx.x == 0) FDA_TRACE_KI(4, n_item);
      for (bool last = false; alive && !last;) {
        const uint32_t u = gc & 1u, stage = gc % kStages;
        const uint8_t* stage_base = sStage + stage * Cfg::kStageBytes;
        const float* stats = reinterpret_cast<const float*>(stage_base + 2 * Cfg::kSubTileBytes);
        // wait on the stage barrier ourselves: it orders the header and the bulk copies of lse2 / delta before our reads
        if (!ptx::mbar_wait(&st_full[stage], (gc / kStages) & 1u, abort_flag, 60)) { alive = false; break; }
        int2 hdr;
        hdr.x = reinterpret_cast<const volatile int*>(stage_base + Cfg::kHeaderOffset)[0];
        hdr.y = reinterpret_cast<const volatile int*>(stage_base + Cfg::kHeaderOffset)[1];
        last = (hdr.x & 1) != 0;
        // The per-column statistics of this warp's 16 query columns come into registers now, as four 16-byte loads
        // each, while the S^T / dP^T products are still running: scalar loads inside the arithmetic below queue
        // up behind the operand fetches of the MMAs, which keep the shared-memory pipe busy.
        float l2r[kSubCols], dlr[kSubCols];
        {
          const float4* l2v = reinterpret_cast<const float4*>(stats + wg * kSubCols);
          const float4* dlv = reinterpret_cast<const float4*>(stats + kSub + wg * kSubCols);
#pragma unroll
          for (int i = 0; i < kSubCols / 4; ++i) {
            const float4 a = l2v[i], b = dlv[i];
            l2r[4 * i] = a.x; l2r[4 * i + 1] = a.y; l2r[4 * i + 2] = a.z; l2r[4 * i + 3] = a.w;
            dlr[4 * i] = b.x; dlr[4 * i + 1] = b.y; dlr[4 * i + 2] = b.z; dlr[4 * i + 3] = b.w;
          }
        }
        if (threadIdx.x == 0) FDA_TRACE_AT(5, gc);
        if (!ptx::mbar_wait(&sdp_full[u], (gc >> 1) & 1u, abort_flag, 61)) { alive = false; break; }
        if (threadIdx.x == 0) FDA_TRACE_AT(6, gc);
        if (threadIdx.x == 0) FDA_TRACE_KC(0, gc);
        ++gc;
        ptx::tc_fence_after();
        const uint32_t st_t = tmem + u * 128 + lane_addr + wg * kSubCols;
        const uint32_t dpt_t = st_t + 64;
        uint32_t sv[kSubCols], dpv[kSubCols];
#if FDA_ABL < 2
        ptx::tmem_ld16(st_t, sv);
        ptx::tmem_ld16(dpt_t, dpv);
        ptx::tmem_wait_ld();
#else
        for (int i = 0; i < kSubCols; ++i) { sv[i] = i; dpv[i] = i; }
#endif
        if (threadIdx.x == 0) FDA_TRACE_KC(1, gc - 1);
        uint32_t pk_p[kSubCols / 2], pk_ds[kSubCols / 2];
        const float* l2 = l2r;
        const float* dl = dlr;
#if FDA_ABL >= 1
        for (int i = 0; i < kSubCols / 2; ++i) { pk_p[i] = sv[i]; pk_ds[i] = dpv[i]; }
        if (false) {
#else
        if (hdr.x & 2) {
#endif
          const int lo = ((hdr.x & 4) ? same_lo : cross_lo) - (hdr.y + wg * kSubCols);
          const int hi = ((hdr.x & 4) ? same_hi : cross_hi) - (hdr.y + wg * kSubCols);
          softmax_backward_cols<kSubCols, kBf16, kSoftcap, true, true, true>(sv, dpv, l2, dl, 0.f, 0.f, p.scale_log2,
                                                                              p.softcap_pre, lo, hi, pk_p, pk_ds);
        } else {
#if FDA_ABL < 1
          softmax_backward_cols<kSubCols, kBf16, kSoftcap, true, false, true>(sv, dpv, l2, dl, 0.f, 0.f, p.scale_log2,
                                                                               p.softcap_pre, 0, 0, pk_p, pk_ds);
#endif
        }
        // a warp overwrites only columns it has itself already loaded: its packed P^T / dS^T pieces go to the
        // start of its own kSubCols columns
        if (threadIdx.x == 0) FDA_TRACE_KC(2, gc - 1);
#if FDA_ABL < 2
        ptx::tmem_st8(st_t, pk_p);
        ptx::tmem_st8(dpt_t, pk_ds);
        ptx::tmem_wait_st();
#endif
        ptx::tc_fence_before();
        if (threadIdx.x == 0) FDA_TRACE_KC(3, gc - 1);
        ptx::mbar_arrive_warp(&pds_full[u]);
        if (threadIdx.x == 0) FDA_TRACE_KC(4, gc - 1);
        if (threadIdx.x == 0) FDA_TRACE_AT(7, gc - 1);
      }
      if (!alive) break;
      ++n_item;
      if (threadIdx.x == 0) FDA_TRACE_KI(5, n_item - 1);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
#ifdef FDA_CLOCKRATE
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    unsigned long long t1;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
    g_fda_clockrate[0] = clock64() - cr_c0;
    g_fda_clockrate[1] = t1 - cr_t0;
  }
#endif
  FDA_CTA_STAMP(0, 1);
  if (warp == kLoadWarpB) ptx::tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------------------
// 3. dQ
// ------------------------------------------------------------------------------------------------------------
struct QItem {
  int b, h, hk, qh, qa, qb, n, row0, bcoord;
  bool valid;
};

__device__ __forceinline__ QItem decode_q_item(const BwdParams& p, int idx) {
  // (sample, head)-major for L2 reuse of K / V; inside a head late query tiles first (they see the most keys).
  QItem it;
  const int per_bh = 2 * p.tiles_per_half;
  int bh, rem;
  two_phase_order(idx, per_bh, p.n_long_q, p.batch * p.heads, bh, rem);
  it.qh = rem & 1;
  const int t_rev = rem >> 1;
  it.b = bh / p.heads;
  it.h = bh - it.b * p.heads;
  it.hk = it.h / (p.heads / p.heads_k);
  const Sample sm = sample_of(p, it.b);
  it.n = sm.n;
  it.row0 = sm.row0;
  it.bcoord = sm.bcoord;
  it.qa = (p.tiles_per_half - 1 - t_rev) * kTile;
  it.valid = it.qa < it.n;
  it.qb = imin(it.qa + kTile, it.n);
  return it;
}

struct QSpans {
  Span half[2];  // key spans of the query tile per key half (0 noisy, 1 clean)
  // selects instead of half[kh]: a run-time index would put the spans in local memory
  __device__ __forceinline__ int classify(int kh, int k0, int keys) const {
    Span s;
    s.lo_first = kh ? half[1].lo_first : half[0].lo_first;
    s.hi_first = kh ? half[1].hi_first : half[0].hi_first;
    s.lo_last = kh ? half[1].lo_last : half[0].lo_last;
    s.hi_last = kh ? half[1].hi_last : half[0].hi_last;
    return s.classify(k0, keys);
  }
};

__device__ __forceinline__ QSpans make_q_spans(const QItem& it, int bs) {
  QSpans sp;
  sp.half[0] = key_span(it.qh, 0, it.qa, it.qb, it.n, bs);
  sp.half[1] = key_span(it.qh, 1, it.qa, it.qb, it.n, bs);
  return sp;
}

template <int kHeadDim, int kStages>
struct DqCfg {
  using T = TileCfg<kHeadDim>;
  // keys per step: 128, or 64 for head dimensions above 128 (Q and dO alone take 128 KB of shared memory there)
  static constexpr int kKeys = kHeadDim > 128 ? 64 : 128;
  static constexpr int kKeyCols = kKeys / kCmpWG;               // key columns per compute warpgroup
  static constexpr int kKvTileBytes = kKeys * kHeadDim * 2;
  static constexpr int kKvPanelBytes = kKeys * 128;
  static constexpr int kSmemBytes = 2 * T::kTileBytes + kStages * kKvTileBytes + 1024 + 512;
  static constexpr int kKSlots = (kStages + 1) / 2;  // K ring; the rest is the V ring
  static constexpr int kVSlots = kStages - kKSlots;
  static_assert(kVSlots >= 1 && kKSlots >= 2, "ring depth");
  __host__ __device__ static constexpr uint32_t k_slot(uint32_t step) { return step % kKSlots; }
  __host__ __device__ static constexpr uint32_t v_slot(uint32_t step) { return kKSlots + step % kVSlots; }
  __host__ __device__ static constexpr uint32_t k_parity(uint32_t step) { return (step / kKSlots) & 1u; }
  __host__ __device__ static constexpr uint32_t v_parity(uint32_t step) { return (step / kVSlots) & 1u; }
  static constexpr int kTmemS = 0, kTmemDP = kKeys, kTmemDS = 2 * kKeys, kTmemDQ = kHeadDim > 128 ? 256 : 384;
  static_assert(kTmemDQ + kHeadDim <= 512 && 2 * kKeys + kKeys / 2 <= kTmemDQ, "tensor memory budget");
};

template <int kHeadDim, int kStages, bool kBf16, bool kSoftcap>
__global__ void __launch_bounds__(kBwdThreads, 1) bwd_dq_kernel(const __grid_constant__ BwdParams p) {
  using Cfg = DqCfg<kHeadDim, kStages>;
  using T = TileCfg<kHeadDim>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = smem + T::kTileBytes;
  uint8_t* sKV = smem + 2 * T::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + kStages * Cfg::kKvTileBytes);
  uint64_t* q_full = bars;
  uint64_t* q_empty = bars + 1;
  uint64_t* kv_full = bars + 2;
  uint64_t* kv_empty = kv_full + kStages;
  uint64_t* sdp_full = kv_empty + kStages;
  uint64_t* sdp_free = sdp_full + 1;
  uint64_t* ds_full = sdp_free + 1;
  uint64_t* ds_free = ds_full + 1;
  uint64_t* dq_full = ds_free + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  SchedMailbox* mbox = reinterpret_cast<SchedMailbox*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  FDA_CTA_STAMP(1, 0);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    sched_init(mbox, 4 * kCmpWG + 2);
    ptx::mbar_init(q_full, 1);
    ptx::mbar_init(q_empty, 1);
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&kv_full[i], 1);
      ptx::mbar_init(&kv_empty[i], 1);
    }
    ptx::mbar_init(sdp_full, 1);
    ptx::mbar_init(sdp_free, 4 * kCmpWG);
    ptx::mbar_init(ds_full, 4 * kCmpWG);
    ptx::mbar_init(ds_free, 1);
    ptx::mbar_init(dq_full, 1);
    ptx::fence_mbar_init();
  }
  if (warp == kLoadWarpB) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int bs = p.block_size;
  const int total_items = p.tiles_per_half * 2 * p.heads * p.batch;

  // Whole warpgroups: four of compute warps, one of the TMA warp, the two MMA warps and an idle warp. The fifth
  // hands registers to the other four. The counts are set inside the role branches, so that the compiler never
  // has to assume the smaller one where the branches meet.
  if (warp >= 4 * kCmpWG) {
  ptx::reg_release_to<kProducerRegs>();
  if (warp == kLoadWarpB) {
    if (lane == 0) {
      uint32_t n_item = 0, slot = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_produce(mbox, n_sched, p.ticket_q, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const QItem it = decode_q_item(p, idx);
        if (!it.valid) continue;
        const KeyPlan plan = make_key_plan(it.qh, it.qa, it.qb, it.n, bs, Cfg::kKeys);
        const QSpans spans = make_q_spans(it, bs);
        if (!ptx::mbar_wait(q_empty, (n_item & 1) ^ 1, abort_flag, 71)) break;
        FDA_TRACE_QI(6, n_item);
        ptx::mbar_expect_tx(q_full, 2 * T::kTileBytes);
        const int q_row = it.row0 + it.qh * it.n + it.qa;
        load_tile<kHeadDim>(sQ, &p.tm_q, q_full, q_row, it.h, it.bcoord);
        load_tile<kHeadDim>(sdO, &p.tm_do, q_full, q_row, it.h, it.bcoord);
        FDA_TRACE_QI(7, n_item);
        for (int s = 0; s < plan.steps() && alive; ++s) {
          int kh, kt;
          plan.step(s, kh, kt);
          if (spans.classify(kh, kt * Cfg::kKeys, Cfg::kKeys) == kTileSkip) continue;
          const int k_row = it.row0 + kh * it.n + kt * Cfg::kKeys;
          // K tiles cycle through slots [0, kKSlots), V tiles through [kKSlots, kStages): a K tile is held until
          // the dQ product of its step, a V tile only until dP, so they need rings of different depth
          for (int which = 0; which < 2; ++which) {
            const uint32_t stage = which == 0 ? Cfg::k_slot(slot) : Cfg::v_slot(slot);
            const uint32_t par = which == 0 ? Cfg::k_parity(slot) : Cfg::v_parity(slot);
            if (!ptx::mbar_wait(&kv_empty[stage], par ^ 1, abort_flag, 72)) { alive = false; break; }
            ptx::mbar_expect_tx(&kv_full[stage], Cfg::kKvTileBytes);
            const CUtensorMap* tm = Cfg::kKeys == 128 ? (which == 0 ? &p.tm_k : &p.tm_v)
                                                      : (which == 0 ? &p.tm_k64 : &p.tm_v64);
#pragma unroll
            for (int c = 0; c < T::kPanels; ++c) {
              ptx::tma_load_4d(sKV + stage * Cfg::kKvTileBytes + c * Cfg::kKvPanelBytes, tm, &kv_full[stage], c * 64,
                               k_row, it.hk, it.bcoord);
            }
          }
          ++slot;
        }
        ++n_item;
      }
      if (*abort_flag) __nanosleep(100000);
    }
  } else if (warp == kMmaWarpB) {
    // ------------------------------------------------------------------ MMA issuer 1: S = Q K^T and dP = dO V^T
    // As in the dK/dV kernel two threads issue MMAs, so that the barrier waits of one overlap the MMAs of the
    // other. They share nothing but the compute warps between them: S / dP of step j + 1 may start as soon as the
    // compute warps have S / dP of step j in registers, whatever the state of dQ.
    if (lane == 0) {
      constexpr int kFmt = kBf16 ? 1 : 0;
      const uint32_t idesc_s = ptx::make_idesc(kTile, Cfg::kKeys, kFmt, false, false);
      constexpr uint32_t kHi = ptx::smem_desc_hi(1024);
      const uint32_t q_lo = ptx::smem_desc_lo(ptx::smem_u32(sQ), 16);
      const uint32_t do_lo = ptx::smem_desc_lo(ptx::smem_u32(sdO), 16);
      const uint32_t kv_lo_k = ptx::smem_desc_lo(ptx::smem_u32(sKV), 16);
      uint32_t n_item = 0, step = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_consume<false>(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const QItem it = decode_q_item(p, idx);
        if (!it.valid) continue;
        const KeyPlan plan = make_key_plan(it.qh, it.qa, it.qb, it.n, bs, Cfg::kKeys);
        const QSpans spans = make_q_spans(it, bs);
        int active = 0;
        for (int s = 0; s < plan.steps(); ++s) {
          int kh, kt;
          plan.step(s, kh, kt);
          active += spans.classify(kh, kt * Cfg::kKeys, Cfg::kKeys) != kTileSkip;
        }
        if (!ptx::mbar_wait(q_full, n_item & 1, abort_flag, 81)) break;
        FDA_TRACE_QI(4, n_item);
        ++n_item;
        for (int j = 0; j < active; ++j, ++step) {
          const uint32_t ks = Cfg::k_slot(step), vs = Cfg::v_slot(step);
          if (!ptx::mbar_wait(&kv_full[ks], Cfg::k_parity(step), abort_flag, 83)) { alive = false; break; }
          if (!ptx::mbar_wait(&kv_full[vs], Cfg::v_parity(step), abort_flag, 84)) { alive = false; break; }
          if (!ptx::mbar_wait(sdp_free, (step & 1) ^ 1, abort_flag, 82)) { alive = false; break; }
          FDA_TRACE_Q(3, step);
          ptx::tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk) {
            const uint32_t a_off = ((kk / 4) * T::kPanelBytes + (kk % 4) * 32) >> 4;
            const uint32_t b_off = ((kk / 4) * Cfg::kKvPanelBytes + (kk % 4) * 32) >> 4;
            ptx::umma_ss_f16_lh(tmem + Cfg::kTmemS, q_lo + a_off, kv_lo_k + ks * (Cfg::kKvTileBytes >> 4) + b_off, kHi,
                                idesc_s, kk > 0);
            ptx::umma_ss_f16_lh(tmem + Cfg::kTmemDP, do_lo + a_off, kv_lo_k + vs * (Cfg::kKvTileBytes >> 4) + b_off, kHi,
                                idesc_s, kk > 0);
          }
          ptx::umma_commit(sdp_full);
          ptx::umma_commit(&kv_empty[vs]);  // V tile no longer needed
          FDA_TRACE_Q(4, step);
        }
        // Q and dO are read by these products only: the tiles of the next item may load while the last dQ
        // product and the epilogue of this one still run
        if (alive) ptx::umma_commit(q_empty);
      }
    }
  } else if (warp == kMmaWarpB + 1) {
    // ------------------------------------------------------------------------------ MMA issuer 2: dQ += dS K
    if (lane == 0) {
      constexpr int kFmt = kBf16 ? 1 : 0;
      const uint32_t idesc_g = ptx::make_idesc(kTile, kHeadDim, kFmt, false, true);
      constexpr uint32_t kHi = ptx::smem_desc_hi(1024);
      const uint32_t kv_lo_mn = ptx::smem_desc_lo(ptx::smem_u32(sKV), Cfg::kKvPanelBytes);
      uint32_t step = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_consume<false>(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const QItem it = decode_q_item(p, idx);
        if (!it.valid) continue;
        const KeyPlan plan = make_key_plan(it.qh, it.qa, it.qb, it.n, bs, Cfg::kKeys);
        const QSpans spans = make_q_spans(it, bs);
        int active = 0;
        for (int s = 0; s < plan.steps(); ++s) {
          int kh, kt;
          plan.step(s, kh, kt);
          active += spans.classify(kh, kt * Cfg::kKeys, Cfg::kKeys) != kTileSkip;
        }
        for (int j = 0; j < active; ++j, ++step) {
          const uint32_t ks = Cfg::k_slot(step);
          // the K tile arrived long ago (S of this step used it); this wait only orders our reads after the copy
          if (!ptx::mbar_wait(&kv_full[ks], Cfg::k_parity(step), abort_flag, 86)) { alive = false; break; }
          FDA_TRACE_Q(0, step);
          if (!ptx::mbar_wait(ds_full, step & 1, abort_flag, 85)) { alive = false; break; }
          FDA_TRACE_Q(1, step);
          ptx::tc_fence_after();
          // dQ += dS K: the packed dS pieces of the compute warpgroups lie side by side, 8 columns per 16 keys
#pragma unroll
          for (int kk = 0; kk < Cfg::kKeys / 16; ++kk) {
            ptx::umma_ts_f16_lh(tmem + Cfg::kTmemDQ, tmem + Cfg::kTmemDS + kk * 8,
                                kv_lo_mn + ks * (Cfg::kKvTileBytes >> 4) + kk * (2048 >> 4), kHi, idesc_g,
                                (j > 0 || kk > 0) ? 1u : 0u);
          }
          ptx::umma_commit(&kv_empty[ks]);
          ptx::umma_commit(ds_free);
          FDA_TRACE_Q(2, step);
        }
        if (!alive) break;
        ptx::umma_commit(dq_full);
        FDA_TRACE_QI(5, n_sched);
      }
    }
  }
  } else {
    ptx::reg_acquire_to<kComputeRegs>();
    const int wg = warp >> 2;                  // which kCols key columns
    const int quad = warp & 3;
    const int row = quad * 32 + lane;          // query row inside the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    uint32_t n_item = 0, cnt = 0, n_sched = 0;
    bool alive = true;

    // What a compute thread keeps of an item. The next item's record is filled while the last dQ product of the
    // current one is still in the tensor pipe, so that its decode and its two statistics loads cost nothing. Two
    // records alternate (no copies: they are meant to stay in registers).
    struct ItemState {
      KeyPlan plan;
      QSpans spans;
      int qh, blk0, blk1;
      int rows_valid;   // of this warp's 32 query rows
      float lse2, delta;
      uint16_t* dst;   // this thread's dQ row
    };
    auto fetch = [&](ItemState& t) -> bool {   // false: no more work (or a wait was abandoned)
      for (;;) {
        const int idx = sched_consume<true>(mbox, n_sched, abort_flag);
        ++n_sched;
        if (idx < 0 || idx >= total_items) return false;
        const QItem it = decode_q_item(p, idx);
        if (!it.valid) continue;
        t.plan = make_key_plan(it.qh, it.qa, it.qb, it.n, bs, Cfg::kKeys);
        t.spans = make_q_spans(it, bs);
        t.qh = it.qh;
        const int r = it.qa + row;
        t.rows_valid = imax(0, imin(32, it.n - (it.qa + quad * 32)));
        const int r_eff = r < it.n ? r : it.n - 1;
        t.blk0 = block_lo(r_eff, bs);
        t.blk1 = imin(t.blk0 + bs, it.n);
        const int64_t seg = stat_segment(p, it.b, it.h, it.qh);
        t.lse2 = p.lse2_pad[seg + r];
        t.delta = p.delta_pad[seg + r];
        const int64_t srow = static_cast<int64_t>(it.row0) + it.qh * it.n + r;
        t.dst = static_cast<uint16_t*>(p.dq) + it.bcoord * p.dq_bs + srow * p.dq_rs + it.h * p.dq_hs;
        return true;
      }
    };

    // One item: its steps, then the next item's record, then the epilogue. Returns whether `nxt` holds an item.
    auto run_item = [&](const ItemState& cur, ItemState& nxt) -> bool {
      if (threadIdx.x == 0) FDA_TRACE_QI(3, n_item);
      for (int s = 0; s < cur.plan.steps() && alive; ++s) {
        int kh, kt;
        cur.plan.step(s, kh, kt);
        constexpr int kKc = Cfg::kKeyCols;
        const int cls = cur.spans.classify(kh, kt * Cfg::kKeys, Cfg::kKeys);
        if (cls == kTileSkip) continue;
        int lo = 0, hi = 0;
        if (cls == kTileMasked) {
          if (cur.qh == 1) { lo = 0; hi = cur.blk1; }
          else if (kh == 1) { lo = 0; hi = cur.blk0; }
          else { lo = cur.blk0; hi = cur.blk1; }
          lo -= kt * Cfg::kKeys + wg * kKc;
          hi -= kt * Cfg::kKeys + wg * kKc;
        }
        if (threadIdx.x == 0) FDA_TRACE_Q(5, cnt);
        if (!ptx::mbar_wait(sdp_full, cnt & 1, abort_flag, 91)) { alive = false; break; }
        if (threadIdx.x == 0) FDA_TRACE_Q(6, cnt);
        ptx::tc_fence_after();
        uint32_t sv[kKc], dpv[kKc];
        if (kKc == 32) {
          ptx::tmem_ld32(tmem + Cfg::kTmemS + lane_addr + wg * kKc, sv);
          ptx::tmem_ld32(tmem + Cfg::kTmemDP + lane_addr + wg * kKc, dpv);
        } else {
          ptx::tmem_ld16(tmem + Cfg::kTmemS + lane_addr + wg * kKc, sv);
          ptx::tmem_ld16(tmem + Cfg::kTmemDP + lane_addr + wg * kKc, dpv);
        }
        ptx::tmem_wait_ld();
        ptx::tc_fence_before();
        ptx::mbar_arrive_warp(sdp_free);
        uint32_t pk_ds[kKc / 2];
        if (cls == kTileMasked) {
          softmax_backward_cols<kKc, kBf16, kSoftcap, false, true, false>(sv, dpv, nullptr, nullptr, cur.lse2, cur.delta,
                                                                          p.scale_log2, p.softcap_pre, lo, hi, nullptr, pk_ds);
        } else {
          softmax_backward_cols<kKc, kBf16, kSoftcap, false, false, false>(sv, dpv, nullptr, nullptr, cur.lse2, cur.delta,
                                                                           p.scale_log2, p.softcap_pre, 0, 0, nullptr, pk_ds);
        }
        if (!ptx::mbar_wait(ds_free, (cnt & 1) ^ 1, abort_flag, 92)) { alive = false; break; }
        ++cnt;
        ptx::tc_fence_after();
        if (kKc == 32) ptx::tmem_st16(tmem + Cfg::kTmemDS + lane_addr + wg * (kKc / 2), pk_ds);
        else ptx::tmem_st8(tmem + Cfg::kTmemDS + lane_addr + wg * (kKc / 2), pk_ds);
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive_warp(ds_full);
        if (threadIdx.x == 0) FDA_TRACE_Q(7, cnt - 1);
      }
      if (!alive) return false;
      const bool have_next = fetch(nxt);
      if (threadIdx.x == 0) FDA_TRACE_QI(2, n_item);
      if (!ptx::mbar_wait(dq_full, n_item & 1, abort_flag, 93)) { alive = false; return false; }
      if (threadIdx.x == 0) FDA_TRACE_QI(0, n_item);
      ++n_item;
      ptx::tc_fence_after();
      constexpr int kChunks = kHeadDim / 32;  // 32-column chunks, dealt round-robin to the warpgroups
#pragma unroll
      for (int g0 = 0; g0 < kChunks; g0 += kCmpWG) {
        const int gidx = g0 + wg;
        if (gidx < kChunks) {
          uint32_t acc[32];
          ptx::tmem_ld32(tmem + Cfg::kTmemDQ + lane_addr + gidx * 32, acc);
          ptx::tmem_wait_ld();
          ptx::store_rows32_grouped<kBf16>(cur.dst, p.dq_rs, cur.rows_valid, gidx * 32, acc, p.softmax_scale, p.head_dim);
        }
      }
      if (threadIdx.x == 0) FDA_TRACE_QI(1, n_item - 1);
      ptx::tc_fence_before();
      return have_next;
    };

    ItemState st0, st1;
    bool have = fetch(st0);
    while (have && alive) {
      have = run_item(st0, st1);
      if (!have || !alive) break;
      have = run_item(st1, st0);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  FDA_CTA_STAMP(1, 1);
  if (warp == kLoadWarpB) ptx::tmem_dealloc(tmem, 512);
}

template <typename Kernel>
int set_smem(Kernel kernel, int bytes, bool* done) {
  int dev = 0;
  FDA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 16 && !done[dev]) {
    FDA_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    done[dev] = true;
  }
  return FDA_OK;
}

template <int kHeadDim, int kStagesKv, int kStagesQ, bool kBf16, bool kSoftcap>
int launch_bwd_instance(const BwdParams& p, int sm_count, unsigned stages, cudaStream_t stream) {
  if (stages & 2u) {
    using Cfg = DkdvCfg<kHeadDim, kStagesKv>;
    auto kernel = bwd_dkdv_kernel<kHeadDim, kStagesKv, kBf16, kSoftcap>;
    static bool done[16] = {false};
    int rc = set_smem(kernel, Cfg::kSmemBytes, done);
    if (rc) return rc;
    const int items = p.tiles_per_half * 2 * p.heads_k * p.batch * Cfg::kPasses;
    const int grid = items < sm_count ? items : sm_count;
    kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    FDA_CUDA_TRY(cudaGetLastError());
  }
  if (stages & 4u) {
    using Cfg = DqCfg<kHeadDim, kStagesQ>;
    auto kernel = bwd_dq_kernel<kHeadDim, kStagesQ, kBf16, kSoftcap>;
    static bool done[16] = {false};
    int rc = set_smem(kernel, Cfg::kSmemBytes, done);
    if (rc) return rc;
    const int items = p.tiles_per_half * 2 * p.heads * p.batch;
    const int grid = items < sm_count ? items : sm_count;
    kernel<<<grid, kBwdThreads, Cfg::kSmemBytes, stream>>>(p);
    FDA_CUDA_TRY(cudaGetLastError());
  }
  return FDA_OK;
}

template <int kHeadDim, int kStagesKv, int kStagesQ>
int dispatch_bwd(const BwdParams& p, int sm_count, bool bf16, bool softcap, unsigned stages, cudaStream_t stream) {
  if (bf16) {
    return softcap ? launch_bwd_instance<kHeadDim, kStagesKv, kStagesQ, true, true>(p, sm_count, stages, stream)
                   : launch_bwd_instance<kHeadDim, kStagesKv, kStagesQ, true, false>(p, sm_count, stages, stream);
  }
  return softcap ? launch_bwd_instance<kHeadDim, kStagesKv, kStagesQ, false, true>(p, sm_count, stages, stream)
                 : launch_bwd_instance<kHeadDim, kStagesKv, kStagesQ, false, false>(p, sm_count, stages, stream);
}

inline int64_t round_up64(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

}  // namespace

// Workspace: delta_pad then lse2_pad, each batch * heads * 2 * n_pad floats (256-byte aligned pieces).
size_t bwd_workspace_bytes(const FdaProblem& pr) {
  const int64_t n_pad = round_up64(pr.seqlen / 2 > 0 ? pr.seqlen / 2 : 1, kTile);
  const int64_t one = round_up64(static_cast<int64_t>(pr.batch) * pr.heads * 2 * n_pad * 4, 256);
  return static_cast<size_t>(2 * one + 256);
}

int launch_bwd(const FdaBwdArgs& a, cudaStream_t stream, unsigned stage_mask) {
  const FdaProblem& pr = a.p;
  DeviceInfo info;
  int rc = current_device_info(&info);
  if (rc) return rc;
  if (info.cc_major != 10) return FDA_ERR_ARCH;
  const int d = pr.head_dim;
  const int d_round = d <= 64 ? 64 : (d <= 128 ? 128 : 256);
  const bool varlen = pr.cu_seqlens != nullptr;
  const int64_t rows = varlen ? pr.total : pr.seqlen;
  const int tma_batch = varlen ? 1 : pr.batch;
  const bool fp16 = pr.dtype == FDA_FP16;

  BwdParams p;
  memset(&p, 0, sizeof(p));
  rc = encode_tile_map(&p.tm_q, a.q.ptr, 2, false, fp16, d, rows, pr.heads, tma_batch, a.q.row_stride,
                       a.q.head_stride, a.q.batch_stride, 64, kTile);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_do, a.dout.ptr, 2, false, fp16, d, rows, pr.heads, tma_batch, a.dout.row_stride,
                       a.dout.head_stride, a.dout.batch_stride, 64, kTile);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_q64, a.q.ptr, 2, false, fp16, d, rows, pr.heads, tma_batch, a.q.row_stride,
                       a.q.head_stride, a.q.batch_stride, 64, kSub);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_do64, a.dout.ptr, 2, false, fp16, d, rows, pr.heads, tma_batch, a.dout.row_stride,
                       a.dout.head_stride, a.dout.batch_stride, 64, kSub);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_k64, a.k.ptr, 2, false, fp16, d, rows, pr.heads_k, tma_batch, a.k.row_stride,
                       a.k.head_stride, a.k.batch_stride, 64, 64);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_v64, a.v.ptr, 2, false, fp16, d, rows, pr.heads_k, tma_batch, a.v.row_stride,
                       a.v.head_stride, a.v.batch_stride, 64, 64);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_k, a.k.ptr, 2, false, fp16, d, rows, pr.heads_k, tma_batch, a.k.row_stride,
                       a.k.head_stride, a.k.batch_stride, 64, kTile);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_v, a.v.ptr, 2, false, fp16, d, rows, pr.heads_k, tma_batch, a.v.row_stride,
                       a.v.head_stride, a.v.batch_stride, 64, kTile);
  if (rc) return rc;
  // the preprocess and the epilogues use 16-byte vector accesses on rows of out / dout / dq / dk / dv
  const FdaTensor* vec[] = {&a.out, &a.dout, &a.dq, &a.dk, &a.dv};
  for (const FdaTensor* t : vec) {
    if ((reinterpret_cast<uintptr_t>(t->ptr) & 15) || (t->row_stride % 8) || (t->head_stride % 8) ||
        (!varlen && (t->batch_stride % 8))) {
      return FDA_ERR_STRIDE;
    }
  }
  p.wide_store = (d % 16 == 0) ? 1 : 0;
  const FdaTensor* grads[] = {&a.dq, &a.dk, &a.dv};
  for (const FdaTensor* t : grads) {
    if ((reinterpret_cast<uintptr_t>(t->ptr) & 31) || (t->row_stride % 16) || (t->head_stride % 16) ||
        (!varlen && (t->batch_stride % 16))) {
      p.wide_store = 0;
    }
  }
  p.out = a.out.ptr;
  p.dout = a.dout.ptr;
  p.dq = a.dq.ptr;
  p.dk = a.dk.ptr;
  p.dv = a.dv.ptr;
  auto set3 = [&](const FdaTensor& t, int64_t& bs_, int64_t& rs_, int64_t& hs_) {
    bs_ = varlen ? 0 : t.batch_stride;
    rs_ = t.row_stride;
    hs_ = t.head_stride;
  };
  set3(a.out, p.o_bs, p.o_rs, p.o_hs);
  set3(a.dout, p.do_bs, p.do_rs, p.do_hs);
  set3(a.dq, p.dq_bs, p.dq_rs, p.dq_hs);
  set3(a.dk, p.dk_bs, p.dk_rs, p.dk_hs);
  set3(a.dv, p.dv_bs, p.dv_rs, p.dv_hs);
  p.lse = a.lse;
  p.cu_seqlens = pr.cu_seqlens;
  p.batch = pr.batch;
  p.seqlen = pr.seqlen;
  p.total = pr.total;
  p.heads = pr.heads;
  p.heads_k = pr.heads_k;
  p.head_dim = d;
  p.block_size = pr.block_size;
  p.n_pad = static_cast<int>(round_up64(pr.seqlen / 2 > 0 ? pr.seqlen / 2 : 1, kTile));
  p.tiles_per_half = p.n_pad / kTile;
  {
    // dK/dV: the noisy key tiles (the second half of the ranks) are short; dQ: the shortest eighth (fractions
    // found by measurement on the benchmark shape)
    const int per_bh = 2 * p.tiles_per_half;
    p.n_long_kv = per_bh - (FDA_SHORT8_KV * per_bh) / 8;
    if (p.n_long_kv < 1) p.n_long_kv = 1;
    p.n_long_q = per_bh - (FDA_SHORT8_Q * per_bh) / 8;
  }
  const int64_t one = round_up64(static_cast<int64_t>(pr.batch) * pr.heads * 2 * p.n_pad * 4, 256);
  p.delta_pad = static_cast<float*>(a.workspace);
  p.lse2_pad = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + one);
  p.ticket_kv = reinterpret_cast<int*>(static_cast<uint8_t*>(a.workspace) + 2 * one);
  p.ticket_q = p.ticket_kv + 32;
  if (stage_mask & 6u) FDA_CUDA_TRY(cudaMemsetAsync(p.ticket_kv, 0, 256, stream));
  const bool softcap = pr.softcap > 0.f;
  p.softmax_scale = pr.softmax_scale;
  if (softcap) {
    p.scale_log2 = pr.softcap * kLog2e;
    p.softcap_pre = pr.softmax_scale / pr.softcap;
  } else {
    p.scale_log2 = pr.softmax_scale * kLog2e;
    p.softcap_pre = 0.f;
  }
  int sm_count = info.sm_count - (pr.sm_margin > 0 ? pr.sm_margin : 0);
  if (sm_count < 1) sm_count = 1;
  const bool bf16 = pr.dtype == FDA_BF16;

  if (stage_mask & 1u) {
    const int lanes = d <= 64 ? 8 : (d <= 128 ? 16 : 32);
    const int rows_per_block = 8 * (32 / lanes) * kPreUnroll;
    dim3 grid((p.n_pad + rows_per_block - 1) / rows_per_block, 2 * pr.heads, pr.batch);
    if (bf16) {
      if (lanes == 8) bwd_preprocess_kernel<true, 8><<<grid, 256, 0, stream>>>(p);
      else if (lanes == 16) bwd_preprocess_kernel<true, 16><<<grid, 256, 0, stream>>>(p);
      else bwd_preprocess_kernel<true, 32><<<grid, 256, 0, stream>>>(p);
    } else {
      if (lanes == 8) bwd_preprocess_kernel<false, 8><<<grid, 256, 0, stream>>>(p);
      else if (lanes == 16) bwd_preprocess_kernel<false, 16><<<grid, 256, 0, stream>>>(p);
      else bwd_preprocess_kernel<false, 32><<<grid, 256, 0, stream>>>(p);
    }
    FDA_CUDA_TRY(cudaGetLastError());
  }
  if (d_round == 64) return dispatch_bwd<64, 6, 7>(p, sm_count, bf16, softcap, stage_mask, stream);
  if (d_round == 128) return dispatch_bwd<128, 4, 5>(p, sm_count, bf16, softcap, stage_mask, stream);
  return dispatch_bwd<256, 1, 3>(p, sm_count, bf16, softcap, stage_mask, stream);
}

#ifdef FDA_WAIT_CLOCKS
extern "C" int fda_debug_waits_bwd(unsigned long long* out256) {
  static unsigned long long zero[256];
  if (cudaMemcpyFromSymbol(out256, g_fda_wait, sizeof(zero)) != cudaSuccess) return 1;
  if (cudaMemcpyToSymbol(g_fda_wait, zero, sizeof(zero)) != cudaSuccess) return 1;
  return 0;
}
#endif

// ------------------------------------------------------------------------------------------------------------
// Backward without a caller-provided workspace (fda_bwd_noalloc). The scratch the three kernels share (delta,
// LSE * log2(e), the two work counters) lives in this fixed array, which every GPU that loads the library holds
// until the process exits. In host code the array's name is only a stand-in for the symbol: the device address
// is looked up once per device, with that device current, and that pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_bwd_noalloc_scratch[FDA_NOALLOC_SCRATCH_BYTES];

int launch_bwd_noalloc(const FdaBwdArgs& a, cudaStream_t stream) {
  if (bwd_workspace_bytes(a.p) > static_cast<size_t>(FDA_NOALLOC_SCRATCH_BYTES)) return FDA_ERR_SCRATCH_LIMIT;
  static void* scratch_of_device[64] = {nullptr};
  int dev = 0;
  FDA_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return FDA_ERR_UNSUPPORTED;
  if (scratch_of_device[dev] == nullptr) {
    void* ptr = nullptr;
    FDA_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_bwd_noalloc_scratch));
    scratch_of_device[dev] = ptr;
  }
  FdaBwdArgs with_scratch = a;
  with_scratch.workspace = scratch_of_device[dev];
  with_scratch.workspace_bytes = FDA_NOALLOC_SCRATCH_BYTES;
  return launch_bwd(with_scratch, stream, 7u);
}

int read_status_bwd(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}

}  // namespace fda
