// Pieces shared by the backward kernels of block-diffusion attention for sm_100a: the launch parameters, the
// per-sample addressing, the statistics layout written by the preprocess, the softmax-backward arithmetic and the
// key-tile work items of the dK/dV-stationary kernels. The reference keeps the equivalent pieces in
// csrc/fda/flash.h:15-137 (parameters), csrc/fda/diffusion.h:43-69, :196-261 (offsets, tile lists) and
// csrc/fda/mainloop_bwd_sm90_tma_gmma_ws.hpp:836-893 (arithmetic).
#pragma once

#include "geometry.h"
#include "host_util.h"
#include "ptx.cuh"
#include "sched.cuh"
#include "varlen_list.cuh"

#ifndef FDA_SHORT8_KV
#define FDA_SHORT8_KV 4   // eighths of a (sample, head)'s items that count as short: dK/dV-stationary kernels
#endif
#ifndef FDA_SHORT8_Q
#define FDA_SHORT8_Q 1    // the same for the dQ kernel
#endif

namespace fda {

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
  float* dq_acc;     // single-pass backward: fp32 dQ accumulator, [heads][acc_tiles][head dim][64 queries]
  int acc_tiles;     // 64-row accumulator tiles per query head
  int64_t acc_floats;   // size of the accumulator
  VarlenList vl;     // packed batches: samples longest first with running 128-row tile counts (base == nullptr otherwise)
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
      // the derivative of the cap goes onto P first: the single-pass backward computes P (1 - tanh^2) in the first
      // half of its arithmetic and meets dP only in the second, and both forms round alike
      float d = (kSoftcap ? pr * dt : pr) * (__uint_as_float(dp[col]) - dl);
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

struct KvItem {
  int b, hk, kh, k0, k1, n, row0, bcoord;
  bool valid;
};

__device__ __forceinline__ KvItem decode_kv_item(const BwdParams& p, int idx) {
  // (sample, KV head)-major: the CTAs running at the same time stream the Q / dO tiles of a few heads, which then
  // stay in L2. Inside a head: clean key tiles first, early ones first (they are seen by the most queries), then
  // the noisy key tiles (one block of queries each) as filler.
  KvItem it;
  int rem, tiles;
  if (p.vl.base != nullptr) {
    // packed batch: exactly the key tiles that exist, longest sample first, head after head inside a sample
    const VarlenPos pos = varlen_locate(p.vl, idx, 2 * p.heads_k);
    tiles = pos.units;
    it.b = pos.b;
    it.hk = pos.rem / (2 * tiles);
    rem = pos.rem - it.hk * (2 * tiles);
  } else {
    const int per_bh = 2 * p.tiles_per_half;
    int bh;
    two_phase_order(idx, per_bh, p.n_long_kv, p.batch * p.heads_k, bh, rem);
    tiles = p.tiles_per_half;
    it.b = bh / p.heads_k;
    it.hk = bh - it.b * p.heads_k;
  }
  it.kh = rem < tiles ? 1 : 0;
  const int kt = rem < tiles ? rem : rem - tiles;
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
// with no visible row is skipped. All roles walk this sequence identically.
// Number of key-tile items of a launch: known to the host for the batched layout, read from the work list otherwise.
__device__ __forceinline__ int kv_item_count(const BwdParams& p) {
  return (p.vl.base != nullptr ? p.vl.base[0] : p.tiles_per_half * p.batch) * 2 * p.heads_k;
}

// Host side: the number of items (128-row tiles x 2 halves x heads) a launch has at most; exact for the batched
// layout, an upper bound for packed batches (whose real count only the device knows).
inline int bwd_item_bound(const BwdParams& p, int heads) {
  if (p.vl.base == nullptr) return p.tiles_per_half * 2 * heads * p.batch;
  const int64_t bound = (static_cast<int64_t>(p.total) / (2 * kTile) + p.batch) * 2 * heads;
  return bound > (1 << 30) ? (1 << 30) : static_cast<int>(bound);
}

struct SubStep {
  int h, qh, sa, sb, cls;
};

// Calls fn(SubStep) for every non-skipped sub-step of the item, in order; stops early when fn returns false.
template <typename Fn>
__device__ __forceinline__ bool for_each_substep(const KvItem& it, const QueryPlan& plan, const KvSpans& spans,
                                                 int group, Fn&& fn) {
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
}

}  // namespace fda
