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
#include "bwd_common.cuh"

namespace fda {
namespace {

// ------------------------------------------------------------------------------------------------------------
// 1. preprocess
// ------------------------------------------------------------------------------------------------------------
// rows per thread group; measured on the benchmark shape (268 MB read): 1 row 0.063 ms, 2 rows 0.053, 4 rows 0.066,
// 8 rows 0.072
constexpr int kPreUnroll = 2;

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

// ------------------------------------------------------------------------------------------------------------
// 2. dK / dV
// ------------------------------------------------------------------------------------------------------------

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
  const int total_items = kv_item_count(p) * Cfg::kPasses;

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
          ptx::mbar_expect_tx(&st_full[stage], 2 * Cfg::kSubTileBytes + 512);
          const int q_row = it.row0 + st.qh * it.n + st.sa;
#pragma unroll
          for (int c = 0; c < T::kPanels; ++c) {
            ptx::tma_load_4d(base + c * Cfg::kSubPanelBytes, &p.tm_q64, &st_full[stage], c * 64, q_row, st.h, it.bcoord);
            ptx::tma_load_4d(base + Cfg::kSubTileBytes + c * Cfg::kSubPanelBytes, &p.tm_do64, &st_full[stage], c * 64,
                             q_row, st.h, it.bcoord);
          }
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
          if (!ptx::mbar_wait(&pds_full[u], (g >> 1) & 1u, abort_flag, 53)) { alive = false; break; }
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
      const int idx = sched_consume<true>(mbox, n_sched, abort_flag);
      if (idx < 0 || idx >= total_items) break;
      const KvItem it = decode_kv_item(p, idx / Cfg::kPasses);
      const int pass_col0 = (idx % Cfg::kPasses) * Cfg::kAccDim;
      if (!it.valid) continue;
      const int kj = it.k0 + row;
      // queries that see this thread's key: same-half tiles and (clean keys only) noisy tiles of later blocks
      int same_lo, same_hi, cross_lo, cross_hi;
      query_interval(it.kh, it.kh, kj, it.n, bs, same_lo, same_hi);
      query_interval(0, 1, kj, it.n, bs, cross_lo, cross_hi);
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
        if (!ptx::mbar_wait(&sdp_full[u], (gc >> 1) & 1u, abort_flag, 61)) { alive = false; break; }
        ++gc;
        ptx::tc_fence_after();
        const uint32_t st_t = tmem + u * 128 + lane_addr + wg * kSubCols;
        const uint32_t dpt_t = st_t + 64;
        uint32_t sv[kSubCols], dpv[kSubCols];
        ptx::tmem_ld16(st_t, sv);
        ptx::tmem_ld16(dpt_t, dpv);
        ptx::tmem_wait_ld();
        uint32_t pk_p[kSubCols / 2], pk_ds[kSubCols / 2];
        const float* l2 = l2r;
        const float* dl = dlr;
        if (hdr.x & 2) {
          const int lo = ((hdr.x & 4) ? same_lo : cross_lo) - (hdr.y + wg * kSubCols);
          const int hi = ((hdr.x & 4) ? same_hi : cross_hi) - (hdr.y + wg * kSubCols);
          softmax_backward_cols<kSubCols, kBf16, kSoftcap, true, true, true>(sv, dpv, l2, dl, 0.f, 0.f, p.scale_log2,
                                                                              p.softcap_pre, lo, hi, pk_p, pk_ds);
        } else {
          softmax_backward_cols<kSubCols, kBf16, kSoftcap, true, false, true>(sv, dpv, l2, dl, 0.f, 0.f, p.scale_log2,
                                                                               p.softcap_pre, 0, 0, pk_p, pk_ds);
        }
        // a warp overwrites only columns it has itself already loaded: its packed P^T / dS^T pieces go to the
        // start of its own kSubCols columns
        ptx::tmem_st8(st_t, pk_p);
        ptx::tmem_st8(dpt_t, pk_ds);
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive_warp(&pds_full[u]);
      }
      if (!alive) break;
      ++n_item;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
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
  int rem, tiles;
  if (p.vl.base != nullptr) {
    // packed batch: exactly the query tiles that exist, longest sample first, head after head inside a sample
    const VarlenPos pos = varlen_locate(p.vl, idx, 2 * p.heads);
    tiles = pos.units;
    it.b = pos.b;
    it.h = pos.rem / (2 * tiles);
    rem = pos.rem - it.h * (2 * tiles);
  } else {
    const int per_bh = 2 * p.tiles_per_half;
    int bh;
    two_phase_order(idx, per_bh, p.n_long_q, p.batch * p.heads, bh, rem);
    tiles = p.tiles_per_half;
    it.b = bh / p.heads;
    it.h = bh - it.b * p.heads;
  }
  it.qh = rem & 1;
  const int t_rev = rem >> 1;
  it.hk = it.h / (p.heads / p.heads_k);
  const Sample sm = sample_of(p, it.b);
  it.n = sm.n;
  it.row0 = sm.row0;
  it.bcoord = sm.bcoord;
  it.qa = (tiles - 1 - t_rev) * kTile;
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
  const int total_items = (p.vl.base != nullptr ? p.vl.base[0] : p.tiles_per_half * p.batch) * 2 * p.heads;

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
        ptx::mbar_expect_tx(q_full, 2 * T::kTileBytes);
        const int q_row = it.row0 + it.qh * it.n + it.qa;
        load_tile<kHeadDim>(sQ, &p.tm_q, q_full, q_row, it.h, it.bcoord);
        load_tile<kHeadDim>(sdO, &p.tm_do, q_full, q_row, it.h, it.bcoord);
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
        ++n_item;
        for (int j = 0; j < active; ++j, ++step) {
          const uint32_t ks = Cfg::k_slot(step), vs = Cfg::v_slot(step);
          if (!ptx::mbar_wait(&kv_full[ks], Cfg::k_parity(step), abort_flag, 83)) { alive = false; break; }
          if (!ptx::mbar_wait(&kv_full[vs], Cfg::v_parity(step), abort_flag, 84)) { alive = false; break; }
          if (!ptx::mbar_wait(sdp_free, (step & 1) ^ 1, abort_flag, 82)) { alive = false; break; }
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
          if (!ptx::mbar_wait(ds_full, step & 1, abort_flag, 85)) { alive = false; break; }
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
        }
        if (!alive) break;
        ptx::umma_commit(dq_full);
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
        if (!ptx::mbar_wait(sdp_full, cnt & 1, abort_flag, 91)) { alive = false; break; }
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
      }
      if (!alive) return false;
      const bool have_next = fetch(nxt);
      if (!ptx::mbar_wait(dq_full, n_item & 1, abort_flag, 93)) { alive = false; return false; }
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
  if (warp == kLoadWarpB) ptx::tmem_dealloc(tmem, 512);
}

template <int kHeadDim, int kStagesKv, int kStagesQ, bool kBf16, bool kSoftcap>
int launch_bwd_instance(const BwdParams& p, int sm_count, unsigned stages, cudaStream_t stream) {
  if (stages & 2u) {
    using Cfg = DkdvCfg<kHeadDim, kStagesKv>;
    auto kernel = bwd_dkdv_kernel<kHeadDim, kStagesKv, kBf16, kSoftcap>;
    static PerDeviceFlags smem_set;
    int rc = set_dynamic_smem(kernel, Cfg::kSmemBytes, smem_set);
    if (rc) return rc;
    const int items = bwd_item_bound(p, p.heads_k) * Cfg::kPasses;
    const int grid = items < sm_count ? items : sm_count;
    kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
    FDA_CUDA_TRY(cudaGetLastError());
  }
  if (stages & 4u) {
    using Cfg = DqCfg<kHeadDim, kStagesQ>;
    auto kernel = bwd_dq_kernel<kHeadDim, kStagesQ, kBf16, kSoftcap>;
    static PerDeviceFlags smem_set;
    int rc = set_dynamic_smem(kernel, Cfg::kSmemBytes, smem_set);
    if (rc) return rc;
    const int items = bwd_item_bound(p, p.heads);
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

// bwd_fused_sm100.cu
size_t bwd_fused_acc_bytes(const FdaProblem& pr);
int64_t bwd_fused_acc_tiles(const FdaProblem& pr);
int launch_bwd_fused(const BwdParams& p, int d_round, bool bf16, bool softcap, int sm_count, unsigned stages,
                     cudaStream_t stream);

// The single-pass backward adds dQ partials in an order that depends on scheduling and needs head dim <= 128.
bool bwd_single_pass(const FdaProblem& pr) { return pr.deterministic == 0 && pr.head_dim <= 128; }

// Scratch of the split backward: delta_pad then lse2_pad, each batch * heads * 2 * n_pad floats (256-byte aligned
// pieces), then 256 bytes of work counters.
size_t bwd_split_workspace_bytes(const FdaProblem& pr) {
  const int64_t n_pad = round_up64(pr.seqlen / 2 > 0 ? pr.seqlen / 2 : 1, kTile);
  const int64_t one = round_up64(static_cast<int64_t>(pr.batch) * pr.heads * 2 * n_pad * 4, 256);
  // ... and for packed batches the work list (samples longest first, running tile counts)
  return static_cast<size_t>(2 * one + 256) + (pr.cu_seqlens != nullptr ? varlen_list_bytes(pr.batch) : 0);
}

// The single-pass backward keeps its fp32 dQ accumulator behind that.
size_t bwd_workspace_bytes(const FdaProblem& pr) {
  size_t bytes = bwd_split_workspace_bytes(pr);
  if (bwd_single_pass(pr)) bytes += static_cast<size_t>(round_up64(static_cast<int64_t>(bwd_fused_acc_bytes(pr)), 256));
  return bytes;
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
  const int64_t one = round_up64(static_cast<int64_t>(pr.batch) * pr.heads * 2 * p.n_pad * 4, 256);
  p.delta_pad = static_cast<float*>(a.workspace);
  p.lse2_pad = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + one);
  p.ticket_kv = reinterpret_cast<int*>(static_cast<uint8_t*>(a.workspace) + 2 * one);
  p.ticket_q = p.ticket_kv + 32;
  const bool single_pass = bwd_single_pass(pr) && (stage_mask & FDA_BWD_FORCE_SPLIT) == 0;
  if (single_pass) {
    if (a.workspace_bytes < bwd_workspace_bytes(pr)) return FDA_ERR_WORKSPACE;
    p.dq_acc = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + bwd_split_workspace_bytes(pr));
    p.acc_tiles = static_cast<int>(bwd_fused_acc_tiles(pr));
    p.acc_floats = static_cast<int64_t>(bwd_fused_acc_bytes(pr) / 4);
  }
  if (stage_mask & 6u) FDA_CUDA_TRY(cudaMemsetAsync(p.ticket_kv, 0, 256, stream));
  if (varlen) {
    // the work list of the persistent kernels is built on the device (no host synchronisation); every stage call
    // rebuilds it, so stages may be launched one by one
    int* list = reinterpret_cast<int*>(static_cast<uint8_t*>(a.workspace) + 2 * one + 256);
    if (stage_mask & 6u) {
      rc = launch_varlen_prepare(pr.cu_seqlens, pr.batch, kTile, list, stream);
      if (rc) return rc;
    }
    p.vl.base = list;
    p.vl.batch = pr.batch;
  }
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
  {
    // dK/dV: the noisy key tiles (the second half of the ranks) are short; dQ: the shortest eighth (fractions
    // found by measurement on the benchmark shape); few items per CTA: rank for rank over all of them
    const int per_bh = 2 * p.tiles_per_half;
    p.n_long_kv = order_n_long(per_bh, FDA_SHORT8_KV, static_cast<long long>(per_bh) * pr.batch * pr.heads_k, sm_count);
    p.n_long_q = order_n_long(per_bh, FDA_SHORT8_Q, static_cast<long long>(per_bh) * pr.batch * pr.heads, sm_count);
  }
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
  if (single_pass) return launch_bwd_fused(p, d_round, bf16, softcap, sm_count, stage_mask, stream);
  if (d_round == 64) return dispatch_bwd<64, 6, 7>(p, sm_count, bf16, softcap, stage_mask, stream);
  if (d_round == 128) return dispatch_bwd<128, 4, 5>(p, sm_count, bf16, softcap, stage_mask, stream);
  return dispatch_bwd<256, 1, 3>(p, sm_count, bf16, softcap, stage_mask, stream);
}


// ------------------------------------------------------------------------------------------------------------
// Backward without a caller-provided workspace (fda_bwd_noalloc). It always runs the split backward, whose
// scratch (delta, LSE * log2(e), the two work counters) is small; that scratch lives in this fixed array, which
// every GPU that loads the library holds until the process exits. In host code the array's name is only a
// stand-in for the symbol: the device address is looked up once per device, with that device current, and that
// pointer is what the kernels receive.
// ------------------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_bwd_noalloc_scratch[FDA_NOALLOC_SCRATCH_BYTES];

int launch_bwd_noalloc(const FdaBwdArgs& a, cudaStream_t stream) {
  if (bwd_split_workspace_bytes(a.p) > static_cast<size_t>(FDA_NOALLOC_SCRATCH_BYTES)) return FDA_ERR_SCRATCH_LIMIT;
  static std::atomic<void*> scratch_of_device[kMaxCachedDevices];
  int dev = 0;
  FDA_CUDA_TRY(cudaGetDevice(&dev));
  const bool cached = dev >= 0 && dev < kMaxCachedDevices;
  void* ptr = cached ? scratch_of_device[dev].load(std::memory_order_acquire) : nullptr;
  if (ptr == nullptr) {
    FDA_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_bwd_noalloc_scratch));
    if (cached) scratch_of_device[dev].store(ptr, std::memory_order_release);
  }
  FdaBwdArgs with_scratch = a;
  with_scratch.workspace = ptr;
  with_scratch.workspace_bytes = FDA_NOALLOC_SCRATCH_BYTES;
  return launch_bwd(with_scratch, stream, 7u | FDA_BWD_FORCE_SPLIT);
}

int read_status_bwd(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}

}  // namespace fda
