// Single-pass backward of block-diffusion attention for sm_100a: dK, dV and dQ from five GEMMs per tile pair.
//
// One CTA per (128-key tile, KV head, sample, half), persistent. K and V stay in shared memory; the visible query
// rows of every query head of the group stream through in sub-tiles of 64 rows. Per sub-tile:
//   S^T = K Q^T, dP^T = V dO^T          (keys on tensor-memory lanes, 64 columns each, double buffered)
//   P^T = exp2(S^T c - LSE2), dS^T = P^T (dP^T - delta)          (compute warps; P^T back to tensor memory,
//                                                                 dS^T to shared memory, both 16-bit)
//   dV += P^T dO, dK += dS^T Q          (accumulators in tensor memory for the whole key tile)
//   dQ^T = K^T dS^T                     (head dim on lanes, 64 query columns, written over the consumed dP^T buffer)
// The partial dQ^T of a (key tile, query sub-tile) pair is added into an fp32 accumulator in global memory with
// vector reductions (red.global.add.v4.f32); `bwd_dq_convert_kernel` then scales, rounds and transposes it into dQ.
// The accumulator is private scratch, so its layout is chosen for the adds: one 64-query sub-tile is stored as
// [head dim][64 queries], which is the tensor-memory layout of dQ^T (a thread owns one head-dim row).
//
// The reference does the same five GEMMs per pair with an fp32 dQ accumulator reduced through global memory
// (csrc/fda/mainloop_bwd_sm90_tma_gmma_ws.hpp:815-984 `bwd_step`, :605-664 `store_dq`, there with
// cp.reduce.async.bulk from shared memory) and converts afterwards (flash_bwd_postprocess_kernel.h:160-264).
// The order of the adds depends on scheduling, so this path serves deterministic == 0 only; the deterministic
// backward keeps the two-kernel split (dK/dV kernel + dQ kernel), which has no cross-CTA reduction.
#include "bwd_common.cuh"

namespace fda {
namespace {

template <int kHeadDim, int kStages>
struct FusedCfg {
  using T = TileCfg<kHeadDim>;
  static constexpr int kSubTileBytes = kSub * kHeadDim * 2;     // Q or dO sub-tile
  static constexpr int kSubPanelBytes = kSub * 128;             // one 64-column panel of a sub-tile
  static constexpr int kStageBytes = 2 * kSubTileBytes + 1024;  // Q, dO, lse2[64], delta[64], header
  static constexpr int kHeaderOffset = 2 * kSubTileBytes + 512;
  static constexpr int kDsBytes = kTile * kSub * 2;             // dS^T: [128 keys][64 queries], 128-byte rows
  static constexpr int kSmemBytes = 2 * T::kTileBytes + kStages * kStageBytes + 2 * kDsBytes + 1024 + 512;
  // tensor memory: buffer u holds S^T at u*128 (P^T written back in place) and dP^T at u*128 + 64 (dQ^T of the
  // same sub-step lands there once dP^T is in registers); dK and dV behind
  static constexpr int kTmemDK = 256, kTmemDV = 256 + kHeadDim;
  static_assert(kHeadDim == 64 || kHeadDim == 128, "the fused backward covers head dimensions up to 128");
  static_assert(kStageBytes % 1024 == 0 && kDsBytes % 1024 == 0, "tiles stay 1024-byte aligned for the swizzle");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
};

// Index of the 64-row accumulator tile that holds query row `sa` (a multiple of 64) of half `qh` of a sample whose
// first row in the packed row space is `grow0`. Every half starts at its own tile: the "+ 2 b + qh" gives each of
// the 2 * batch halves one tile of slack, so rounding the start down never lets two halves share a tile.
__device__ __forceinline__ int acc_tile_of(int grow0, int n, int b, int qh, int sa) {
  return (grow0 + qh * n) / kSub + 2 * b + qh + sa / kSub;
}

__device__ __forceinline__ void red_add_v4(float* addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(__uint_as_float(a)),
               "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d))
               : "memory");
}

template <int kHeadDim, int kStages, bool kBf16, bool kSoftcap>
__global__ void __launch_bounds__(kDkdvThreads, 1) bwd_fused_kernel(const __grid_constant__ BwdParams p) {
  using Cfg = FusedCfg<kHeadDim, kStages>;
  using T = TileCfg<kHeadDim>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = smem + T::kTileBytes;   // directly behind K: for head dim 64 it is the second panel of the M = 128
                                        // operand of dQ^T (rows 64..127 of that product are never read)
  uint8_t* sStage = smem + 2 * T::kTileBytes;
  uint8_t* sDs = sStage + kStages * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sDs + 2 * Cfg::kDsBytes);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + 1;
  uint64_t* st_full = bars + 2;
  uint64_t* st_empty = st_full + kStages;
  uint64_t* sdp_full = st_empty + kStages;   // [2] S^T / dP^T of buffer u are complete
  uint64_t* pds_full = sdp_full + 2;         // [2] P^T (tensor memory) and dS^T (shared memory) are written
  uint64_t* dq_full = pds_full + 2;          // [2] dQ^T of buffer u is complete
  uint64_t* buf_free = dq_full + 2;          // [2] dV / dK have read buffer u and dQ^T is in the drain warps' registers
  uint64_t* acc_full = buf_free + 2;
  uint64_t* acc_free = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* dq_desc = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2][2]: {last sub-step, accumulator tile}
  SchedMailbox* mbox = reinterpret_cast<SchedMailbox*>(reinterpret_cast<uint8_t*>(bars) + 256);
  static_assert((12 + 2 * kStages) * 8 + 6 * 4 <= 256, "barrier area");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    sched_init(mbox, 4 * kCmpWG + 2 + 4);   // compute warps, two MMA issuers, four drain / epilogue warps
    ptx::mbar_init(kv_full, 1);
    ptx::mbar_init(kv_empty, 1);
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&st_full[i], 1);
      ptx::mbar_init(&st_empty[i], 1);
    }
    for (int u = 0; u < 2; ++u) {
      ptx::mbar_init(&sdp_full[u], 1);
      ptx::mbar_init(&pds_full[u], 4 * kCmpWG);
      ptx::mbar_init(&dq_full[u], 1);
      ptx::mbar_init(&buf_free[u], 1 + 4);   // the commit behind dV / dK and the four drain warps
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
  const int total_items = p.tiles_per_half * 2 * p.heads_k * p.batch;

  if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------------------------- dQ drain + dK/dV epilogue
    // Four warps, one per quarter of the tensor-memory lanes. Per sub-step they add the partial dQ^T (lane = head-dim
    // row, 64 query columns) into the global accumulator; after the last sub-step of an item they write dK and dV.
    ptx::reg_release_to<kDkdvEpilogueRegs>();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const bool drain_rows = quad * 32 < kHeadDim;   // head dim 64: the upper two quarters hold nothing of dQ^T
    uint32_t n_item = 0, gd = 0;
    bool alive = true;
    for (uint32_t n_sched = 0; alive; ++n_sched) {
      const int idx = sched_consume<true>(mbox, n_sched, abort_flag);
      if (idx < 0 || idx >= total_items) break;
      const KvItem it = decode_kv_item(p, idx);
      if (!it.valid) continue;
      for (bool last = false; alive && !last; ++gd) {
        const uint32_t u = gd & 1u, par = (gd >> 1) & 1u;
        // the compute warps' barrier orders their description of the sub-step before our read of it
        if (!ptx::mbar_wait(&pds_full[u], par, abort_flag, 63)) { alive = false; break; }
        last = dq_desc[2 * u] != 0;
        const int tile = dq_desc[2 * u + 1];
        if (!ptx::mbar_wait(&dq_full[u], par, abort_flag, 64)) { alive = false; break; }
        ptx::tc_fence_after();
        float* dst = p.dq_acc + static_cast<size_t>(tile) * (kSub * kHeadDim) + row * kSub;
        const bool row_used = row < p.head_dim;
        if (drain_rows) {
          uint32_t a[32];
          ptx::tmem_ld32(tmem + u * 128 + 64 + lane_addr, a);
          ptx::tmem_wait_ld();
          if (row_used) {
#pragma unroll
            for (int i = 0; i < 8; ++i) red_add_v4(dst + 4 * i, a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
          }
          ptx::tmem_ld32(tmem + u * 128 + 64 + lane_addr + 32, a);
          ptx::tmem_wait_ld();
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(&buf_free[u]);
          if (row_used) {
#pragma unroll
            for (int i = 0; i < 8; ++i) red_add_v4(dst + 32 + 4 * i, a[4 * i], a[4 * i + 1], a[4 * i + 2], a[4 * i + 3]);
          }
        } else {
          ptx::mbar_arrive_warp(&buf_free[u]);
        }
      }
      if (!alive) break;
      const int kj = it.k0 + row;
      const int rows_valid = imax(0, imin(32, it.n - (it.k0 + quad * 32)));  // of this warp's 32 key rows
      const int64_t srow = static_cast<int64_t>(it.row0) + it.kh * it.n + kj;
      uint16_t* dk_row = static_cast<uint16_t*>(p.dk) + it.bcoord * p.dk_bs + srow * p.dk_rs + it.hk * p.dk_hs;
      uint16_t* dv_row = static_cast<uint16_t*>(p.dv) + it.bcoord * p.dv_bs + srow * p.dv_rs + it.hk * p.dv_hs;
      if (!ptx::mbar_wait(acc_full, n_item & 1, abort_flag, 62)) break;
      ++n_item;
      ptx::tc_fence_after();
      constexpr int kChunks = 2 * kHeadDim / 32;   // dK and dV sit side by side in tensor memory
#pragma unroll 1
      for (int gidx = 0; gidx < kChunks; ++gidx) {
        const bool is_dv = gidx * 32 >= kHeadDim;
        const int col0 = gidx * 32 - (is_dv ? kHeadDim : 0);
        uint32_t accv[32];
        ptx::tmem_ld32(tmem + Cfg::kTmemDK + lane_addr + gidx * 32, accv);
        ptx::tmem_wait_ld();
        if (gidx == kChunks - 1) {
          // everything is in registers: the first dV / dK products of the next item may overwrite the accumulators
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(acc_free);
        }
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
        const KvItem it = decode_kv_item(p, idx);
        if (!it.valid) continue;
        const QueryPlan plan = make_query_plan(it.kh, it.k0, it.k1, it.n, bs, kTile);
        const KvSpans spans = make_kv_spans(it, bs);
        const int grow0 = p.cu_seqlens != nullptr ? it.row0 : it.b * p.seqlen;
        if (!ptx::mbar_wait(kv_empty, (n_item & 1) ^ 1, abort_flag, 41)) break;
        ptx::mbar_expect_tx(kv_full, 2 * T::kTileBytes);
        const int k_row = it.row0 + it.kh * it.n + it.k0;
        load_tile<kHeadDim>(sK, &p.tm_k, kv_full, k_row, it.hk, it.bcoord);
        load_tile<kHeadDim>(sV, &p.tm_v, kv_full, k_row, it.hk, it.bcoord);
        // The loader alone walks the item's geometry. Each stage carries a header for the other roles:
        // {bit 0 last sub-step of the item, bit 1 partially masked, bit 2 queries of the keys' own half; first row;
        // accumulator tile of the sub-step's dQ}. A sub-step is sent when its successor is known, so that the last
        // one can be marked.
        auto emit = [&](const SubStep& st, bool last) -> bool {
          const uint32_t stage = gc % kStages;
          if (!ptx::mbar_wait(&st_empty[stage], ((gc / kStages) & 1) ^ 1, abort_flag, 42)) return false;
          uint8_t* base = sStage + stage * Cfg::kStageBytes;
          volatile int* hdr = reinterpret_cast<volatile int*>(base + Cfg::kHeaderOffset);
          hdr[0] = (last ? 1 : 0) | (st.cls == kTileMasked ? 2 : 0) | (st.qh == it.kh ? 4 : 0);
          hdr[1] = st.sa;
          hdr[2] = st.h * p.acc_tiles + acc_tile_of(grow0, it.n, it.b, st.qh, st.sa);
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
        alive = for_each_substep(it, plan, spans, group, [&](const SubStep& st) -> bool {
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
    // Two threads issue the MMAs of this kernel, so that the barrier waits and commits of one overlap the MMAs of
    // the other. Sub-step g may overwrite buffer g & 1 once dV / dK of sub-step g - 2 have read P^T from it and
    // its dQ^T has been drained (buf_free).
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
        const KvItem it = decode_kv_item(p, idx);
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
        ++n_item;
      }
    }
  } else if (warp == kMmaWarpB + 1) {
    // -------------------------------------------------- MMA issuer 2: dQ^T = K^T dS^T, dV += P^T dO, dK += dS^T Q
    if (lane == 0) {
      constexpr int kFmt = kBf16 ? 1 : 0;
      const uint32_t idesc_g = ptx::make_idesc(kTile, kHeadDim, kFmt, false, true);   // A K-major, B MN-major
      const uint32_t idesc_q = ptx::make_idesc(kTile, kSub, kFmt, true, true);        // A and B MN-major
      constexpr uint32_t kHi = ptx::smem_desc_hi(1024);
      const uint32_t st_lo_mn = ptx::smem_desc_lo(ptx::smem_u32(sStage), Cfg::kSubPanelBytes);   // Q / dO, MN-major B
      const uint32_t kt_lo = ptx::smem_desc_lo(ptx::smem_u32(sK), T::kPanelBytes);   // K^T: the key rows are the reduction
      const uint32_t ds_lo = ptx::smem_desc_lo(ptx::smem_u32(sDs), 16);              // dS^T, one 64-query panel
      uint32_t g = 0, n_item_b = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_consume<false>(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const KvItem it = decode_kv_item(p, idx);
        if (!it.valid) continue;
        bool acc = false;
        // the first dV / dK products of an item overwrite the accumulators: the epilogue must have read the last item's
        if (!ptx::mbar_wait(acc_free, (n_item_b & 1u) ^ 1u, abort_flag, 57)) break;
        ++n_item_b;
        for (bool last = false; alive && !last; ++g) {
          const uint32_t u = g & 1u, stage = g % kStages;
          if (!ptx::mbar_wait(&st_full[stage], (g / kStages) & 1u, abort_flag, 55)) { alive = false; break; }
          last = (*reinterpret_cast<const volatile int*>(sStage + stage * Cfg::kStageBytes + Cfg::kHeaderOffset) & 1) != 0;
          if (!ptx::mbar_wait(&pds_full[u], (g >> 1) & 1u, abort_flag, 53)) { alive = false; break; }
          ptx::tc_fence_after();
          const uint32_t q_off = stage * (Cfg::kStageBytes >> 4);
          const uint32_t do_off = q_off + (Cfg::kSubTileBytes >> 4);
          const uint32_t st_t = tmem + u * 128, dq_t = tmem + u * 128 + 64;
          const uint32_t ds_u = ds_lo + u * (Cfg::kDsBytes >> 4);
          // dQ^T first: its drain (tensor memory -> registers -> global adds) then runs under dV / dK
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            ptx::umma_ss_f16_lh(dq_t, kt_lo + kk * (2048 >> 4), ds_u + kk * (2048 >> 4), kHi, idesc_q, kk > 0);
          }
          ptx::umma_commit(&dq_full[u]);
          // K is read by S^T (already complete for every sub-step of this item) and by dQ^T: after the last dQ^T
          // the next item's K and V may load
          if (last) ptx::umma_commit(kv_empty);
#pragma unroll
          for (int kk = 0; kk < kSub / 16; ++kk) {
            ptx::umma_ts_f16_lh(tmem + Cfg::kTmemDV, st_t + kk * kSubCols, st_lo_mn + do_off + kk * (2048 >> 4), kHi,
                                idesc_g, (acc || kk > 0) ? 1u : 0u);
            ptx::umma_ss_f16_lh(tmem + Cfg::kTmemDK, ds_u + kk * (32 >> 4), st_lo_mn + q_off + kk * (2048 >> 4), kHi,
                                idesc_g, (acc || kk > 0) ? 1u : 0u);
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
    // this thread's two 16-byte pieces of its dS^T row (128-byte swizzle: piece c of row r sits at c ^ (r & 7))
    const uint32_t ds_off0 = row * 128 + (((2 * wg) ^ (row & 7)) << 4);
    const uint32_t ds_off1 = row * 128 + (((2 * wg + 1) ^ (row & 7)) << 4);
    uint32_t gc = 0;
    bool alive = true;
    for (uint32_t n_sched = 0; alive; ++n_sched) {
      const int idx = sched_consume<true>(mbox, n_sched, abort_flag);
      if (idx < 0 || idx >= total_items) break;
      const KvItem it = decode_kv_item(p, idx);
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
        // the stage barrier orders the header and the bulk copies of lse2 / delta before our reads
        if (!ptx::mbar_wait(&st_full[stage], (gc / kStages) & 1u, abort_flag, 60)) { alive = false; break; }
        int hdr0, hdr1, hdr2;
        hdr0 = reinterpret_cast<const volatile int*>(stage_base + Cfg::kHeaderOffset)[0];
        hdr1 = reinterpret_cast<const volatile int*>(stage_base + Cfg::kHeaderOffset)[1];
        hdr2 = reinterpret_cast<const volatile int*>(stage_base + Cfg::kHeaderOffset)[2];
        last = (hdr0 & 1) != 0;
        // the per-column statistics of this warp's 16 query columns come into registers now, as 16-byte loads, while
        // the S^T / dP^T products are still running (scalar loads later would queue behind the MMAs' operand fetches)
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
        if (hdr0 & 2) {
          const int lo = ((hdr0 & 4) ? same_lo : cross_lo) - (hdr1 + wg * kSubCols);
          const int hi = ((hdr0 & 4) ? same_hi : cross_hi) - (hdr1 + wg * kSubCols);
          softmax_backward_cols<kSubCols, kBf16, kSoftcap, true, true, true>(sv, dpv, l2r, dlr, 0.f, 0.f, p.scale_log2,
                                                                              p.softcap_pre, lo, hi, pk_p, pk_ds);
        } else {
          softmax_backward_cols<kSubCols, kBf16, kSoftcap, true, false, true>(sv, dpv, l2r, dlr, 0.f, 0.f, p.scale_log2,
                                                                               p.softcap_pre, 0, 0, pk_p, pk_ds);
        }
        // P^T goes back to tensor memory, to the start of this warp's own (already loaded) S^T columns; dS^T goes to
        // shared memory, where it is the A operand of dK (keys x queries) and the B operand of dQ^T
        ptx::tmem_st8(st_t, pk_p);
        uint8_t* ds_tile = sDs + u * Cfg::kDsBytes;
        ptx::st_shared_v4(ds_tile + ds_off0, pk_ds[0], pk_ds[1], pk_ds[2], pk_ds[3]);
        ptx::st_shared_v4(ds_tile + ds_off1, pk_ds[4], pk_ds[5], pk_ds[6], pk_ds[7]);
        if (threadIdx.x == 0) {
          dq_desc[2 * u] = hdr0 & 1;
          dq_desc[2 * u + 1] = hdr2;
        }
        ptx::fence_async_smem();
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive_warp(&pds_full[u]);
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kLoadWarpB) ptx::tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------------------
// dQ = round(accumulator * softmax_scale), transposed back to rows of queries. One block per 64-row sub-tile of a
// (sample, head, half); stands where the reference converts its accumulator
// (csrc/fda/flash_bwd_postprocess_kernel.h:160-264 there).
// ------------------------------------------------------------------------------------------------------------
template <int kHeadDim, bool kBf16>
__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const __grid_constant__ BwdParams p) {
  __shared__ float tile[kHeadDim][kSub + 1];
  const int t = blockIdx.x;            // sub-tile of the half
  const int h = blockIdx.y >> 1, half = blockIdx.y & 1;
  const int b = blockIdx.z;
  const Sample sm = sample_of(p, b);
  const int sa = t * kSub;
  if (sa >= sm.n) return;
  const int grow0 = p.cu_seqlens != nullptr ? sm.row0 : b * p.seqlen;
  const float* src = p.dq_acc + (static_cast<size_t>(h) * p.acc_tiles + acc_tile_of(grow0, sm.n, b, half, sa)) *
                                    (kSub * kHeadDim);
  // accumulator tile: [head dim][64 queries]; 16 threads read one row of 64 floats
  for (int r = threadIdx.x / 16; r < kHeadDim; r += 16) {
    const float4 v = *reinterpret_cast<const float4*>(src + r * kSub + (threadIdx.x % 16) * 4);
    const int c = (threadIdx.x % 16) * 4;
    tile[r][c] = v.x; tile[r][c + 1] = v.y; tile[r][c + 2] = v.z; tile[r][c + 3] = v.w;
  }
  __syncthreads();
  // output: 64 query rows x head_dim values, 8 values (16 bytes) per thread and step
  constexpr int kPieces = kHeadDim / 8;
  for (int i = threadIdx.x; i < kSub * kPieces; i += 256) {
    const int qr = i / kPieces, piece = i % kPieces;
    if (sa + qr >= sm.n || piece * 8 >= p.head_dim) continue;
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      w[j] = ptx::pack2<kBf16>(tile[piece * 8 + 2 * j][qr] * p.softmax_scale,
                               tile[piece * 8 + 2 * j + 1][qr] * p.softmax_scale);
    }
    const int64_t srow = static_cast<int64_t>(sm.row0) + half * sm.n + sa + qr;
    uint16_t* dst = static_cast<uint16_t*>(p.dq) + sm.bcoord * p.dq_bs + srow * p.dq_rs + h * p.dq_hs + piece * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

template <int kHeadDim, int kStages, bool kBf16, bool kSoftcap>
int launch_fused_instance(const BwdParams& p, int sm_count, unsigned stages, cudaStream_t stream) {
  if (stages & 2u) {
    using Cfg = FusedCfg<kHeadDim, kStages>;
    auto kernel = bwd_fused_kernel<kHeadDim, kStages, kBf16, kSoftcap>;
    static PerDeviceFlags smem_set;
    const int rc = set_dynamic_smem(kernel, Cfg::kSmemBytes, smem_set);
    if (rc) return rc;
    FDA_CUDA_TRY(cudaMemsetAsync(p.dq_acc, 0, static_cast<size_t>(p.heads) * p.acc_tiles * kSub * kHeadDim * 4, stream));
    const int items = p.tiles_per_half * 2 * p.heads_k * p.batch;
    const int grid = items < sm_count ? items : sm_count;
    kernel<<<grid, kDkdvThreads, Cfg::kSmemBytes, stream>>>(p);
    FDA_CUDA_TRY(cudaGetLastError());
  }
  if (stages & 4u) {
    dim3 grid(p.n_pad / kSub, 2 * p.heads, p.batch);
    bwd_dq_convert_kernel<kHeadDim, kBf16><<<grid, 256, 0, stream>>>(p);
    FDA_CUDA_TRY(cudaGetLastError());
  }
  return FDA_OK;
}

}  // namespace

// Number of 64-row accumulator tiles per query head (see acc_tile_of): every half of every sample gets whole tiles.
int64_t bwd_fused_acc_tiles(const FdaProblem& pr) {
  return static_cast<int64_t>(pr.total) / kSub + 2 * static_cast<int64_t>(pr.batch) + 1;
}

size_t bwd_fused_acc_bytes(const FdaProblem& pr) {
  const int d_round = pr.head_dim <= 64 ? 64 : 128;
  return static_cast<size_t>(pr.heads) * bwd_fused_acc_tiles(pr) * kSub * d_round * 4;
}

// stages: bit 1 = accumulator zero-fill + fused kernel, bit 2 = dQ convert.
int launch_bwd_fused(const BwdParams& p, int d_round, bool bf16, bool softcap, int sm_count, unsigned stages,
                     cudaStream_t stream) {
  if (d_round == 64) {
    if (bf16) return softcap ? launch_fused_instance<64, 6, true, true>(p, sm_count, stages, stream)
                             : launch_fused_instance<64, 6, true, false>(p, sm_count, stages, stream);
    return softcap ? launch_fused_instance<64, 6, false, true>(p, sm_count, stages, stream)
                   : launch_fused_instance<64, 6, false, false>(p, sm_count, stages, stream);
  }
  if (bf16) return softcap ? launch_fused_instance<128, 3, true, true>(p, sm_count, stages, stream)
                           : launch_fused_instance<128, 3, true, false>(p, sm_count, stages, stream);
  return softcap ? launch_fused_instance<128, 3, false, true>(p, sm_count, stages, stream)
                 : launch_fused_instance<128, 3, false, false>(p, sm_count, stages, stream);
}

int read_status_bwd_fused(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}

}  // namespace fda
