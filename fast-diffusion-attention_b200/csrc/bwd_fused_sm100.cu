// Single-pass backward of block-diffusion attention for sm_100a: dK, dV and dQ from five GEMMs per tile pair.
//
// One CTA per (128-key tile, KV head, sample, half), persistent. K and V stay in shared memory; the visible
// 128-row query tiles of every query head of the group stream through. Per (key tile, query tile) step:
//   S^T  = K Q^T                        keys on tensor-memory lanes, 128 query columns
//   P^T  = exp2(S^T c - LSE2)           compute warps; written back over S^T as 16-bit (with a score cap: of
//                                       cap * tanh(S^T / cap), and the factor kept for dS^T is P^T (1 - tanh^2))
//   dP^T = V dO^T                       a second 128-column buffer
//   dS^T = P^T (dP^T - delta)           compute warps; to shared memory as 16-bit, [keys][queries]
//   dV  += P^T dO, dK += dS^T Q         accumulators in tensor memory for the whole key tile
//   dQ^T = K^T dS^T                     head dim on lanes, 128 query columns, written over the consumed dP^T buffer
//                                       (head dim 64 leaves room for columns of its own)
// The two halves of the arithmetic hang on different products, so they overlap different MMAs: P^T is computed while
// dP^T (and the tail of the previous step) runs, dS^T while dV runs. The partial dQ^T of a step is added into an fp32
// accumulator in global memory: the drain warps move it from tensor memory through a small shared-memory staging
// area and out as 4 KB bulk reductions (cp.reduce.async.bulk add.f32); `bwd_dq_convert_kernel` then scales and
// rounds the accumulator into dQ. About 30 bytes per clock leave an SM towards L2 whatever the instruction (plain
// red, vector red and bulk reductions measured alike), so the 64 KB of a step take about 2200 cycles: the drain is
// the long pole of the chain dP^T -> dS^T -> dQ^T -> drain -> next dP^T.
//
// The reference does the same five GEMMs per pair with an fp32 dQ accumulator reduced through global memory
// (csrc/fda/mainloop_bwd_sm90_tma_gmma_ws.hpp:815-984 `bwd_step`, :605-664 `store_dq`, there with
// cp.reduce.async.bulk from shared memory) and converts afterwards (flash_bwd_postprocess_kernel.h:160-264).
// The order of the adds depends on scheduling, so this path serves deterministic == 0 only; the deterministic
// backward keeps the two-kernel split (dK/dV kernel + dQ kernel), which has no cross-CTA reduction.
#include <type_traits>

#include "bwd_common.cuh"


namespace fda {
namespace {

template <int kHeadDim, int kSlots, int kDoSlots>
struct FusedCfg {
  using T = TileCfg<kHeadDim>;
  static constexpr int kDsPanelBytes = kTile * 128;          // [128 keys][64 queries] 16-bit
  static constexpr int kDsBytes = 2 * kDsPanelBytes;         // dS^T: two 64-query panels
  static constexpr int kStatBytes = 2 * kTile * 4;           // lse2[128], delta[128] of a query tile
  static constexpr int kOffQ = 2 * T::kTileBytes;            // K, V first (V directly behind K)
  static constexpr int kOffDo = kOffQ + kSlots * T::kTileBytes;
  static constexpr int kOffDs = kOffDo + kDoSlots * T::kTileBytes;
  static constexpr int kStageChunk = 32 * 32 * 4;            // one warp's 32 head-dim rows x 32 query columns of dQ^T
  static constexpr int kOffStage = kOffDs + kDsBytes;        // [4 warps][2 slots][kStageChunk]
  static constexpr int kOffStat = kOffStage + 4 * 2 * kStageChunk;
  static constexpr int kOffBar = kOffStat + kSlots * kStatBytes;
  static constexpr int kSmemBytes = kOffBar + 512;
  // tensor memory: S^T / P^T at 0, dP^T / dQ^T at 128, dK and dV behind
  static constexpr int kTmemS = 0, kTmemDP = 128, kTmemDK = 256, kTmemDV = 256 + kHeadDim;
  // Head dimension 64 leaves 128 columns behind the accumulators: dQ^T gets them, and the next dP^T no longer waits
  // for the drain of this step's dQ^T. At 128 all 512 columns are taken and dQ^T overwrites dP^T.
  static constexpr bool kOwnDq = 256 + 2 * kHeadDim + 128 <= 512;
  static constexpr int kTmemDQ = kOwnDq ? 256 + 2 * kHeadDim : kTmemDP;
  static_assert(kHeadDim == 64 || kHeadDim == 128, "the single-pass backward covers head dimensions up to 128");
  static_assert(kOffStat % 1024 == 0, "tiles stay 1024-byte aligned for the swizzle");
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  static_assert((12 + 2 * kSlots + 2 * kDoSlots) * 8 + 8 + 16 + 16 * kSlots <= 384, "barrier area");
};

// 768 threads start with 80 registers each. The compute warps hold a step's 32 probabilities per thread across the
// two halves of the arithmetic; the producer warpgroup and the drain / epilogue warpgroup get by with less.
constexpr uint32_t kFusedComputeRegs = 88, kFusedProducerRegs = 64, kFusedDrainRegs = 64;
static_assert(kCmpThreads * kFusedComputeRegs + 128 * kFusedProducerRegs + 128 * kFusedDrainRegs <= kDkdvThreads * 80,
              "register pool");

// Rows of the dQ accumulator come in blocks of 64. Every half of every sample starts at its own block: the
// "+ 2 b + qh" gives each of the 2 * batch halves one block of slack, so rounding the start down never lets two
// halves share a block. Returns the first accumulator row of query row `qa` (a multiple of 64) of half `qh` of a
// sample whose first row in the packed row space is `grow0`.
__device__ __forceinline__ int acc_row_of(int grow0, int n, int b, int qh, int qa) {
  return ((grow0 + qh * n) / 64 + 2 * b + qh) * 64 + qa;
}

// One step of an item: a visible 128-row query tile of one query head.
struct QStep {
  int h, qh, qa, cls;
};

template <typename Fn>
__device__ __forceinline__ bool for_each_qstep(const KvItem& it, const QueryPlan& plan, const KvSpans& spans, int group,
                                               Fn&& fn) {
  for (int g = 0; g < group; ++g) {
    for (int s = 0; s < plan.steps(); ++s) {
      QStep st;
      int qt;
      plan.step(s, it.kh, st.qh, qt);
      st.qa = qt * kTile;
      const int qb = imin(st.qa + kTile, it.n);
      st.cls = spans.classify(st.qh, it.kh, st.qa, qb);
      if (st.cls == kTileSkip) continue;
      st.h = it.hk * group + g;
      if (!fn(st)) return false;
    }
  }
  return true;
}

template <int kHeadDim, int kSlots, int kDoSlots, bool kBf16, bool kSoftcap>
__global__ void __launch_bounds__(kDkdvThreads, 1) bwd_fused_kernel(const __grid_constant__ BwdParams p) {
  using Cfg = FusedCfg<kHeadDim, kSlots, kDoSlots>;
  using T = TileCfg<kHeadDim>;
  // The tiles need 1024-byte alignment for the 128-byte swizzle. Dynamic shared memory starts at the beginning of the
  // block's window, which is aligned that far; the budget leaves no room to round the base up, so a base that is not
  // aligned is reported through the status word instead.
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* sK = smem;
  uint8_t* sV = smem + T::kTileBytes;   // directly behind K: for head dim 64 it is the second panel of the M = 128
                                        // operand of dQ^T (rows 64..127 of that product are never read)
  uint8_t* sQ = smem + Cfg::kOffQ;
  uint8_t* sDo = smem + Cfg::kOffDo;
  uint8_t* sDs = smem + Cfg::kOffDs;
  uint8_t* sStage = smem + Cfg::kOffStage;
  uint8_t* sStat = smem + Cfg::kOffStat;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kOffBar);
  uint64_t* kv_full = bars;
  uint64_t* kv_empty = bars + 1;
  uint64_t* q_full = bars + 2;                 // [kSlots] Q tile, its statistics and the step header
  uint64_t* q_empty = q_full + kSlots;
  uint64_t* do_full = q_empty + kSlots;        // [kDoSlots] dO tile
  uint64_t* do_empty = do_full + kDoSlots;
  uint64_t* s_full = do_empty + kDoSlots;      // S^T complete
  uint64_t* dp_full = s_full + 1;              // dP^T complete
  uint64_t* p_full = dp_full + 1;              // P^T written over S^T
  uint64_t* ds_full = p_full + 1;              // dS^T in shared memory, dP^T in registers
  uint64_t* s_free = ds_full + 1;              // dV has read P^T: the next S^T may overwrite it
  uint64_t* dq_full = s_free + 1;              // dQ^T complete
  uint64_t* dp_free = dq_full + 1;             // dQ^T is in the drain warps' registers: its columns may be overwritten
                                               // (by the next dP^T, or by the next dQ^T where it has columns of its own)
  uint64_t* ds_free = dp_free + 1;             // dQ^T and dK have read dS^T: the next step may overwrite it
  uint64_t* acc_full = ds_free + 1;
  uint64_t* acc_free = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* dq_desc = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [2][2]: {flags, first accumulator row}
  volatile int* hdr = reinterpret_cast<volatile int*>(tmem_slot + 6);       // [kSlots][4]
  SchedMailbox* mbox = reinterpret_cast<SchedMailbox*>(reinterpret_cast<uint8_t*>(bars) + 384);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if ((ptx::smem_u32(smem) & 1023u) != 0) {
    if (threadIdx.x == 0 && atomicCAS(&g_fda_status[0], 0, 120) == 0) {
      g_fda_status[1] = static_cast<int>(blockIdx.x);
      g_fda_status[2] = 0;
      g_fda_status[3] = static_cast<int>(ptx::smem_u32(smem) & 1023u);
    }
    return;
  }
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    sched_init(mbox, 4 * kCmpWG + 2 + 4);   // compute warps, two MMA issuers, four drain / epilogue warps
    ptx::mbar_init(kv_full, 1);
    ptx::mbar_init(kv_empty, 1);
    for (int i = 0; i < kSlots; ++i) {
      ptx::mbar_init(&q_full[i], 1);
      ptx::mbar_init(&q_empty[i], 1);
    }
    for (int i = 0; i < kDoSlots; ++i) {
      ptx::mbar_init(&do_full[i], 1);
      ptx::mbar_init(&do_empty[i], 2);   // dP^T (issuer 1) and dV (issuer 2) have both read the tile
    }
    ptx::mbar_init(s_full, 1);
    ptx::mbar_init(dp_full, 1);
    ptx::mbar_init(p_full, 4 * kCmpWG);
    ptx::mbar_init(ds_full, 4 * kCmpWG);
    ptx::mbar_init(s_free, 1);
    ptx::mbar_init(dq_full, 1);
    ptx::mbar_init(dp_free, 4);
    ptx::mbar_init(ds_free, 1);
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
  const int total_items = kv_item_count(p);

  if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------------------------------- dQ drain + dK/dV epilogue
    // Four warps, one per quarter of the tensor-memory lanes. Per step they add the partial dQ^T (lane = head-dim
    // row, 128 query columns) into the global accumulator; after the last step of an item they write dK and dV.
    ptx::reg_release_to<kFusedDrainRegs>();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const bool drain_rows = quad * 32 < kHeadDim;   // head dim 64: the upper two quarters hold nothing of dQ^T
    uint32_t n_item = 0, gd = 0, n_bulk = 0;
    bool alive = true;
    for (uint32_t n_sched = 0; alive; ++n_sched) {
      const int idx = sched_consume<true>(mbox, n_sched, abort_flag);
      if (idx < 0 || idx >= total_items) break;
      const KvItem it = decode_kv_item(p, idx);
      if (!it.valid) continue;
      for (bool last = false; alive && !last; ++gd) {
        const uint32_t par = gd & 1u;
        // the compute warps' barrier orders their description of the step before our read of it
        if (!ptx::mbar_wait(ds_full, par, abort_flag, 63)) { alive = false; break; }
        const int flags = dq_desc[2 * par];
        const int acc_row = dq_desc[2 * par + 1];
        last = (flags & 1) != 0;
        const int rows_left = flags >> 8;   // query rows of this tile that exist (1..128)
        if (!ptx::mbar_wait(dq_full, par, abort_flag, 64)) { alive = false; break; }
        ptx::tc_fence_after();
        // Blocks of 32 query rows of the accumulator are stored as [head dim / 32][32 queries][32 head-dim values]: a
        // warp's 32 x 32 piece of dQ^T goes through shared memory (a thread writes its head-dim value of each query,
        // 32 lanes = 128 consecutive bytes) and out as ONE 4 KB bulk reduction, issued by lane 0. Two staging slots per
        // warp alternate, so tensor memory is read out at shared-memory speed and the adds drain in the background.
        float* dst = p.dq_acc + static_cast<size_t>(acc_row) * kHeadDim + quad * 1024;
        if (drain_rows) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t a[32];
            ptx::tmem_ld32(tmem + Cfg::kTmemDQ + lane_addr + c * 32, a);
            float* stage = reinterpret_cast<float*>(sStage + (quad * 2 + (n_bulk & 1u)) * Cfg::kStageChunk);
            // the bulk reduction that last read this slot (two chunks ago) must have finished reading it
            if (lane == 0) ptx::bulk_wait_group_read<1>();
            __syncwarp();
            ptx::tmem_wait_ld();
            if (c == 3) {
              ptx::tc_fence_before();
              ptx::mbar_arrive_warp(dp_free);
            }
            if (c * 32 < rows_left) {
#pragma unroll
              for (int i = 0; i < 32; ++i) stage[i * 32 + lane] = __uint_as_float(a[i]);
              ptx::fence_async_smem();
              __syncwarp();
              if (lane == 0) {
                float* target = dst + c * (32 * kHeadDim);
                if (target >= p.dq_acc && target + 1024 <= p.dq_acc + p.acc_floats) {
                  ptx::bulk_reduce_add_f32(target, stage, Cfg::kStageChunk);
                  ptx::bulk_commit_group();
                } else if (atomicCAS(&g_fda_status[0], 0, 121) == 0) {   // never expected: recorded, not performed
                  g_fda_status[1] = static_cast<int>(blockIdx.x);
                  g_fda_status[2] = acc_row;
                  g_fda_status[3] = flags;
                }
              }
              ++n_bulk;
            }
          }
        } else {
          ptx::mbar_arrive_warp(dp_free);
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
    if (lane == 0) ptx::bulk_wait_group0();   // every reduction this warp issued has been performed
  } else if (warp >= 4 * kCmpWG) {
  ptx::reg_release_to<kFusedProducerRegs>();
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
        // The loader alone walks the item's geometry. Each step carries a header for the other roles:
        // {bit 0 last step of the item, bit 1 partially masked, bit 2 queries of the keys' own half, bits 8.. the
        // number of query rows that exist; first query row; first accumulator row of the step's dQ}. A step is sent
        // when its successor is known, so that the last one can be marked.
        auto emit = [&](const QStep& st, bool last) -> bool {
          const uint32_t slot = gc % kSlots, par = ((gc / kSlots) & 1u) ^ 1u;
          if (!ptx::mbar_wait(&q_empty[slot], par, abort_flag, 42)) return false;
          volatile int* h4 = hdr + 4 * slot;
          h4[0] = (last ? 1 : 0) | (st.cls == kTileMasked ? 2 : 0) | (st.qh == it.kh ? 4 : 0) |
                  (imin(kTile, it.n - st.qa) << 8);
          h4[1] = st.qa;
          h4[2] = st.h * p.acc_tiles * 64 + acc_row_of(grow0, it.n, it.b, st.qh, st.qa);
          ptx::mbar_expect_tx(&q_full[slot], T::kTileBytes + Cfg::kStatBytes);
          const int q_row = it.row0 + st.qh * it.n + st.qa;
          load_tile<kHeadDim>(sQ + slot * T::kTileBytes, &p.tm_q, &q_full[slot], q_row, st.h, it.bcoord);
          const int64_t seg = stat_segment(p, it.b, st.h, st.qh) + st.qa;
          ptx::bulk_load_1d(sStat + slot * Cfg::kStatBytes, p.lse2_pad + seg, kTile * 4, &q_full[slot]);
          ptx::bulk_load_1d(sStat + slot * Cfg::kStatBytes + kTile * 4, p.delta_pad + seg, kTile * 4, &q_full[slot]);
          const uint32_t dslot = gc % kDoSlots, dpar = ((gc / kDoSlots) & 1u) ^ 1u;
          if (!ptx::mbar_wait(&do_empty[dslot], dpar, abort_flag, 43)) return false;
          ptx::mbar_expect_tx(&do_full[dslot], T::kTileBytes);
          load_tile<kHeadDim>(sDo + dslot * T::kTileBytes, &p.tm_do, &do_full[dslot], q_row, st.h, it.bcoord);
          ++gc;
          return true;
        };
        QStep pend{};
        bool have = false;
        alive = for_each_qstep(it, plan, spans, group, [&](const QStep& st) -> bool {
          if (have && !emit(pend, false)) return false;
          pend = st;
          have = true;
          return true;
        });
        // every valid key tile is seen at least by the queries of its own rows, so there is a last step
        if (alive && have) alive = emit(pend, true);
        ++n_item;
      }
      if (*abort_flag) __nanosleep(100000);
    }
  } else if (warp == kMmaWarpB) {
    // ------------------------------------------------------------------- MMA issuer 1: S^T = K Q^T, dP^T = V dO^T
    // Two threads issue the MMAs of this kernel, so that the barrier waits and commits of one overlap the MMAs of
    // the other. S^T of step g + 1 may overwrite P^T of step g once dV has read it (s_free); dP^T of step g + 1
    // may overwrite dQ^T of step g once the drain warps hold it (dp_free) or, where dQ^T has its own columns, dP^T of
    // step g once the compute warps hold it (ds_full).
    if (lane == 0) {
      constexpr int kFmt = kBf16 ? 1 : 0;
      const uint32_t idesc_s = ptx::make_idesc(kTile, kTile, kFmt, false, false);
      constexpr uint32_t kHi = ptx::smem_desc_hi(1024);
      const uint32_t k_lo = ptx::smem_desc_lo(ptx::smem_u32(sK), 16);
      const uint32_t v_lo = ptx::smem_desc_lo(ptx::smem_u32(sV), 16);
      const uint32_t q_lo = ptx::smem_desc_lo(ptx::smem_u32(sQ), 16);
      const uint32_t do_lo = ptx::smem_desc_lo(ptx::smem_u32(sDo), 16);
      uint32_t n_item = 0, g = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_consume<false>(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const KvItem it = decode_kv_item(p, idx);
        if (!it.valid) continue;
        if (!ptx::mbar_wait(kv_full, n_item & 1, abort_flag, 51)) break;
        for (bool last = false; alive && !last; ++g) {
          const uint32_t slot = g % kSlots, spar = (g / kSlots) & 1u;
          const uint32_t t_off = slot * (T::kTileBytes >> 4);
          if (!ptx::mbar_wait(&q_full[slot], spar, abort_flag, 52)) { alive = false; break; }
          last = (hdr[4 * slot] & 1) != 0;
          if (!ptx::mbar_wait(s_free, (g & 1u) ^ 1u, abort_flag, 54)) { alive = false; break; }
          ptx::tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk) {
            const uint32_t off = ((kk / 4) * T::kPanelBytes + (kk % 4) * 32) >> 4;
            ptx::umma_ss_f16_lh(tmem + Cfg::kTmemS, k_lo + off, q_lo + t_off + off, kHi, idesc_s, kk > 0);
          }
          ptx::umma_commit(s_full);
          const uint32_t dslot = g % kDoSlots;
          if (!ptx::mbar_wait(&do_full[dslot], (g / kDoSlots) & 1u, abort_flag, 56)) { alive = false; break; }
          if (!ptx::mbar_wait(Cfg::kOwnDq ? ds_full : dp_free, (g & 1u) ^ 1u, abort_flag, 58)) { alive = false; break; }
          ptx::tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk) {
            const uint32_t off = ((kk / 4) * T::kPanelBytes + (kk % 4) * 32) >> 4;
            ptx::umma_ss_f16_lh(tmem + Cfg::kTmemDP, v_lo + off, do_lo + dslot * (T::kTileBytes >> 4) + off, kHi, idesc_s,
                                kk > 0);
          }
          ptx::umma_commit(dp_full);
          ptx::umma_commit(&do_empty[dslot]);
        }
        ++n_item;
      }
    }
  } else if (warp == kMmaWarpB + 1) {
    // -------------------------------------------------- MMA issuer 2: dV += P^T dO, dQ^T = K^T dS^T, dK += dS^T Q
    if (lane == 0) {
      constexpr int kFmt = kBf16 ? 1 : 0;
      const uint32_t idesc_g = ptx::make_idesc(kTile, kHeadDim, kFmt, false, true);   // A K-major, B MN-major
      const uint32_t idesc_q = ptx::make_idesc(kTile, kTile, kFmt, true, true);       // A and B MN-major
      constexpr uint32_t kHi = ptx::smem_desc_hi(1024);
      const uint32_t q_mn = ptx::smem_desc_lo(ptx::smem_u32(sQ), T::kPanelBytes);     // Q / dO as MN-major B: rows of
      const uint32_t do_mn = ptx::smem_desc_lo(ptx::smem_u32(sDo), T::kPanelBytes);   // queries are the reduction
      const uint32_t kt_lo = ptx::smem_desc_lo(ptx::smem_u32(sK), T::kPanelBytes);    // K^T: key rows are the reduction
      const uint32_t ds_mn = ptx::smem_desc_lo(ptx::smem_u32(sDs), Cfg::kDsPanelBytes);   // dS^T as B of dQ^T
      const uint32_t ds_k = ptx::smem_desc_lo(ptx::smem_u32(sDs), 16);                // dS^T as K-major A of dK
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
          const uint32_t slot = g % kSlots, spar = (g / kSlots) & 1u;
          const uint32_t t_off = slot * (T::kTileBytes >> 4);
          if (!ptx::mbar_wait(&q_full[slot], spar, abort_flag, 55)) { alive = false; break; }
          last = (hdr[4 * slot] & 1) != 0;
          if (!ptx::mbar_wait(p_full, g & 1u, abort_flag, 53)) { alive = false; break; }
          // dO usually landed long ago (dP^T of this step reads it too), but nothing this thread has waited for so far
          // says so
          if (!ptx::mbar_wait(&do_full[g % kDoSlots], (g / kDoSlots) & 1u, abort_flag, 67)) { alive = false; break; }
          ptx::tc_fence_after();
          // dV += P^T dO: P^T of the 16 queries of reduction step kk sits at column 32 (kk / 2) + 8 (kk % 2)
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            ptx::umma_ts_f16_lh(tmem + Cfg::kTmemDV, tmem + Cfg::kTmemS + 32 * (kk / 2) + 8 * (kk % 2),
                                do_mn + (g % kDoSlots) * (T::kTileBytes >> 4) + kk * (2048 >> 4), kHi, idesc_g,
                                (acc || kk > 0) ? 1u : 0u);
          }
          ptx::umma_commit(s_free);
          ptx::umma_commit(&do_empty[g % kDoSlots]);
          if (!ptx::mbar_wait(ds_full, g & 1u, abort_flag, 59)) { alive = false; break; }
          ptx::tc_fence_after();
          // dQ^T before dK: its drain (tensor memory -> registers -> global adds) then runs under dK
          if (Cfg::kOwnDq) {
            // the drain warps hold dQ^T of the previous step
            if (!ptx::mbar_wait(dp_free, (g & 1u) ^ 1u, abort_flag, 68)) { alive = false; break; }
            ptx::tc_fence_after();
          }
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            ptx::umma_ss_f16_lh(tmem + Cfg::kTmemDQ, kt_lo + kk * (2048 >> 4), ds_mn + kk * (2048 >> 4), kHi, idesc_q, kk > 0);
          }
          ptx::umma_commit(dq_full);
          // K is read by S^T (complete for every step of this item by now) and by dQ^T: after the last dQ^T the next
          // item's K and V may load
          if (last) ptx::umma_commit(kv_empty);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk) {
            ptx::umma_ss_f16_lh(tmem + Cfg::kTmemDK, ds_k + (((kk / 4) * Cfg::kDsPanelBytes + (kk % 4) * 32) >> 4),
                                q_mn + t_off + kk * (2048 >> 4), kHi, idesc_g, (acc || kk > 0) ? 1u : 0u);
          }
          acc = true;
          ptx::umma_commit(&q_empty[slot]);
          ptx::umma_commit(ds_free);
        }
        if (!alive) break;
        ptx::umma_commit(acc_full);
      }
    }
  }
  } else {
    ptx::reg_acquire_to<kFusedComputeRegs>();
    // -------------------------------------------------------------------------------------- softmax backward
    const int wg = warp >> 2;                  // which 32 query columns of the step
    const int quad = warp & 3;
    const int row = quad * 32 + lane;          // key row inside the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t s_t = tmem + Cfg::kTmemS + lane_addr + wg * kCols;
    const uint32_t dp_t = tmem + Cfg::kTmemDP + lane_addr + wg * kCols;
    // this thread's row of the dS^T panel that holds its 32 queries: four 16-byte pieces starting at piece 4 (wg & 1)
    // (128-byte swizzle: piece c of row r sits at c ^ (r & 7))
    uint8_t* ds_row = sDs + (wg >> 1) * Cfg::kDsPanelBytes + row * 128;
    const int ds_piece0 = 4 * (wg & 1);
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
      for (bool last = false; alive && !last; ++gc) {
        const uint32_t slot = gc % kSlots, par = gc & 1u;
        const float* stats = reinterpret_cast<const float*>(sStat + slot * Cfg::kStatBytes) + wg * kCols;
        // the Q barrier orders the header and the bulk copies of lse2 / delta before our reads
        if (!ptx::mbar_wait(&q_full[slot], (gc / kSlots) & 1u, abort_flag, 60)) { alive = false; break; }
        const int hdr0 = hdr[4 * slot], hdr1 = hdr[4 * slot + 1], hdr2 = hdr[4 * slot + 2];
        last = (hdr0 & 1) != 0;
        const bool masked = (hdr0 & 2) != 0;
        // visible query columns of this thread's key, relative to its first column of the step
        const int lo = ((hdr0 & 4) ? same_lo : cross_lo) - (hdr1 + wg * kCols);
        const int hi = ((hdr0 & 4) ? same_hi : cross_hi) - (hdr1 + wg * kCols);
        {
          // First half, once S^T is complete: P^T (16-bit, back to tensor memory for dV) and, kept in registers, the
          // factor of the second half: P, or with the score cap P (1 - tanh^2).
          float pr[kCols];
          if (!ptx::mbar_wait(s_full, par, abort_flag, 61)) { alive = false; break; }
          ptx::tc_fence_after();
          {
            uint32_t sv[kCols], pk[kCols / 2];
            ptx::tmem_ld16(s_t, sv);
            ptx::tmem_ld16(s_t + 16, sv + 16);
            ptx::tmem_wait_ld();
            const float4* l2v = reinterpret_cast<const float4*>(stats);
            // the fully visible tile (the common one) carries no per-element compare
            auto first_half = [&](auto masked_tag) {
              constexpr bool kMasked = decltype(masked_tag)::value;
#pragma unroll
              for (int i = 0; i < kCols / 4; ++i) {
                const float4 l2 = l2v[i];
                const float l2a[4] = {l2.x, l2.y, l2.z, l2.w};
                float pv[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int c = 4 * i + j;
                  float x = __uint_as_float(sv[c]);
                  float dt = 1.f;
                  if (kSoftcap) {
                    x = ptx::tanh_fast(x * p.softcap_pre);
                    dt = 1.f - x * x;
                  }
                  float v = ptx::ex2(fmaf(x, p.scale_log2, -l2a[j]));
                  if (kMasked && (c < lo || c >= hi)) v = 0.f;
                  pv[j] = v;
                  pr[c] = kSoftcap ? v * dt : v;
                }
                pk[2 * i] = ptx::pack2<kBf16>(pv[0], pv[1]);
                pk[2 * i + 1] = ptx::pack2<kBf16>(pv[2], pv[3]);
              }
            };
            if (masked) first_half(std::true_type{});
            else first_half(std::false_type{});
            // a warp overwrites only columns it has itself already loaded: the 16-bit P^T of its 32 queries goes to
            // the first 16 of its own 32 columns
            ptx::tmem_st16(s_t, pk);
          }
          ptx::tmem_wait_st();
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(p_full);
          if (!ptx::mbar_wait(dp_full, par, abort_flag, 65)) { alive = false; break; }
          // dQ^T and dK of the previous step have read the dS^T tile (long ago in the steady state)
          if (!ptx::mbar_wait(ds_free, par ^ 1u, abort_flag, 66)) { alive = false; break; }
          ptx::tc_fence_after();
          {
            uint32_t dpv[kCols];
            ptx::tmem_ld16(dp_t, dpv);
            ptx::tmem_ld16(dp_t + 16, dpv + 16);
            ptx::tmem_wait_ld();
            const float4* dlv = reinterpret_cast<const float4*>(stats + kTile);
            // masked positions have P = 0, so dS = 0 there without another compare
#pragma unroll
            for (int i = 0; i < kCols / 8; ++i) {
              const float4 d0 = dlv[2 * i], d1 = dlv[2 * i + 1];
              const float dl[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
              uint32_t pk[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int c = 8 * i + 2 * j;
                pk[j] = ptx::pack2<kBf16>(pr[c] * (__uint_as_float(dpv[c]) - dl[2 * j]),
                                          pr[c + 1] * (__uint_as_float(dpv[c + 1]) - dl[2 * j + 1]));
              }
              ptx::st_shared_v4(ds_row + (((ds_piece0 + i) ^ (row & 7)) << 4), pk[0], pk[1], pk[2], pk[3]);
            }
          }
        }
        if (threadIdx.x == 0) {
          dq_desc[2 * par] = hdr0 & ~6;
          dq_desc[2 * par + 1] = hdr2;
        }
        ptx::fence_async_smem();
        ptx::tc_fence_before();
        ptx::mbar_arrive_warp(ds_full);
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == kLoadWarpB) ptx::tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------------------------
// dQ = round(accumulator * softmax_scale). One block per 64 query rows of a (sample, head, half); stands where the
// reference converts its accumulator (csrc/fda/flash_bwd_postprocess_kernel.h:160-264 there).
// ------------------------------------------------------------------------------------------------------------
template <int kHeadDim, bool kBf16>
__global__ void __launch_bounds__(256) bwd_dq_convert_kernel(const __grid_constant__ BwdParams p) {
  const int h = blockIdx.y >> 1, half = blockIdx.y & 1;
  const int b = blockIdx.z;
  const Sample sm = sample_of(p, b);
  const int qa = blockIdx.x * 64;
  if (qa >= sm.n) return;
  const int grow0 = p.cu_seqlens != nullptr ? sm.row0 : b * p.seqlen;
  const float* src =
      p.dq_acc + (static_cast<size_t>(h) * p.acc_tiles * 64 + acc_row_of(grow0, sm.n, b, half, qa)) * kHeadDim;
  // a thread turns 8 consecutive values of a row into one 16-byte store
  constexpr int kPieces = kHeadDim / 8;
#pragma unroll
  for (int i = threadIdx.x; i < 64 * kPieces; i += 256) {
    const int qr = i / kPieces, piece = i % kPieces;
    if (qa + qr >= sm.n || piece * 8 >= p.head_dim) continue;
    // blocks of 32 rows are stored [head dim / 32][32 rows][32 values]
    const float* s8 = src + (qr / 32) * (32 * kHeadDim) + (piece / 4) * 1024 + (qr % 32) * 32 + (piece % 4) * 8;
    const float4 lo = *reinterpret_cast<const float4*>(s8);
    const float4 hi = *reinterpret_cast<const float4*>(s8 + 4);
    const float sc = p.softmax_scale;
    const int64_t srow = static_cast<int64_t>(sm.row0) + half * sm.n + qa + qr;
    uint16_t* dst = static_cast<uint16_t*>(p.dq) + sm.bcoord * p.dq_bs + srow * p.dq_rs + h * p.dq_hs + piece * 8;
    *reinterpret_cast<uint4*>(dst) = make_uint4(ptx::pack2<kBf16>(lo.x * sc, lo.y * sc), ptx::pack2<kBf16>(lo.z * sc, lo.w * sc),
                                                ptx::pack2<kBf16>(hi.x * sc, hi.y * sc), ptx::pack2<kBf16>(hi.z * sc, hi.w * sc));
  }
}

template <int kHeadDim, int kSlots, int kDoSlots, bool kBf16, bool kSoftcap>
int launch_fused_instance(const BwdParams& p, int sm_count, unsigned stages, cudaStream_t stream) {
  if (stages & 2u) {
    using Cfg = FusedCfg<kHeadDim, kSlots, kDoSlots>;
    auto kernel = bwd_fused_kernel<kHeadDim, kSlots, kDoSlots, kBf16, kSoftcap>;
    static PerDeviceFlags smem_set;
    const int rc = set_dynamic_smem(kernel, Cfg::kSmemBytes, smem_set);
    if (rc) return rc;
    FDA_CUDA_TRY(cudaMemsetAsync(p.dq_acc, 0, static_cast<size_t>(p.heads) * p.acc_tiles * 64 * kHeadDim * 4, stream));
    const int items = bwd_item_bound(p, p.heads_k);
    const int grid = items < sm_count ? items : sm_count;
    kernel<<<grid, kDkdvThreads, Cfg::kSmemBytes, stream>>>(p);
    FDA_CUDA_TRY(cudaGetLastError());
  }
  if (stages & 4u) {
    dim3 grid(p.n_pad / 64, 2 * p.heads, p.batch);
    bwd_dq_convert_kernel<kHeadDim, kBf16><<<grid, 256, 0, stream>>>(p);
    FDA_CUDA_TRY(cudaGetLastError());
  }
  return FDA_OK;
}

}  // namespace

// Number of 64-row blocks of the dQ accumulator per query head (see acc_row_of): every half of every sample starts at
// its own block, and the last 128-row step of a half may reach one block past the half's rows.
int64_t bwd_fused_acc_tiles(const FdaProblem& pr) {
  return static_cast<int64_t>(pr.total) / 64 + 2 * static_cast<int64_t>(pr.batch) + 3;
}

size_t bwd_fused_acc_bytes(const FdaProblem& pr) {
  const int d_round = pr.head_dim <= 64 ? 64 : 128;
  return static_cast<size_t>(pr.heads) * bwd_fused_acc_tiles(pr) * 64 * d_round * 4;
}

// stages: bit 1 = accumulator zero-fill + single-pass kernel, bit 2 = dQ convert.
int launch_bwd_fused(const BwdParams& p, int d_round, bool bf16, bool softcap, int sm_count, unsigned stages,
                     cudaStream_t stream) {
  if (d_round == 64) {
    if (bf16) return softcap ? launch_fused_instance<64, 3, 3, true, true>(p, sm_count, stages, stream)
                             : launch_fused_instance<64, 3, 3, true, false>(p, sm_count, stages, stream);
    return softcap ? launch_fused_instance<64, 3, 3, false, true>(p, sm_count, stages, stream)
                   : launch_fused_instance<64, 3, 3, false, false>(p, sm_count, stages, stream);
  }
  if (bf16) return softcap ? launch_fused_instance<128, 2, 1, true, true>(p, sm_count, stages, stream)
                           : launch_fused_instance<128, 2, 1, true, false>(p, sm_count, stages, stream);
  return softcap ? launch_fused_instance<128, 2, 1, false, true>(p, sm_count, stages, stream)
                 : launch_fused_instance<128, 2, 1, false, false>(p, sm_count, stages, stream);
}

int read_status_bwd_fused(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}

}  // namespace fda
