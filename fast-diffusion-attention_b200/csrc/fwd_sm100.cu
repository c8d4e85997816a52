// Forward pass of block-diffusion attention for sm_100a.
//
// Replaces the reference's forward stack (csrc/fda/flash_fwd_kernel_sm90.h:165-325,
// csrc/fda/mainloop_fwd_sm90_tma_gmma_ws.hpp:334-880, csrc/fda/epilogue_fwd.hpp:126-272,
// csrc/fda/softmax.h:92-168 and the forward scheduler csrc/fda/tile_scheduler.hpp:51-185) with a design
// built around tcgen05:
//
//   * a work item is kQTiles consecutive 128-row query tiles of one half of one (sample, head); both tiles
//     walk ONE list of 128-key tiles (clean prefix, then the noisy diagonal), so a K/V tile fetched once by TMA
//     feeds both; a tile that one of the query tiles cannot see is skipped for that query tile only;
//   * warp roles: kQTiles softmax warpgroups (thread = one query row), one TMA producer warp, one MMA warp;
//   * S = Q K^T and O += P V are tcgen05.mma with fp32 accumulators in tensor memory; P is written back over
//     S as 16-bit and consumed from tensor memory as the A operand; V is used MN-major straight from its TMA
//     layout;
//   * online softmax with the scale folded into one FMA + exp2, a running row maximum that is only advanced
//     when it grows by more than 2^8 (O is rescaled in tensor memory only then), LSE in natural-log units;
//   * only visible tiles are enumerated, only tiles crossing a block boundary (or the end of a half) get the
//     element mask;
//   * persistent CTAs; items are ordered longest first (query tiles near the end of a half see most keys).
//
// Numerics contract kept from the reference: fp32 accumulation, softcap applied before the mask
// (mainloop_fwd...hpp:679-683), P rounded to the input dtype before P V (:782), row sums accumulated in fp32
// from the unrounded P, LSE = max * scale + ln(sum) (softmax.h:137-154).
#include "geometry.h"
#include "host_util.h"
#include "ptx.cuh"
#include "sched.cuh"
#include "varlen_list.cuh"


#ifndef FDA_SHORT8_FWD
#define FDA_SHORT8_FWD 2   // eighths of a (sample, head)'s items that count as short
#endif

namespace fda {
namespace {


constexpr int kBlockM = 128;  // query rows per tile (= tensor-memory lanes)
constexpr int kBlockN = 128;  // keys per tile
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;  // in log2 units

struct FwdParams {
  CUtensorMap tm_q, tm_k, tm_v;
  CUtensorMap tm_o;    // out, boxes of 64 columns x 32 rows (used when o_tma != 0)
  int o_tma;           // out's strides allow tile stores
  void* out;
  float* lse;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  const int32_t* cu_seqlens;
  int batch, seqlen, total, heads, heads_k, head_dim, block_size;
  int items_per_half;  // ceil(max n / rows per item)
  int n_long;          // of the 2 * items_per_half items of a (sample, head): how many count as long
  int total_items;     // batched layout; packed batches read the count from the work list
  VarlenList vl;       // packed batches: samples longest first with running item counts (base == nullptr otherwise)
  int* ticket;         // global work counter, zeroed before the launch
  int wide_store;      // rows of out allow 32-byte stores
  const float* q_descale;  // FP8 only: (batch, heads_k) factors, element strides below; nullptr = 1
  const float* k_descale;
  const float* v_descale;
  int64_t descale_bs[3], descale_hs[3];
  float scale_log2;    // exponent scale: softmax_scale*log2(e), or softcap*log2(e) with softcapping
  float softcap_pre;   // softmax_scale / softcap (tanh argument scale)
  float lse_scale;     // natural-log scale of the row maximum: softmax_scale, or softcap
};

struct Item {
  int b, h, hk, qh, qa, qb, n;
  int row0;    // tensor row of the first token of the sample
  int bcoord;  // batch coordinate for TMA (0 when packed)
  bool valid;
};

template <int kQTiles>
__device__ __forceinline__ Item decode_item(const FwdParams& p, int idx) {
  // (sample, head)-major so that the CTAs running at the same time share the K/V of a few heads in L2; inside a
  // head the items with the most key tiles (late query rows) come first.
  Item it;
  int rem, items_per_half;
  if (p.vl.base != nullptr) {
    // packed batch: the work list holds exactly the items that exist, longest sample first; inside a sample the
    // heads follow each other, inside a head the items with the most key tiles come first
    const VarlenPos pos = varlen_locate(p.vl, idx, 2 * p.heads);
    items_per_half = pos.units;
    it.b = pos.b;
    it.h = pos.rem / (2 * pos.units);
    rem = pos.rem - it.h * (2 * pos.units);
  } else {
    const int per_bh = 2 * p.items_per_half;
    int bh;
    two_phase_order(idx, per_bh, p.n_long, p.batch * p.heads, bh, rem);
    items_per_half = p.items_per_half;
    it.b = bh / p.heads;
    it.h = bh - it.b * p.heads;
  }
  it.qh = rem & 1;
  const int p_rev = rem >> 1;
  it.hk = it.h / (p.heads / p.heads_k);
  const int pidx = items_per_half - 1 - p_rev;
  if (p.cu_seqlens != nullptr) {
    const int s = p.cu_seqlens[it.b];
    const int e = p.cu_seqlens[it.b + 1];
    it.n = (e - s) / 2;
    it.row0 = s;
    it.bcoord = 0;
  } else {
    it.n = p.seqlen / 2;
    it.row0 = 0;
    it.bcoord = it.b;
  }
  it.qa = pidx * kQTiles * kBlockM;
  it.valid = it.qa < it.n;
  it.qb = imin(it.qa + kQTiles * kBlockM, it.n);
  return it;
}

// Key spans of query tile t of the item, one per key half (index 0 noisy, 1 clean). Built once per item (the
// divisions by the block size happen here); classifying a key tile afterwards is a few compares. A query tile
// without rows gets empty spans, so every key tile is "skip" for it.
struct TileSpans {
  Span half[2];
  // selects instead of half[kh]: a run-time index would put the spans in local memory
  __device__ __forceinline__ int classify(int kh, int kt) const {
    Span s;
    s.lo_first = kh ? half[1].lo_first : half[0].lo_first;
    s.hi_first = kh ? half[1].hi_first : half[0].hi_first;
    s.lo_last = kh ? half[1].lo_last : half[0].lo_last;
    s.hi_last = kh ? half[1].hi_last : half[0].hi_last;
    return s.classify(kt * kBlockN, kBlockN);
  }
};

__device__ __forceinline__ TileSpans make_tile_spans(const Item& it, int t, int bs) {
  TileSpans ts;
  const int ta = it.qa + t * kBlockM;
  if (ta >= it.qb) {
    ts.half[0] = Span{0, 0, 0, 0};
    ts.half[1] = Span{0, 0, 0, 0};
    return ts;
  }
  const int tb = imin(ta + kBlockM, it.qb);
  ts.half[0] = key_span(it.qh, 0, ta, tb, it.n, bs);
  ts.half[1] = key_span(it.qh, 1, ta, tb, it.n, bs);
  return ts;
}

// What the roles need to know about an item. The TMA warp works it out once (that is where the divisions by the
// block size and the head counts happen) and leaves it in shared memory next to the scheduler's mailbox; the MMA
// thread and the softmax warps copy it from there.
struct ItemDesc {
  Item it;
  KeyPlan plan;
  TileSpans spans[2];
};

template <int kHeadDim, int kQTiles, int kStages, int kType, bool kSoftcap>
struct FwdConfig {
  // kType: 0 bf16, 1 fp16, 2 fp8 e4m3 (forward only; the output is bf16)
  static constexpr bool kFp8 = kType == 2;
  static constexpr int kElemBytes = kFp8 ? 1 : 2;
  static constexpr int kTileBytes = kBlockN * kHeadDim * kElemBytes;  // one 128-row tile of Q, K or V
  static constexpr int kPanelElems = 128 / kElemBytes;                // elements per 128-byte panel row
  static constexpr int kPanels = kHeadDim / kPanelElems;
  static constexpr int kPanelBytes = 128 * 128;
  static constexpr int kStepElems = 32 / kElemBytes;                  // reduction elements per MMA (32 bytes)
  static constexpr int kPCols = kBlockN * kElemBytes / 4;             // tensor-memory columns of the packed P
  static_assert(kHeadDim % kPanelElems == 0, "head dimension must fill whole 128-byte panels");
  // Two query tiles: the two softmax warpgroups need more registers than an even split of the file gives them
  // (168 per thread with the block rounded up to whole warpgroups), so the block is padded to three whole
  // warpgroups and the third (TMA warp, MMA warp, two idle warps) hands most of its registers to the other two.
  static constexpr bool kRegRealloc = kQTiles == 2;
  static constexpr int kThreads = kRegRealloc ? 384 : 128 * kQTiles + 64;
  static constexpr uint32_t kSoftmaxRegs = 216, kProducerRegs = 72;
  // the pool is what the block got at launch, 384 threads x 168 registers: 2 * 128 * 216 + 128 * 72 = 384 * 168.
  // Asking for more than the pool holds would block the warpgroup for ever.
  static_assert(2 * 128 * kSoftmaxRegs + 128 * kProducerRegs <= 384 * 168, "register pool");
  static constexpr int kLoadWarp = 4 * kQTiles;
  static constexpr int kMmaWarp = 4 * kQTiles + 1;
  // epilogue staging: per query tile one [128 rows][64 columns] 16-bit tile, stored to out as a whole
  static constexpr int kStageOBytes = kBlockM * 128;
  static constexpr int kSmemBytes = (kQTiles + kStages) * kTileBytes + kQTiles * kStageOBytes +
                                    1024 /*alignment slack*/ + 1024 /*barriers, mailbox, item descriptions*/;
  static_assert(kSmemBytes <= 232448, "shared memory budget");
  static constexpr int kTmemS = 0;                  // S_t at t*128
  static constexpr int kTmemO = 128 * kQTiles;      // O_t at kTmemO + t*kHeadDim
  static_assert(kTmemO + kQTiles * kHeadDim <= 512, "tensor memory budget");
  // Where columns are left over (head dimensions up to 64) the packed P gets columns of its own instead of
  // overwriting S, and every query tile gets its own MMA issuer. The next S of a tile is then issued as soon as its
  // softmax warps have read this one and runs under their arithmetic; with P in place of S it has to wait for the
  // P V product, and the chain softmax -> P V -> S -> softmax sets the pace. (One issuer for both tiles is held in
  // the issue of 24 small MMAs per step for longer than a softmax takes.)
  static constexpr bool kOwnP = kQTiles == 2 && kQTiles * (128 + kHeadDim + kPCols) <= 512;
  static constexpr int kTmemP = kOwnP ? kTmemO + kQTiles * kHeadDim : kTmemS;   // P_t at kTmemP + t*kPStride
  static constexpr int kPStride = kOwnP ? kPCols : 128;
  // (Two issuers with P in place of S, as head dimension 128 would need, are slower than one: 0.38 against 0.31 ms
  // on the benchmark shape, the two threads' products interleave in the pipe and every one of them takes longer.)
  static constexpr int kIssuers = kOwnP ? kQTiles : 1;
};

template <int kHeadDim, int kQTiles, int kStages, int kType, bool kSoftcap>
__global__ void __launch_bounds__(kQTiles == 2 ? 384 : 128 * kQTiles + 64, 1) fwd_kernel(const __grid_constant__ FwdParams p) {
  using Cfg = FwdConfig<kHeadDim, kQTiles, kStages, kType, kSoftcap>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + kQTiles * Cfg::kTileBytes;
  uint8_t* sStageO = sKV + kStages * Cfg::kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStageO + kQTiles * Cfg::kStageOBytes);
  uint64_t* q_full = bars;                       // 1
  uint64_t* q_empty = bars + 1;                  // 1
  uint64_t* kv_full = bars + 2;                  // kStages
  uint64_t* kv_empty = kv_full + kStages;        // kStages
  uint64_t* s_full = kv_empty + kStages;         // kQTiles
  uint64_t* p_full = s_full + kQTiles;           // kQTiles
  uint64_t* o_full = p_full + kQTiles;           // kQTiles
  uint64_t* s_free = o_full + kQTiles;           // kQTiles; used where P has its own columns: S is in registers
  uint64_t* p_free = s_free + kQTiles;           // kQTiles; likewise: P V has read P (and updated O)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_free + kQTiles);
  static_assert((2 + 2 * kStages + 5 * kQTiles) * 8 + 8 <= 256, "barrier area");
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  SchedMailbox* mbox = reinterpret_cast<SchedMailbox*>(reinterpret_cast<uint8_t*>(bars) + 256);
  ItemDesc* desc = reinterpret_cast<ItemDesc*>(reinterpret_cast<uint8_t*>(bars) + 512);  // two slots
  static_assert(2 * sizeof(ItemDesc) <= 512, "item descriptions");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_items = p.vl.base != nullptr ? p.vl.base[0] * 2 * p.heads : p.total_items;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    sched_init(mbox, 4 * kQTiles + Cfg::kIssuers);
    ptx::mbar_init(q_full, 1);
    ptx::mbar_init(q_empty, Cfg::kIssuers);
    for (int i = 0; i < kStages; ++i) {
      ptx::mbar_init(&kv_full[i], 1);
      ptx::mbar_init(&kv_empty[i], Cfg::kIssuers);   // every issuer lets go of the tile
    }
    for (int t = 0; t < kQTiles; ++t) {
      ptx::mbar_init(&s_full[t], 1);
      ptx::mbar_init(&p_full[t], 4);  // one arrival per softmax warp
      ptx::mbar_init(&o_full[t], 1);
      ptx::mbar_init(&s_free[t], 4);
      ptx::mbar_init(&p_free[t], 1);
    }
    ptx::fence_mbar_init();
  }
  if (warp == Cfg::kLoadWarp) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
    if (lane == 0) {
      ptx::prefetch_tensormap(&p.tm_q);
      ptx::prefetch_tensormap(&p.tm_k);
      ptx::prefetch_tensormap(&p.tm_v);
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int bs = p.block_size;

  // The register counts are set inside the role branches: after a point where the branches meet again the
  // compiler would have to assume the smaller count for everything.
  if (warp >= 4 * kQTiles) {
  if (Cfg::kRegRealloc) ptx::reg_release_to<Cfg::kProducerRegs>();
  if (warp == Cfg::kLoadWarp) {
    // ------------------------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t slot = 0, n_item = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_take(mbox, n_sched, p.ticket, abort_flag);
        if (idx < 0) break;
        if (idx >= total_items) {
          sched_publish(mbox, n_sched, idx);
          break;
        }
        const Item it = decode_item<kQTiles>(p, idx);
        KeyPlan plan{};
        {
          ItemDesc& d = desc[n_sched & 1u];
          d.it = it;
          if (it.valid) {
            plan = make_key_plan(it.qh, it.qa, it.qb, it.n, bs, kBlockN);
            d.plan = plan;
#pragma unroll
            for (int t = 0; t < kQTiles; ++t) d.spans[t] = make_tile_spans(it, t, bs);
          }
        }
        sched_publish(mbox, n_sched, idx);
        if (!it.valid) continue;
        const int steps = plan.steps();
        const int q_row = it.row0 + it.qh * it.n + it.qa;
        const int ntiles = ceil_div(it.qb - it.qa, kBlockM);
        for (int s = 0; s < steps && alive; ++s) {
          int kh, kt;
          plan.step(s, kh, kt);
          const int k_row = it.row0 + kh * it.n + kt * kBlockN;
          for (int which = 0; which < 2; ++which) {  // 0: K tile, 1: V tile
            const uint32_t stage = slot % kStages;
            if (!ptx::mbar_wait(&kv_empty[stage], ((slot / kStages) & 1) ^ 1, abort_flag, 11)) { alive = false; break; }
            ptx::mbar_expect_tx(&kv_full[stage], Cfg::kTileBytes);
            uint8_t* dst = sKV + stage * Cfg::kTileBytes;
            const CUtensorMap* tm = which == 0 ? &p.tm_k : &p.tm_v;
#pragma unroll
            for (int c = 0; c < Cfg::kPanels; ++c) {
              ptx::tma_load_4d(dst + c * Cfg::kPanelBytes, tm, &kv_full[stage], c * Cfg::kPanelElems, k_row, it.hk,
                               it.bcoord);
            }
            ++slot;
            if (s == 0 && which == 0) {
              // Q after the first K tile: the first MMA needs both, the previous item may still own Q.
              if (!ptx::mbar_wait(q_empty, (n_item & 1) ^ 1, abort_flag, 12)) { alive = false; break; }
              ptx::mbar_expect_tx(q_full, ntiles * Cfg::kTileBytes);
              for (int t = 0; t < ntiles; ++t) {
#pragma unroll
                for (int c = 0; c < Cfg::kPanels; ++c) {
                  ptx::tma_load_4d(sQ + t * Cfg::kTileBytes + c * Cfg::kPanelBytes, &p.tm_q, q_full, c * Cfg::kPanelElems,
                                   q_row + t * kBlockM, it.h, it.bcoord);
                }
              }
            }
          }
        }
        ++n_item;
      }
      if (*abort_flag) __nanosleep(100000);  // let copies in flight land before the CTA exits
    }
  } else if (Cfg::kOwnP && warp >= Cfg::kMmaWarp && warp < Cfg::kMmaWarp + Cfg::kIssuers) {
    // ------------------------------------------------------------------------------- MMA issuer of one query tile
    // P has its own columns: S of step s is issued as soon as the softmax warps hold S of step s - 1 (s_free), P V of
    // step s - 1 when they have written P (p_full). Every issuer waits for every K / V tile and lets go of it, also
    // where its own query tile skips the step: an issuer can then never be a whole ring ahead of the other.
    if (lane == 0) {
      const int t = warp - Cfg::kMmaWarp;
      constexpr int kFmt = kType == 0 ? 1 : 0;
      const uint32_t idesc_s = ptx::make_idesc(kBlockM, kBlockN, kFmt, false, false);
      const uint32_t idesc_o = ptx::make_idesc(kBlockM, kHeadDim, kFmt, false, true);
      constexpr uint32_t kDescHi = ptx::smem_desc_hi(1024);
      const uint32_t q_lo = ptx::smem_desc_lo(ptx::smem_u32(sQ), 16) + t * (Cfg::kTileBytes >> 4);
      const uint32_t k_lo0 = ptx::smem_desc_lo(ptx::smem_u32(sKV), 16);
      const uint32_t v_lo0 = ptx::smem_desc_lo(ptx::smem_u32(sKV), Cfg::kPanelBytes);
      const uint32_t tmem_s_t = tmem + Cfg::kTmemS + t * 128;
      const uint32_t tmem_p_t = tmem + Cfg::kTmemP + t * Cfg::kPStride;
      const uint32_t tmem_o_t = tmem + Cfg::kTmemO + t * kHeadDim;
      uint32_t slot = 0, n_item = 0, cnt_p = 0, cnt_s = 0;
      bool alive = true;
      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_peek(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const Item it = desc[n_sched & 1u].it;
        const KeyPlan plan = desc[n_sched & 1u].plan;
        const TileSpans spans = desc[n_sched & 1u].spans[t];
        sched_release<false>(mbox, n_sched);
        if (!it.valid) continue;
        const int steps = plan.steps();
        if (!ptx::mbar_wait(q_full, n_item & 1, abort_flag, 21)) { alive = false; break; }
        bool pend = false, o_acc = false;
        for (int s = 0; s <= steps && alive; ++s) {
          const uint32_t slot_k = slot + 2 * s;        // K tile of step s
          const uint32_t slot_v = slot + 2 * s - 1;    // V tile of step s-1
          bool vis = false;
          if (s < steps) {
            int kh, kt;
            plan.step(s, kh, kt);
            vis = spans.classify(kh, kt) != kTileSkip;
          }
          // S of step s
          auto do_s = [&]() -> bool {
            if (s >= steps) return true;
            if (!ptx::mbar_wait(&kv_full[slot_k % kStages], (slot_k / kStages) & 1, abort_flag, 22)) return false;
            if (vis) {
              if (!ptx::mbar_wait(&s_free[t], (cnt_s & 1) ^ 1, abort_flag, 25)) return false;
              ++cnt_s;
              ptx::tc_fence_after();
              const uint32_t b_lo = k_lo0 + (slot_k % kStages) * (Cfg::kTileBytes >> 4);
#pragma unroll
              for (int kk = 0; kk < kHeadDim / Cfg::kStepElems; ++kk) {
                const uint32_t off = ((kk / 4) * Cfg::kPanelBytes + (kk % 4) * 32) >> 4;
                if (Cfg::kFp8) ptx::umma_ss_f8_lh(tmem_s_t, q_lo + off, b_lo + off, kDescHi, idesc_s, kk > 0);
                else ptx::umma_ss_f16_lh(tmem_s_t, q_lo + off, b_lo + off, kDescHi, idesc_s, kk > 0);
              }
              ptx::umma_commit(&s_full[t]);
            }
            // arrives when this thread's products so far are complete (at once if it issued none on the tile)
            ptx::umma_commit(&kv_empty[slot_k % kStages]);
            if (s == steps - 1) ptx::umma_commit(q_empty);   // Q is read by the S products only
            return true;
          };
          // P V of step s - 1
          auto do_pv = [&]() -> bool {
            if (s == 0) return true;
            if (!ptx::mbar_wait(&kv_full[slot_v % kStages], (slot_v / kStages) & 1, abort_flag, 23)) return false;
            if (pend) {
              if (!ptx::mbar_wait(&p_full[t], cnt_p & 1, abort_flag, 24)) return false;
              ++cnt_p;
              ptx::tc_fence_after();
              const uint32_t b_lo = v_lo0 + (slot_v % kStages) * (Cfg::kTileBytes >> 4);
#pragma unroll
              for (int kk = 0; kk < kBlockN / Cfg::kStepElems; ++kk) {
                const uint32_t b = b_lo + kk * ((Cfg::kStepElems * 128) >> 4);
                const uint32_t acc = (o_acc || kk > 0) ? 1u : 0u;
                if (Cfg::kFp8) ptx::umma_ts_f8_lh(tmem_o_t, tmem_p_t + kk * 8, b, kDescHi, idesc_o, acc);
                else ptx::umma_ts_f16_lh(tmem_o_t, tmem_p_t + kk * 8, b, kDescHi, idesc_o, acc);
              }
              ptx::umma_commit(&p_free[t]);
              o_acc = true;
            }
            ptx::umma_commit(&kv_empty[slot_v % kStages]);
            return true;
          };
          // S first: it only needs the previous S to have been read
          if (!do_s() || !do_pv()) { alive = false; break; }
          pend = vis;
        }
        if (!alive) break;
        if (steps == 0) ptx::umma_commit(q_empty);
        if (it.qa + t * kBlockM < it.qb) ptx::umma_commit(&o_full[t]);
        slot += 2 * steps;
        ++n_item;
      }
    }
  } else if (!Cfg::kOwnP && warp == Cfg::kMmaWarp) {
    // --------------------------------------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr int kFmt = kType == 0 ? 1 : 0;  // kind::f16: 1 = bf16, 0 = f16; kind::f8f6f4: 0 = e4m3
      const uint32_t idesc_s = ptx::make_idesc(kBlockM, kBlockN, kFmt, false, false);
      const uint32_t idesc_o = ptx::make_idesc(kBlockM, kHeadDim, kFmt, false, true);
      uint32_t slot = 0, n_item = 0;
      uint32_t cnt_p[kQTiles];
#pragma unroll
      for (int t = 0; t < kQTiles; ++t) cnt_p[t] = 0;
      bool alive = true;

      // descriptor low words of stage 0 / tile 0; a stage or tile step adds kTileBytes / 16, a k-step a constant
      constexpr uint32_t kDescHi = ptx::smem_desc_hi(1024);
      const uint32_t q_lo0 = ptx::smem_desc_lo(ptx::smem_u32(sQ), 16);
      const uint32_t k_lo0 = ptx::smem_desc_lo(ptx::smem_u32(sKV), 16);
      const uint32_t v_lo0 = ptx::smem_desc_lo(ptx::smem_u32(sKV), Cfg::kPanelBytes);
      auto issue_s = [&](int t, uint32_t k_stage) {
        const uint32_t a_lo = q_lo0 + t * (Cfg::kTileBytes >> 4);
        const uint32_t b_lo = k_lo0 + k_stage * (Cfg::kTileBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < kHeadDim / Cfg::kStepElems; ++kk) {
          const uint32_t off = ((kk / 4) * Cfg::kPanelBytes + (kk % 4) * 32) >> 4;
          if (Cfg::kFp8) ptx::umma_ss_f8_lh(tmem + Cfg::kTmemS + t * 128, a_lo + off, b_lo + off, kDescHi, idesc_s, kk > 0);
          else ptx::umma_ss_f16_lh(tmem + Cfg::kTmemS + t * 128, a_lo + off, b_lo + off, kDescHi, idesc_s, kk > 0);
        }
      };
      auto issue_pv = [&](int t, uint32_t v_stage, bool accumulate) {
        const uint32_t b_lo = v_lo0 + v_stage * (Cfg::kTileBytes >> 4);
#pragma unroll
        for (int kk = 0; kk < kBlockN / Cfg::kStepElems; ++kk) {
          // one MMA consumes 32 bytes of every P row (8 columns) and kStepElems rows of V (128 bytes each)
          const uint32_t a_t = tmem + Cfg::kTmemS + t * 128 + kk * 8;
          const uint32_t b = b_lo + kk * ((Cfg::kStepElems * 128) >> 4);
          if (Cfg::kFp8) ptx::umma_ts_f8_lh(tmem + Cfg::kTmemO + t * kHeadDim, a_t, b, kDescHi, idesc_o, (accumulate || kk > 0) ? 1u : 0u);
          else ptx::umma_ts_f16_lh(tmem + Cfg::kTmemO + t * kHeadDim, a_t, b, kDescHi, idesc_o, (accumulate || kk > 0) ? 1u : 0u);
        }
      };

      for (uint32_t n_sched = 0; alive; ++n_sched) {
        const int idx = sched_peek(mbox, n_sched, abort_flag);
        if (idx < 0 || idx >= total_items) break;
        const Item it = desc[n_sched & 1u].it;
        const KeyPlan plan = desc[n_sched & 1u].plan;
        TileSpans spans[kQTiles];
#pragma unroll
        for (int t = 0; t < kQTiles; ++t) spans[t] = desc[n_sched & 1u].spans[t];
        sched_release<false>(mbox, n_sched);
        if (!it.valid) continue;
        const int steps = plan.steps();
        if (!ptx::mbar_wait(q_full, n_item & 1, abort_flag, 21)) { alive = false; break; }
        bool pend[kQTiles], o_acc[kQTiles];
#pragma unroll
        for (int t = 0; t < kQTiles; ++t) { pend[t] = false; o_acc[t] = false; }
        for (int s = 0; s <= steps && alive; ++s) {
          const uint32_t slot_k = slot + 2 * s;        // K tile of step s
          const uint32_t slot_v = slot + 2 * s - 1;    // V tile of step s-1
          int kh = 0, kt = 0;
          if (s < steps) {
            plan.step(s, kh, kt);
            if (!ptx::mbar_wait(&kv_full[slot_k % kStages], (slot_k / kStages) & 1, abort_flag, 22)) { alive = false; break; }
          }
          if (s > 0) {
            if (!ptx::mbar_wait(&kv_full[slot_v % kStages], (slot_v / kStages) & 1, abort_flag, 23)) { alive = false; break; }
          }
          ptx::tc_fence_after();
#pragma unroll
          for (int t = 0; t < kQTiles; ++t) {
            if (pend[t]) {
              if (!ptx::mbar_wait(&p_full[t], cnt_p[t] & 1, abort_flag, 24)) { alive = false; break; }
              ++cnt_p[t];
              ptx::tc_fence_after();
              issue_pv(t, slot_v % kStages, o_acc[t]);
              o_acc[t] = true;
              pend[t] = false;
            }
            if (s < steps && spans[t].classify(kh, kt) != kTileSkip) {
              issue_s(t, slot_k % kStages);
              ptx::umma_commit(&s_full[t]);
              pend[t] = true;
            }
          }
          if (!alive) break;
          if (s > 0) ptx::umma_commit(&kv_empty[slot_v % kStages]);
          if (s < steps) ptx::umma_commit(&kv_empty[slot_k % kStages]);
          // Q is read by the S products only: after the last of them the next item's Q may load, while the last
          // P V products and the epilogue of this item still run
          if (s == steps - 1) ptx::umma_commit(q_empty);
        }
        if (!alive) break;
        if (steps == 0) ptx::umma_commit(q_empty);
#pragma unroll
        for (int t = 0; t < kQTiles; ++t) {
          if (it.qa + t * kBlockM < it.qb) ptx::umma_commit(&o_full[t]);
        }
        slot += 2 * steps;
        ++n_item;
      }
    }
  }
  } else {
    // ------------------------------------------------------------------------------------ softmax + epilogue
    if (Cfg::kRegRealloc) ptx::reg_acquire_to<Cfg::kSoftmaxRegs>();
    const int t = warp >> 2;                       // query tile of this warpgroup
    const int quad = warp & 3;                     // tensor-memory lane quadrant of this warp
    const int row = quad * 32 + lane;              // row inside the tile
    const uint32_t lane_addr = static_cast<uint32_t>(quad * 32) << 16;
    const uint32_t tmem_s = tmem + Cfg::kTmemS + t * 128 + lane_addr;
    const uint32_t tmem_o = tmem + Cfg::kTmemO + t * kHeadDim + lane_addr;
    const uint32_t tmem_p = tmem + Cfg::kTmemP + t * Cfg::kPStride + lane_addr;
    uint32_t cnt_s = 0, cnt_o = 0;
    bool alive = true;
    uint8_t* stage_o = sStageO + t * Cfg::kStageOBytes;
    for (uint32_t n_sched = 0; alive; ++n_sched) {
      const int idx = sched_peek(mbox, n_sched, abort_flag);
      if (idx < 0 || idx >= total_items) break;
      const Item it = desc[n_sched & 1u].it;
      const TileSpans spans = desc[n_sched & 1u].spans[t];
      const KeyPlan plan = desc[n_sched & 1u].plan;
      sched_release<true>(mbox, n_sched);
      if (!it.valid) continue;
      const int ta = it.qa + t * kBlockM;
      if (ta >= it.qb) continue;
      const int steps = plan.steps();
      const int r = ta + row;                      // position in the half
      const bool row_valid = r < it.n;
      const int r_eff = row_valid ? r : it.n - 1;
      const int blk0 = block_lo(r_eff, bs);
      const int blk1 = imin(blk0 + bs, it.n);
      // FP8: the per-(sample, KV head) descales of q and k fold into the score scale, the descale of v into the
      // final normalisation (the reference does the same, flash_fwd_kernel_sm90.h:299-305, mainloop_fwd...:818-822)
      float scale_log2 = p.scale_log2, softcap_pre = p.softcap_pre, lse_scale = p.lse_scale, out_scale = 1.f;
      if (Cfg::kFp8) {
        float qk = 1.f;
        if (p.q_descale != nullptr) qk *= p.q_descale[it.b * p.descale_bs[0] + it.hk * p.descale_hs[0]];
        if (p.k_descale != nullptr) qk *= p.k_descale[it.b * p.descale_bs[1] + it.hk * p.descale_hs[1]];
        if (p.v_descale != nullptr) out_scale = p.v_descale[it.b * p.descale_bs[2] + it.hk * p.descale_hs[2]];
        if (kSoftcap) {
          softcap_pre *= qk;
        } else {
          scale_log2 *= qk;
          lse_scale *= qk;
        }
      }
      // P is rounded to e4m3 for FP8: keep it in (0, 2^8] by advancing the maximum at every increase and shifting
      // the exponent by 8 (the reference's Max_offset = 8, softmax.h:67-69 there); 16-bit P may run up to 2^8
      // above 1 before the maximum is advanced.
      constexpr float kThreshold = Cfg::kFp8 ? 0.f : kRescaleThreshold;
      constexpr float kPShift = Cfg::kFp8 ? 8.f : 0.f;
      float m_run = -INFINITY;  // reference maximum (unscaled scores, or tanh values with softcap)
      float l_run = 0.f;
      bool o_started = false;
      for (int s = 0; s < steps && alive; ++s) {
        int kh, kt;
        plan.step(s, kh, kt);
        const int cls = spans.classify(kh, kt);
        if (cls == kTileSkip) continue;
        if (!ptx::mbar_wait(&s_full[t], cnt_s & 1, abort_flag, 31)) { alive = false; break; }
        ++cnt_s;
        ptx::tc_fence_after();
        float v[kBlockN];
        {
          uint32_t* u = reinterpret_cast<uint32_t*>(v);
#pragma unroll
          for (int c = 0; c < kBlockN / 32; ++c) ptx::tmem_ld32(tmem_s + c * 32, u + c * 32);
          ptx::tmem_wait_ld();
        }
        // cnt_s - 1 tiles came before this one. With P in its own columns: S may be overwritten from here on, and
        // the P V product of the previous tile must have completed before O is rescaled or P is overwritten (with P
        // in place of S the S product of this tile already followed it through the pipe).
        bool pv_done = !Cfg::kOwnP;
        auto wait_pv = [&]() -> bool {
          if (pv_done) return true;
          pv_done = true;
          if (!ptx::mbar_wait(&p_free[t], cnt_s & 1, abort_flag, 33)) return false;
          ptx::tc_fence_after();
          return true;
        };
        if (Cfg::kOwnP) {
          ptx::tc_fence_before();
          ptx::mbar_arrive_warp(&s_free[t]);
        }
        if (kSoftcap) {
#pragma unroll
          for (int c = 0; c < kBlockN; ++c) v[c] = ptx::tanh_fast(v[c] * softcap_pre);
        }
        if (cls == kTileMasked) {
          int lo, hi;
          if (it.qh == 1) { lo = 0; hi = blk1; }
          else if (kh == 1) { lo = 0; hi = blk0; }
          else { lo = blk0; hi = blk1; }
          lo -= kt * kBlockN;
          hi -= kt * kBlockN;
#pragma unroll
          for (int c = 0; c < kBlockN; ++c) {
            if (c < lo || c >= hi) v[c] = -INFINITY;
          }
        }
        // eight independent running maxima (a single chain of 127 dependent max operations costs more than the
        // exponentials that follow)
        float mx[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) mx[i] = fmaxf(v[2 * i], v[2 * i + 1]);
#pragma unroll
        for (int c = 16; c < kBlockN; c += 16) {
#pragma unroll
          for (int i = 0; i < 8; ++i) mx[i] = ptx::max3(mx[i], v[c + 2 * i], v[c + 2 * i + 1]);
        }
        const float m_tile = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])),
                                   fmaxf(fmaxf(mx[4], mx[5]), fmaxf(mx[6], mx[7])));
        const float m_new = fmaxf(m_run, m_tile);
        // advance the reference maximum only when it grew by more than the threshold (always on the first tile)
        const bool need = (m_new - m_run) * scale_log2 > kThreshold;
        if (__any_sync(0xffffffffu, need)) {
          const float factor = need ? ptx::ex2((m_run - m_new) * scale_log2) : 1.f;
          if (o_started) {
            if (!wait_pv()) { alive = false; break; }
#pragma unroll
            for (int c = 0; c < kHeadDim / 32; ++c) {
              uint32_t o[32];
              ptx::tmem_ld32(tmem_o + c * 32, o);
              ptx::tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              ptx::tmem_st32(tmem_o + c * 32, o);
            }
          }
          l_run *= factor;
          if (need) m_run = m_new;
        }
        const float m_ref = (m_run == -INFINITY) ? 0.f : m_run;
        const float neg_m = kPShift - m_ref * scale_log2;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t pk[Cfg::kPCols];
        if (Cfg::kFp8) {
#pragma unroll
          for (int c = 0; c < kBlockN; c += 4) {
            const float p0 = ptx::ex2(fmaf(v[c], scale_log2, neg_m));
            const float p1 = ptx::ex2(fmaf(v[c + 1], scale_log2, neg_m));
            const float p2 = ptx::ex2(fmaf(v[c + 2], scale_log2, neg_m));
            const float p3 = ptx::ex2(fmaf(v[c + 3], scale_log2, neg_m));
            sum4[(c / 4) & 3] += (p0 + p1) + (p2 + p3);
            pk[c / 4] = ptx::pack_e4m3x4(p0, p1, p2, p3);
          }
        } else {
          // two elements per FMA and per ADD: the sums run as four pairs of partial sums
          float sumb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int c = 0; c < kBlockN; c += 2) {
            float y0, y1;
            ptx::fma2(y0, y1, v[c], v[c + 1], scale_log2, scale_log2, neg_m, neg_m);
            const float p0 = ptx::ex2(y0);
            const float p1 = ptx::ex2(y1);
            ptx::add2(sum4[(c / 2) & 3], sumb[(c / 2) & 3], sum4[(c / 2) & 3], sumb[(c / 2) & 3], p0, p1);
            pk[c / 2] = ptx::pack2<kType == 0>(p0, p1);
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) sum4[i] += sumb[i];
        }
        l_run += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        if (!wait_pv()) { alive = false; break; }
#pragma unroll
        for (int c = 0; c < Cfg::kPCols / 32; ++c) ptx::tmem_st32(tmem_p + c * 32, pk + c * 32);
        ptx::tmem_wait_st();
        ptx::tc_fence_before();
        ptx::mbar_arrive_warp(&p_full[t]);
        o_started = true;
      }
      if (!alive) break;
      // ---- epilogue: O / l -> global, LSE
      if (!ptx::mbar_wait(&o_full[t], cnt_o & 1, abort_flag, 32)) { alive = false; break; }
      ++cnt_o;
      ptx::tc_fence_after();
      const float inv_l = out_scale / l_run;
      const int64_t srow = static_cast<int64_t>(it.row0) + it.qh * it.n + r;
      bool lse_done = false;
      auto store_lse = [&]() {
        lse_done = true;
        if (row_valid) {
          const float m_ref = (m_run == -INFINITY) ? 0.f : m_run;
          const float lse = (l_run > 0.f) ? m_ref * lse_scale + (__log2f(l_run) - kPShift) * kLn2 : -INFINITY;
          const int64_t li = (p.cu_seqlens != nullptr)
                                 ? static_cast<int64_t>(it.h) * p.total + srow
                                 : (static_cast<int64_t>(it.b) * p.heads + it.h) * p.seqlen + (it.qh * it.n + r);
          p.lse[li] = lse;
        }
      };
      if (p.o_tma != 0 && ta + kBlockM <= it.n) {
        // Whole tile: through shared memory, 64 columns at a time, and out as tile copies, one per warp (32 rows),
        // so that no warp waits for another. (A row per thread written straight to global memory costs one
        // memory transaction per thread and instruction; for a 128 x 128 tile that is thousands of cycles in
        // which the load/store unit serves nobody else.)
        uint8_t* my_stage = stage_o + quad * (32 * 128);
#pragma unroll
        for (int pass = 0; pass < kHeadDim / 64; ++pass) {
          if (pass * 64 < p.head_dim) {
            uint32_t o[64];
            ptx::tmem_ld32(tmem_o + pass * 64, o);
            ptx::tmem_ld32(tmem_o + pass * 64 + 32, o + 32);
            ptx::tmem_wait_ld();
            uint32_t w[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              w[i] = ptx::pack2<kType != 1>(__uint_as_float(o[2 * i]) * inv_l, __uint_as_float(o[2 * i + 1]) * inv_l);
            }
            // the previous copy out of this warp's buffer (last pass or last item) must have read it completely
            if (lane == 0) ptx::bulk_wait_group_read0();
            __syncwarp();
            ptx::st_shared_row128_sw(my_stage, lane, w);
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_4d(&p.tm_o, my_stage, pass * 64, it.row0 + it.qh * it.n + ta + quad * 32, it.h, it.bcoord);
              ptx::bulk_commit_group();
            }
            // the log-sum-exp goes out while the tile copy reads the buffer
            if (!lse_done) store_lse();
          }
        }
      } else {
        uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + it.bcoord * p.o_batch_stride + srow * p.o_row_stride +
                         it.h * p.o_head_stride;
        // all loads first, one wait: the stores of a chunk then overlap the conversion of the next
        uint32_t o[kHeadDim <= 128 ? kHeadDim : 128];
        constexpr int kPass = kHeadDim <= 128 ? 1 : kHeadDim / 128;
#pragma unroll
        for (int pass = 0; pass < kPass; ++pass) {
          constexpr int kPassCols = kHeadDim <= 128 ? kHeadDim : 128;
#pragma unroll
          for (int c = 0; c < kPassCols / 32; ++c) ptx::tmem_ld32(tmem_o + pass * 128 + c * 32, o + c * 32);
          ptx::tmem_wait_ld();
          if (row_valid) {
#pragma unroll
            for (int c = 0; c < kPassCols / 32; ++c) {
              ptx::store_row32<kType != 1>(orow, pass * 128 + c * 32, o + c * 32, inv_l, p.head_dim, p.wide_store != 0);
            }
          }
        }
      }
      if (!lse_done) store_lse();
      ptx::tc_fence_before();
    }
    // shared memory must outlive the tile copies that read it
    if (lane == 0) ptx::bulk_wait_group0();
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == Cfg::kLoadWarp) ptx::tmem_dealloc(tmem, 512);
}

template <int kHeadDim, int kQTiles, int kStages, int kType, bool kSoftcap>
int launch_fwd_instance(const FwdParams& p, int grid, cudaStream_t stream) {
  using Cfg = FwdConfig<kHeadDim, kQTiles, kStages, kType, kSoftcap>;
  auto kernel = fwd_kernel<kHeadDim, kQTiles, kStages, kType, kSoftcap>;
  static PerDeviceFlags smem_set;
  const int rc = set_dynamic_smem(kernel, Cfg::kSmemBytes, smem_set);
  if (rc) return rc;
  kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(p);
  FDA_CUDA_TRY(cudaGetLastError());
  return FDA_OK;
}

template <int kHeadDim, int kQTiles, int kStages>
int dispatch_fwd(const FwdParams& p, int grid, bool bf16, bool softcap, cudaStream_t stream) {
  if (bf16) {
    return softcap ? launch_fwd_instance<kHeadDim, kQTiles, kStages, 0, true>(p, grid, stream)
                   : launch_fwd_instance<kHeadDim, kQTiles, kStages, 0, false>(p, grid, stream);
  }
  return softcap ? launch_fwd_instance<kHeadDim, kQTiles, kStages, 1, true>(p, grid, stream)
                 : launch_fwd_instance<kHeadDim, kQTiles, kStages, 1, false>(p, grid, stream);
}

template <int kHeadDim, int kQTiles, int kStages>
int dispatch_fwd_fp8(const FwdParams& p, int grid, bool softcap, cudaStream_t stream) {
  return softcap ? launch_fwd_instance<kHeadDim, kQTiles, kStages, 2, true>(p, grid, stream)
                 : launch_fwd_instance<kHeadDim, kQTiles, kStages, 2, false>(p, grid, stream);
}

}  // namespace

size_t fwd_workspace_bytes(const FdaProblem& pr) {
  // scheduler words, and for packed batches the work list
  return 256 + (pr.cu_seqlens != nullptr ? varlen_list_bytes(pr.batch) : 0);
}

int launch_fwd(const FdaFwdArgs& a, cudaStream_t stream) {
  const FdaProblem& pr = a.p;
  DeviceInfo info;
  int rc = current_device_info(&info);
  if (rc) return rc;
  if (info.cc_major != 10) return FDA_ERR_ARCH;

  const int d = pr.head_dim;
  const bool fp8 = pr.dtype == FDA_E4M3;
  // FP8 rows are padded to whole 128-byte panels, so the smallest FP8 kernel is the 128-wide one
  const int d_round = (d <= 64 && !fp8) ? 64 : (d <= 128 ? 128 : 256);
  const int q_tiles = d_round <= 128 ? 2 : 1;
  const int eb = fp8 ? 1 : 2;
  const int box_cols = 128 / eb;
  const bool varlen = pr.cu_seqlens != nullptr;
  const int64_t rows = varlen ? pr.total : pr.seqlen;
  const int tma_batch = varlen ? 1 : pr.batch;
  const bool fp16 = pr.dtype == FDA_FP16;

  FwdParams p;
  memset(&p, 0, sizeof(p));
  rc = encode_tile_map(&p.tm_q, a.q.ptr, eb, fp8, fp16, d, rows, pr.heads, tma_batch, a.q.row_stride,
                       a.q.head_stride, a.q.batch_stride, box_cols, kBlockM);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_k, a.k.ptr, eb, fp8, fp16, d, rows, pr.heads_k, tma_batch, a.k.row_stride,
                       a.k.head_stride, a.k.batch_stride, box_cols, kBlockN);
  if (rc) return rc;
  rc = encode_tile_map(&p.tm_v, a.v.ptr, eb, fp8, fp16, d, rows, pr.heads_k, tma_batch, a.v.row_stride,
                       a.v.head_stride, a.v.batch_stride, box_cols, kBlockN);
  if (rc) return rc;
  if (fp8) {
    p.q_descale = a.q_descale;
    p.k_descale = a.k_descale;
    p.v_descale = a.v_descale;
    for (int i = 0; i < 3; ++i) {
      p.descale_bs[i] = a.descale_batch_stride[i];
      p.descale_hs[i] = a.descale_head_stride[i];
    }
  }
  {
    // out: 16-bit whatever the inputs are. What the tile copy wants of out (16-byte aligned base and strides) is
    // also what the row stores of partial tiles need, so a refusal here is final.
    const int orc = encode_tile_map(&p.tm_o, a.out.ptr, 2, false, fp16, d, rows, pr.heads, tma_batch, a.out.row_stride,
                                    a.out.head_stride, a.out.batch_stride, 64, 32);
    if (orc != FDA_OK) return orc;
    p.o_tma = 1;
  }
  p.out = a.out.ptr;
  p.lse = a.lse;
  p.o_batch_stride = varlen ? 0 : a.out.batch_stride;
  p.o_row_stride = a.out.row_stride;
  p.o_head_stride = a.out.head_stride;
  p.wide_store = (d % 16 == 0 && (reinterpret_cast<uintptr_t>(a.out.ptr) & 31) == 0 && a.out.row_stride % 16 == 0 &&
                  a.out.head_stride % 16 == 0 && (varlen || a.out.batch_stride % 16 == 0))
                     ? 1
                     : 0;
  p.cu_seqlens = pr.cu_seqlens;
  p.batch = pr.batch;
  p.seqlen = pr.seqlen;
  p.total = pr.total;
  p.heads = pr.heads;
  p.heads_k = pr.heads_k;
  p.head_dim = d;
  p.block_size = pr.block_size;
  const int max_n = pr.seqlen / 2;
  p.items_per_half = ceil_div(max_n, q_tiles * kBlockM);
  p.total_items = p.items_per_half * 2 * pr.heads * pr.batch;
  const bool softcap = pr.softcap > 0.f;
  if (softcap) {
    p.scale_log2 = pr.softcap * kLog2e;
    p.softcap_pre = pr.softmax_scale / pr.softcap;
    p.lse_scale = pr.softcap;
  } else {
    p.scale_log2 = pr.softmax_scale * kLog2e;
    p.softcap_pre = 0.f;
    p.lse_scale = pr.softmax_scale;
  }
  if (p.total_items <= 0) return FDA_OK;
  if (!a.workspace || a.workspace_bytes < fwd_workspace_bytes(pr)) return FDA_ERR_WORKSPACE;
  p.ticket = static_cast<int*>(a.workspace);
  FDA_CUDA_TRY(cudaMemsetAsync(p.ticket, 0, 256, stream));
  int grid = info.sm_count - (pr.sm_margin > 0 ? pr.sm_margin : 0);
  if (grid < 1) grid = 1;
  // the shortest eighths of every (sample, head) run at the end; few items per CTA: rank for rank over all of them
  p.n_long = order_n_long(2 * p.items_per_half, FDA_SHORT8_FWD, p.total_items, grid);
  if (varlen) {
    // the work list is built on the device from cu_seqlens (no host synchronisation): the host only knows an upper
    // bound of the number of items, blocks beyond the real number find no work and leave
    int* list = reinterpret_cast<int*>(static_cast<uint8_t*>(a.workspace) + 256);
    const int rc = launch_varlen_prepare(pr.cu_seqlens, pr.batch, q_tiles * kBlockM, list, stream);
    if (rc) return rc;
    p.vl.base = list;
    p.vl.batch = pr.batch;
    const int64_t bound = (static_cast<int64_t>(pr.total) / (2 * q_tiles * kBlockM) + pr.batch) * 2 * pr.heads;
    if (grid > bound) grid = static_cast<int>(bound);
  } else if (grid > p.total_items) {
    grid = p.total_items;
  }
  const bool bf16 = pr.dtype == FDA_BF16;
  if (fp8) {
    if (d_round == 128) return dispatch_fwd_fp8<128, 2, 6>(p, grid, softcap, stream);
    return dispatch_fwd_fp8<256, 1, 4>(p, grid, softcap, stream);
  }
  if (d_round == 64) return dispatch_fwd<64, 2, 6>(p, grid, bf16, softcap, stream);
  if (d_round == 128) return dispatch_fwd<128, 2, 4>(p, grid, bf16, softcap, stream);
  return dispatch_fwd<256, 1, 2>(p, grid, bf16, softcap, stream);
}



int read_status_fwd(int32_t* out4) {
  int zero[4] = {0, 0, 0, 0};
  FDA_CUDA_TRY(cudaMemcpyFromSymbol(out4, g_fda_status, sizeof(int) * 4));
  FDA_CUDA_TRY(cudaMemcpyToSymbol(g_fda_status, zero, sizeof(int) * 4));
  return FDA_OK;
}

}  // namespace fda
