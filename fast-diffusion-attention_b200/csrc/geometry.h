// Geometry of the block-diffusion mask: which key tiles a query tile visits, which query tiles a key tile
// visits, and which of those need an element mask. Plain C++ (no CUDA types) so the same code runs in the
// kernels and in host unit tests.
//
// A sample is [noisy half (n rows) | clean half (n rows)]; positions of a half are cut into blocks of `bs`
// counted from the start of the half. half index: 0 = noisy, 1 = clean. Visibility (the reference states it
// in csrc/fda/diffusion.h:6-19 and fast_diffusion_attention/reference.py:4-11):
//   noisy i -> noisy j : same block           noisy i -> clean c : block(c) <  block(i)
//   clean c -> clean c': block(c') <= block(c) clean -> noisy     : never
// For a query the visible keys of one half are one interval, and so are the queries that see a key
// (csrc/fda/diffusion.h:94-119 there gives the same intervals); both interval ends are non-decreasing in the
// position, which is what the tile classification below relies on.
#pragma once

#if defined(__CUDACC__)
#define FDA_HD __host__ __device__ __forceinline__
#else
#define FDA_HD inline
#endif

namespace fda {

FDA_HD int imin(int a, int b) { return a < b ? a : b; }
FDA_HD int imax(int a, int b) { return a > b ? a : b; }
FDA_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Start / end (exclusive, clipped to n) of the block that holds position x of a half.
FDA_HD int block_lo(int x, int bs) { return (x / bs) * bs; }
FDA_HD int block_hi(int x, int bs, int n) { return imin((x / bs) * bs + bs, n); }

// Keys of half kh visible from query position qi (< n) of half qh: [lo, hi). Empty for clean -> noisy.
FDA_HD void key_interval(int qh, int kh, int qi, int n, int bs, int& lo, int& hi) {
  const int b0 = block_lo(qi, bs);
  const int b1 = imin(b0 + bs, n);
  if (qh == 1) { lo = 0; hi = (kh == 1) ? b1 : 0; }
  else if (kh == 1) { lo = 0; hi = b0; }
  else { lo = b0; hi = b1; }
}

// Queries of half qh that see key position kj of half kh: [lo, hi). Empty if kj >= n or clean -> noisy.
FDA_HD void query_interval(int qh, int kh, int kj, int n, int bs, int& lo, int& hi) {
  if (kj >= n || (qh == 1 && kh == 0)) { lo = 0; hi = 0; return; }
  const int b0 = block_lo(kj, bs);
  if (kh == 1) { lo = (qh == 1) ? b0 : imin(b0 + bs, n); hi = n; }
  else { lo = b0; hi = imin(b0 + bs, n); }
}

enum TileClass : int { kTileSkip = 0, kTileFull = 1, kTileMasked = 2 };

// Classify the (query rows [qa, qb) of half qh) x (keys [k0, k0 + bn) of half kh) tile; qa < qb <= n.
// Full: every query row sees every one of the bn keys (so all bn keys exist). Skip: nothing visible.
// With need_full_rows (backward) a tile whose query rows stop short of `bm` rows is never "full", because
// the padding rows must be masked out of the column sums.
FDA_HD int classify_tile(int qh, int kh, int qa, int qb, int k0, int bn, int n, int bs,
                         int bm = 0, bool need_full_rows = false) {
  int lo_a, hi_a, lo_b, hi_b;
  key_interval(qh, kh, qa, n, bs, lo_a, hi_a);
  key_interval(qh, kh, qb - 1, n, bs, lo_b, hi_b);
  const int k1 = k0 + bn;
  // union over the rows is [lo_a, hi_b): the ends are non-decreasing in the row
  if (k0 >= hi_b || k1 <= lo_a || hi_b <= lo_a) return kTileSkip;
  // with several blocks inside the query tile a middle row may see keys the first and last do not, but a key
  // tile between lo_a and hi_b always meets some row's interval, so "skip" above is exact for same-half
  // noisy tiles too: consecutive blocks tile the key axis without gaps.
  if (lo_b <= k0 && k1 <= hi_a && !(need_full_rows && (qb - qa) < bm)) return kTileFull;
  return kTileMasked;
}

// Division-free classification for the kernels' inner loops. A span holds the visibility intervals of the FIRST
// and the LAST position of a fixed tile on one axis (queries for the forward / dQ kernels, keys for the dK/dV
// kernel); it is built once per work item (that is where the divisions by the block size happen) and then
// classifies any tile [x0, x0 + len) on the other axis with compares only. Both interval ends are monotone, so
// the union over the fixed tile is [lo_first, hi_last) and the intersection is [lo_last, hi_first).
struct Span {
  int lo_first, hi_first, lo_last, hi_last;
  // `limit` = number of valid positions on the other axis (n): a full tile must lie inside it.
  FDA_HD int classify(int x0, int len) const {
    const int x1 = x0 + len;
    if (x0 >= hi_last || x1 <= lo_first || hi_last <= lo_first) return kTileSkip;
    if (lo_last <= x0 && x1 <= hi_first) return kTileFull;
    return kTileMasked;
  }
};

// Keys of half kh seen by the query rows [qa, qb) of half qh (qa < qb <= n). classify(k0, bn) then agrees with
// classify_tile(qh, kh, qa, qb, k0, bn, n, bs).
FDA_HD Span key_span(int qh, int kh, int qa, int qb, int n, int bs) {
  Span s;
  key_interval(qh, kh, qa, n, bs, s.lo_first, s.hi_first);
  key_interval(qh, kh, qb - 1, n, bs, s.lo_last, s.hi_last);
  return s;
}

// Query rows of half qh that see the keys [k0, k1) of half kh (k0 < k1 <= n). classify(qa, rows) calls a query
// tile full when all of its `rows` positions see every key of [k0, k1); the caller still has to treat a key
// tile that runs past n (k1 - k0 < tile) as masked.
FDA_HD Span query_span(int qh, int kh, int k0, int k1, int n, int bs) {
  Span s;
  query_interval(qh, kh, k0, n, bs, s.lo_first, s.hi_first);
  query_interval(qh, kh, k1 - 1, n, bs, s.lo_last, s.hi_last);
  return s;
}

// ---------------------------------------------------------------------------------------------------------
// Forward-shaped enumeration (also used by the dQ kernel): key tiles visited by the query rows [qa, qb) of
// half qh. Steps 0..n_clean-1 are clean key tiles 0.., the remaining n_noisy steps are noisy key tiles
// noisy_lo.. (only for noisy queries). The reference enumerates the same set in csrc/fda/diffusion.h:134-183.
// ---------------------------------------------------------------------------------------------------------
struct KeyPlan {
  int n_clean;
  int noisy_lo;
  int n_noisy;
  FDA_HD int steps() const { return n_clean + n_noisy; }
  FDA_HD void step(int s, int& kh, int& kt) const {
    if (s < n_clean) { kh = 1; kt = s; } else { kh = 0; kt = noisy_lo + (s - n_clean); }
  }
};

FDA_HD KeyPlan make_key_plan(int qh, int qa, int qb, int n, int bs, int bn) {
  KeyPlan p;
  const int last = qb - 1;
  const int clean_hi = (qh == 1) ? block_hi(last, bs, n) : block_lo(last, bs);
  p.n_clean = ceil_div(clean_hi, bn);
  if (qh == 0) {
    p.noisy_lo = block_lo(qa, bs) / bn;
    p.n_noisy = ceil_div(block_hi(last, bs, n), bn) - p.noisy_lo;
  } else {
    p.noisy_lo = 0;
    p.n_noisy = 0;
  }
  return p;
}

// ---------------------------------------------------------------------------------------------------------
// Backward (dK/dV-stationary) enumeration: query tiles of `bm` rows that see the keys [k0, k1) (k1 <= n) of
// half kh. List 0 = query tiles of the same half, list 1 = noisy query tiles of later blocks (clean keys
// only). The reference's equivalent is csrc/fda/diffusion.h:196-261.
// ---------------------------------------------------------------------------------------------------------
struct QueryPlan {
  int same_lo, n_same;     // query tiles of half kh
  int cross_lo, n_cross;   // noisy query tiles seeing clean keys
  FDA_HD int steps() const { return n_same + n_cross; }
  FDA_HD void step(int s, int kh, int& qh, int& qt) const {
    if (s < n_same) { qh = kh; qt = same_lo + s; } else { qh = 0; qt = cross_lo + (s - n_same); }
  }
};

FDA_HD QueryPlan make_query_plan(int kh, int k0, int k1, int n, int bs, int bm) {
  QueryPlan p;
  int lo, hi, lo2, hi2;
  query_interval(kh, kh, k0, n, bs, lo, hi);
  query_interval(kh, kh, k1 - 1, n, bs, lo2, hi2);
  hi = imax(hi, hi2);
  p.same_lo = lo / bm;
  p.n_same = ceil_div(hi, bm) - p.same_lo;
  p.cross_lo = 0;
  p.n_cross = 0;
  if (kh == 1) {
    query_interval(0, 1, k0, n, bs, lo, hi);
    if (lo < hi) {
      p.cross_lo = lo / bm;
      p.n_cross = ceil_div(hi, bm) - p.cross_lo;
    }
  }
  return p;
}

// ---------------------------------------------------------------------------------------------------------
// Order in which the persistent kernels take their items
// ---------------------------------------------------------------------------------------------------------
// Order of the items. Every group (a sample and head) has `per_group` items ranked longest first. Rank for rank the
// groups follow each other (group-major), so that the CTAs running at the same time share a group's tiles in L2;
// but the short items of ALL groups come after the long items of all groups: the kernel then ends on short
// items, and the CTAs finish within one short item of each other instead of one long one.
//
// A launch with only a few items per CTA (n_long < 0) drops the grouping: rank for rank over all groups, so that
// every group's longest items start first. (Group-major, the CTAs would reach the last groups' longest items only
// after a full round, and the launch would end one long item later than it has to.)
FDA_HD void two_phase_order(int idx, int per_group, int n_long, int n_groups, int& group, int& rank) {
  if (n_long < 0) {
    rank = idx / n_groups;
    group = idx - rank * n_groups;
    return;
  }
  const int long_total = n_long * n_groups;
  if (idx < long_total) {
    group = idx / n_long;
    rank = idx - group * n_long;
  } else {
    const int j = idx - long_total;
    const int n_short = per_group - n_long;   // > 0 here, or long_total would cover every index
    group = j / n_short;
    rank = n_long + (j - group * n_short);
  }
}

// Host side: the n_long of a launch. `short8` eighths of a group's items count as short. Launches with at most
// FDA_RANK_MAJOR_ITEMS_PER_CTA items per CTA use the rank-major order (-1); with more items the tail matters less
// than sharing a group's tiles in L2.
#ifndef FDA_RANK_MAJOR_ITEMS_PER_CTA
#define FDA_RANK_MAJOR_ITEMS_PER_CTA 8
#endif
FDA_HD int order_n_long(int per_group, int short8, long long total_items, int ctas) {
  if (total_items <= static_cast<long long>(FDA_RANK_MAJOR_ITEMS_PER_CTA) * ctas) return -1;
  const int n_long = per_group - (short8 * per_group) / 8;
  return n_long < 1 ? 1 : n_long;
}

}  // namespace fda
