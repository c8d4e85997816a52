// Work list for packed ("varlen") batches: samples ordered longest first, with running tile counts, built on the
// device from cu_seqlens so that no host synchronisation is needed. The kernels' persistent schedulers then
// enumerate exactly the tiles that exist (no ticket is spent on a tile past the end of a short sample) and start
// with the long samples, so a long sample late in the batch cannot become the tail of the launch.
//
// The reference prepares the same thing for its forward (csrc/fda/flash_prepare_scheduler.cu:25-84: sort by
// length with cub::BlockMergeSort, per-sample tile counts, virtual -> actual batch index) and consumes it in
// VarlenDynamicPersistentTileScheduler (csrc/fda/tile_scheduler.hpp:191-353, prefix-sum search per tile). Here one
// list serves the forward and all backward kernels; the order is found by counting (batches are small).
#pragma once

#include <cstdint>

namespace fda {

// Device memory, in ints: [0] sum of units, [1 .. 1 + batch) order (virtual -> actual sample),
// [1 + batch .. 2 + 2 batch) cum (units of the samples before virtual sample v; cum[batch] = the sum).
struct VarlenList {
  const int* base;   // nullptr: batched layout, every sample has the same length
  int batch;
  __host__ __device__ const int* order() const { return base + 1; }
  __host__ __device__ const int* cum() const { return base + 1 + batch; }
};

inline size_t varlen_list_bytes(int batch) { return ((static_cast<size_t>(2 * batch + 2) * 4) + 255) / 256 * 256; }

// Position of flat item `idx` when every unit of every sample carries `per_unit` items (2 halves x heads):
// virtual sample v, actual sample b, its number of units, and the item's index inside the sample.
struct VarlenPos {
  int b, units, rem;
};

__device__ __forceinline__ VarlenPos varlen_locate(const VarlenList& vl, int idx, int per_unit) {
  const int* cum = vl.cum();
  const int key = idx / per_unit;          // units before the item's unit
  int lo = 0, hi = vl.batch;               // largest v with cum[v] <= key (cum[batch] > key for a valid idx)
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cum[mid] <= key) lo = mid; else hi = mid;
  }
  VarlenPos pos;
  pos.b = vl.order()[lo];
  pos.units = cum[lo + 1] - cum[lo];
  pos.rem = idx - cum[lo] * per_unit;
  return pos;
}

// One block. unit_rows = rows of a half that one unit covers (128-row tiles in the backward, the forward's item).
__global__ void varlen_prepare_kernel(const int32_t* __restrict__ cu_seqlens, int batch, int unit_rows, int* out);

int launch_varlen_prepare(const int32_t* cu_seqlens, int batch, int unit_rows, int* out, void* stream);

}  // namespace fda
