// Persistent work-item scheduler shared by the kernels: every CTA starts with item blockIdx.x and then takes
// items from a global ticket counter, so long items (issued first) do not leave SMs idle at the end. One
// producer thread (the TMA warp) fetches the ticket and hands the item index to the other roles through a
// two-slot shared-memory mailbox guarded by mbarriers; because it runs ahead, the loads of the next item start
// while the current one is still being computed.
//
// The reference has the same idea for its forward only (atomicAdd ticket + named barriers,
// csrc/fda/tile_scheduler.hpp:51-185 there) and launches one CTA per key tile for the backward
// (tile_scheduler.hpp:362-482); here all three kernels are persistent and share this code.
#pragma once

#include "geometry.h"
#include "ptx.cuh"

namespace fda {

struct SchedMailbox {
  uint64_t full[2];
  uint64_t empty[2];
  int idx[2];
  int pad[2];
};

// Call from one thread before the CTA-wide barrier that publishes the mbarrier initialisation.
// `consumer_arrivals` = number of arrive() calls the consumers make per item (one per consumer warp here).
__device__ __forceinline__ void sched_init(SchedMailbox* m, int consumer_arrivals) {
  for (int i = 0; i < 2; ++i) {
    ptx::mbar_init(&m->full[i], 1);
    ptx::mbar_init(&m->empty[i], consumer_arrivals);
  }
}

// Producer side, one thread, in two halves so that the producer can leave a description of the item in shared
// memory (two slots, indexed like the mailbox: it & 1) before the consumers see the index. `it` counts the
// items this CTA has taken (0, 1, 2, ...). sched_take returns the item index (>= total means "no more work"), or
// -1 if a wait was abandoned; from then on slot it & 1 belongs to the producer until sched_publish.
__device__ __forceinline__ int sched_take(SchedMailbox* m, uint32_t it, int* ticket, volatile int* abort_flag) {
  const uint32_t slot = it & 1u;
  if (!ptx::mbar_wait(&m->empty[slot], ((it >> 1) & 1u) ^ 1u, abort_flag, 5)) return -1;
  return (it == 0) ? static_cast<int>(blockIdx.x) : static_cast<int>(gridDim.x) + atomicAdd(ticket, 1);
}
__device__ __forceinline__ void sched_publish(SchedMailbox* m, uint32_t it, int idx) {
  const uint32_t slot = it & 1u;
  m->idx[slot] = idx;
  ptx::mbar_arrive(&m->full[slot]);  // release: the index and the description are visible to whoever sees the
                                     // phase complete
}
__device__ __forceinline__ int sched_produce(SchedMailbox* m, uint32_t it, int* ticket, volatile int* abort_flag) {
  const int v = sched_take(m, it, ticket, abort_flag);
  if (v >= 0) sched_publish(m, it, v);
  return v;
}

// Consumer side, also in two halves: sched_peek waits for item `it` and returns its index; the consumer may then
// read the item's description; sched_release hands the slot back. kWholeWarp: called by every lane of a consumer
// warp, lane 0 makes the arrival for the warp after all lanes are done with the slot. Otherwise: called by a
// single thread that makes its own arrival.
__device__ __forceinline__ int sched_peek(SchedMailbox* m, uint32_t it, volatile int* abort_flag) {
  const uint32_t slot = it & 1u;
  if (!ptx::mbar_wait(&m->full[slot], (it >> 1) & 1u, abort_flag, 6)) return -1;
  return m->idx[slot];
}
template <bool kWholeWarp>
__device__ __forceinline__ void sched_release(SchedMailbox* m, uint32_t it) {
  const uint32_t slot = it & 1u;
  if (kWholeWarp) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(&m->empty[slot]);
  } else {
    ptx::mbar_arrive(&m->empty[slot]);
  }
}
template <bool kWholeWarp>
__device__ __forceinline__ int sched_consume(SchedMailbox* m, uint32_t it, volatile int* abort_flag) {
  const int v = sched_peek(m, it, abort_flag);
  if (v >= 0) sched_release<kWholeWarp>(m, it);
  return v;
}

}  // namespace fda
