"""Worker for tests/test_multirank_cpu.py: run under torchrun with the gloo backend (no GPU)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import bench  # noqa: E402


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # the slowest rank defines the step time
    got = bench.max_over_ranks(10.0 + 3.0 * rank, dist, world, torch.device("cpu"))
    assert got == 10.0 + 3.0 * (world - 1), got
    # shards are disjoint streams of synthetic samples
    seeds = [None] * world
    dist.all_gather_object(seeds, bench.shard_seed(rank))
    assert len(set(seeds)) == world, seeds
    g = torch.Generator().manual_seed(bench.shard_seed(rank))
    mine = torch.randn(4, generator=g)
    both = [torch.zeros(4) for _ in range(world)]
    dist.all_gather(both, mine)
    assert not torch.equal(both[0], both[-1])
    dist.barrier()
    if rank == 0:
        print("GLOO_WORKER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
