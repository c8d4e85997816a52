"""Worker for tests/test_multirank_cpu.py: run under torchrun with the gloo backend (no GPU).

Every rank plays one GPU of the multi-GPU benchmark on the CPU: rank 0 holds a whole problem, the slices are
scattered, each rank evaluates the oracle on its slice (standing in for the kernels), the results are gathered, and
rank 0 checks that the reassembled tensors are bitwise what one rank computes on the whole problem.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "fast-diffusion-attention_b200"))
import bench  # noqa: E402
from oracle import diffusion_oracle as orc  # noqa: E402

# sharding.py has no CUDA dependency; the package __init__ loads the CUDA library, which a CPU rank does not need
import importlib.util  # noqa: E402
_spec = importlib.util.spec_from_file_location(
    "fda_sharding", os.path.join(ROOT, "fast-diffusion-attention_b200", "fast_diffusion_attention", "sharding.py"))
sharding = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(sharding)


def run_case(rank, world, batch, n, heads, heads_k, d, bs):
    kind, per = sharding.plan(batch, heads, heads_k, world)
    shapes = [(batch, 2 * n, h, d) for h in (heads, heads_k, heads_k, heads)]
    full = None
    if rank == 0:
        g = torch.Generator().manual_seed(7)
        full = [torch.randn(s, generator=g) for s in shapes]
    mine = [sharding.scatter(full[i] if rank == 0 else None, shapes[i], torch.float32, torch.device("cpu"), kind)
            for i in range(4)]
    q, k, v, do = mine
    out, _ = orc.forward(q, k, v, bs)
    dq, dk, dv = orc.backward(q, k, v, do, bs)
    got = [sharding.gather(t, kind) for t in (out, dq, dk, dv)]
    if rank == 0:
        want_out, _ = orc.forward(*full[:3], bs)
        want = (want_out,) + tuple(orc.backward(*full, bs))
        for name, a, b in zip(("out", "dq", "dk", "dv"), got, want):
            assert a.shape == b.shape, (name, a.shape, b.shape)
            assert torch.equal(a, b), f"{name} differs after {kind} sharding"
    else:
        assert all(t is None for t in got)
    return kind


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # the slowest rank defines the step time
    got = bench.max_over_ranks(10.0 + 3.0 * rank, dist, world, torch.device("cpu"))
    assert got == 10.0 + 3.0 * (world - 1), got
    # key/value heads divide by the world size: slices over heads (grouped query heads travel with their head)
    assert run_case(rank, world, batch=2, n=24, heads=8, heads_k=4, d=16, bs=8) == "heads"
    # one key/value head: slices over samples
    assert run_case(rank, world, batch=4, n=10, heads=3, heads_k=1, d=8, bs=4) == "batch"
    # neither divides: refused on every rank alike
    try:
        sharding.plan(3, 3, 1, world)
        raise AssertionError("expected ValueError")
    except ValueError:
        pass
    dist.barrier()
    if rank == 0:
        print("GLOO_WORKER_OK", world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
