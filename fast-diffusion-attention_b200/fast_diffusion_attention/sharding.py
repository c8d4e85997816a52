"""Splitting one attention problem over the GPUs of a box, and putting the results back together.

Block-diffusion attention has no exchange step: a (sample, key/value head) unit with its group of query heads is
independent of every other unit. A fixed problem is therefore cut into equal slices, one per rank, either over
key/value heads (every rank keeps all samples, which also keeps every rank's `cu_seqlens` identical for packed
inputs) or, when there are fewer key/value heads than ranks, over samples. The only communication is the scatter
of q, k, v, dO from the rank that holds them and the gather of out, dq, dk, dv back to it; the kernels never touch
another GPU's memory. The reference has no multi-GPU code; this is the data-parallel harness around its operator.

Works with any torch.distributed backend (NCCL on GPUs, gloo on CPU ranks in the tests).
"""

from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def plan(batch: int, heads: int, heads_k: int, world: int, packed: bool = False) -> Tuple[str, int]:
    """("heads", key/value heads per rank) or ("batch", samples per rank). Raises if neither divides evenly."""
    if world < 1:
        raise ValueError("world size must be positive")
    if heads % heads_k != 0:
        raise ValueError("Number of heads in key/value must divide number of heads in query")
    if heads_k % world == 0:
        return "heads", heads_k // world
    if not packed and batch % world == 0:
        return "batch", batch // world
    raise ValueError(f"cannot cut batch={batch}, heads_k={heads_k} into {world} equal slices")


def shard(t: torch.Tensor, rank: int, world: int, kind: str) -> torch.Tensor:
    """Contiguous copy of rank `rank`'s slice of a (batch, rows, heads, dim) or (total, heads, dim) tensor. The
    head slice of q / out / dq holds the query heads of the rank's key/value heads (heads are grouped contiguously:
    query head h belongs to key/value head h // (heads / heads_k))."""
    if kind == "heads":
        per = t.shape[-2] // world
        return t[..., rank * per:(rank + 1) * per, :].contiguous()
    per = t.shape[0] // world
    return t[rank * per:(rank + 1) * per].contiguous()


def reassemble(parts: Sequence[torch.Tensor], kind: str) -> torch.Tensor:
    """Inverse of `shard` over all ranks, in rank order."""
    return torch.cat(list(parts), dim=-2 if kind == "heads" else 0)


def shard_shape(shape: Sequence[int], world: int, kind: str) -> Tuple[int, ...]:
    shape = list(shape)
    if kind == "heads":
        shape[-2] //= world
    else:
        shape[0] //= world
    return tuple(shape)


def scatter(full: Optional[torch.Tensor], shape: Sequence[int], dtype, device, kind: str, src: int = 0,
            group=None) -> torch.Tensor:
    """Every rank receives its slice of `full`, which only rank `src` holds (shape = the FULL tensor's shape)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    mine = torch.empty(shard_shape(shape, world, kind), dtype=dtype, device=device)
    pieces = [shard(full, r, world, kind) for r in range(world)] if rank == src else None
    dist.scatter(mine, pieces, src=src, group=group)
    return mine


def gather(mine: torch.Tensor, kind: str, dst: int = 0, group=None) -> Optional[torch.Tensor]:
    """Rank `dst` receives every rank's slice and returns the reassembled tensor; the other ranks return None."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    mine = mine.contiguous()
    parts: Optional[List[torch.Tensor]] = [torch.empty_like(mine) for _ in range(world)] if rank == dst else None
    dist.gather(mine, parts, dst=dst, group=group)
    return reassemble(parts, kind) if rank == dst else None
