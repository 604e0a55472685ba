"""Host-side arithmetic of batch sharding across ranks (one process per GPU): which slab of the
outermost extent a rank owns, and torch.distributed forms of the gather / weight-gradient sum that run
on any backend.

Every benchmarked op shards over its outermost extent with no data-path exchange (images for conv
fprop/dgrad, matrices for batched matmul, batch for SDPA, rows for norms and row reductions); the
shards are dense leading slabs of the full tensors. The only real exchange is wgrad: each rank reduces
over its own images and the partial filter gradients are summed (fp32) across ranks before the final
rounding. On GPUs that sum and the output gather are `fusilli_b200.comm.Comm` (the C ABI's fb_comm_*:
fused peer-memory kernel, NCCL all-reduce, NCCL all-gather); the torch.distributed helpers below state
the same operations for the CPU tests (gloo, world size 2, results from the CPU oracle).

The reference has no multi-device code (one Handle = one device,
include/fusilli/backend/runtime.h:19-24).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """[begin, end) of the leading extent owned by `rank`; sizes differ by at most one
    and earlier ranks take the remainder."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def shard_leading(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's dense slab of a tensor sharded on dim 0."""
    b, e = shard_range(t.shape[0], rank, world)
    return t[b:e]


def all_gather_leading(local: torch.Tensor, total: int) -> torch.Tensor:
    """Concatenates every rank's slab along dim 0 (slabs may differ by one row)."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        return local
    sizes = [shard_range(total, r, world) for r in range(world)]
    if all(e - b == sizes[0][1] - sizes[0][0] for b, e in sizes):
        out = torch.empty((total,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous())
        return out
    # uneven slabs: collectives want equal sizes, so pad to the largest slab and trim
    biggest = max(e - b for b, e in sizes)
    padded = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([p[: e - b] for p, (b, e) in zip(parts, sizes)], 0)


def all_reduce_wgrad(partial_dw: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Sums per-rank filter gradients in fp32 and rounds once to the gradient's dtype."""
    acc = partial_dw.to(torch.float32)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(acc, op=dist.ReduceOp.SUM)
    return acc.to(out_dtype)


def max_over_ranks(value: float, device="cpu") -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
