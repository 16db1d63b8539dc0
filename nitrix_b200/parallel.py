"""Data-parallel partition of attention over the GPUs of one node.

Every (batch, head) pair is an independent attention problem -- the reference
already launches one program column per pair (reference
``src/nitrix/_kernels/cuda/attention.py:218,452,492``) -- so the path shards with
no exchange step: rank ``r`` of ``W`` takes a contiguous range of the flattened
``b * H + h`` axis and runs the ordinary kernels on it.  The only collective is
an optional all-gather of the output for callers that want a replicated result
(NCCL over NVLink through ``torch.distributed``); it is enqueued after the
kernels, outside the hot loop.

One process per GPU (``torchrun``); nothing here spawns threads or streams.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def bh_partition(n_units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous ``[begin, end)`` share of ``n_units`` for ``rank``: sizes differ by at most one."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    base, extra = divmod(n_units, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_axis(batch: int, heads: int, world_size: int) -> str:
    """Which axis a node-level launcher slices: whole batches when they divide evenly
    (key-padding workloads: 4 sequences per GPU), else heads (one long sequence: 2 heads
    per GPU), else the flattened pair index."""
    if batch % world_size == 0:
        return "batch"
    if heads % world_size == 0:
        return "heads"
    return "pairs"


def local_slice(x: Optional[torch.Tensor], axis: str, world_size: int, rank: int, *, batch_dim: int = 0,
                head_dim: int = 1) -> Optional[torch.Tensor]:
    """This rank's view of a (B, H, ...) operand; an axis of extent 1 (broadcast) is kept whole."""
    if x is None:
        return None
    dim = batch_dim if axis == "batch" else head_dim
    n = x.shape[dim]
    if n == 1:
        return x
    lo, hi = bh_partition(n, world_size, rank)
    return x.narrow(dim, lo, hi - lo)


class _AllGatherCat(torch.autograd.Function):
    """all-gather along ``dim``; the gradient of a replicated consumer is this rank's slice."""

    @staticmethod
    def forward(ctx, x, dim, group):
        world = dist.get_world_size(group)
        ctx.dim, ctx.rank, ctx.n = dim, dist.get_rank(group), x.shape[dim]
        moved = x.movedim(dim, 0).contiguous()
        out = torch.empty((world * moved.shape[0], *moved.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, moved, group=group)
        return out.movedim(0, dim)

    @staticmethod
    def backward(ctx, g):
        return g.narrow(ctx.dim, ctx.rank * ctx.n, ctx.n), None, None


def all_gather_output(out_local: torch.Tensor, axis: str, group=None, *, batch_dim: int = 0,
                      head_dim: int = 1) -> torch.Tensor:
    """Replicate the sharded output on every rank (equal shard sizes required)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return out_local
    dim = batch_dim if axis == "batch" else head_dim
    return _AllGatherCat.apply(out_local, dim, group)


def max_over_ranks(value: float, device=None, group=None) -> float:
    """Max of a host scalar over all ranks (timing reduction for multi-GPU measurements)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
