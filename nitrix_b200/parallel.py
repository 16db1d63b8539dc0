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
    if axis not in ("batch", "heads"):
        raise ValueError(f"local_slice: axis must be 'batch' or 'heads', got {axis!r} (a flattened 'pairs' split is "
                         "expressed with bh_begin / bh_end on the whole tensors)")
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
    """Replicate the sharded output on every rank.

    ``axis`` is ``'batch'`` or ``'heads'`` and every rank must hold a shard of the same size along it (the
    flattened ``'pairs'`` split of :func:`shard_axis` has no tensor axis to gather along: slice with
    ``bh_begin`` / ``bh_end`` on a full-size buffer instead).  A bias that is broadcast over the sharded axis is
    held whole by every rank, so its gradient is a partial sum per rank: the caller adds them with
    ``torch.distributed.all_reduce`` (see :func:`all_reduce_shared_bias_grad`)."""
    if axis not in ("batch", "heads"):
        raise ValueError(f"all_gather_output: axis must be 'batch' or 'heads', got {axis!r}")
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return out_local
    dim = batch_dim if axis == "batch" else head_dim
    sizes = torch.tensor([out_local.shape[dim]], dtype=torch.int64, device=out_local.device)
    lo, hi = sizes.clone(), sizes.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=group)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=group)
    if int(lo) != int(hi):
        raise ValueError(f"all_gather_output: shards differ in size along {axis} ({int(lo)}..{int(hi)}); "
                         "pad the axis or use bh_begin / bh_end on a shared full-size buffer")
    return _AllGatherCat.apply(out_local, dim, group)


def all_reduce_shared_bias_grad(dbias: torch.Tensor, group=None) -> torch.Tensor:
    """Sum, over ranks, the gradient of a bias that every rank holds whole because it is broadcast over the
    sharded axis (each rank's kernels saw only its own (batch, head) pairs).  In place; returns ``dbias``."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(dbias, op=dist.ReduceOp.SUM, group=group)
    return dbias


def max_over_ranks(value: float, device=None, group=None) -> float:
    """Max of a host scalar over all ranks (timing reduction for multi-GPU measurements)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
