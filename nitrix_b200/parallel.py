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


# ---------------------------------------------------------------------------
# fused output all-gather: the forward kernel's epilogue stores into the peers' buffers
# ---------------------------------------------------------------------------
class ReplicatedOutput:
    """One full-size output buffer per rank, each mapped into every other rank's process.

    ``local`` is this rank's ``(B, H, S, Dv)`` buffer; ``peer_ptrs`` are the device addresses of the other ranks'
    buffers in this process (CUDA IPC mappings with peer access over NVLink, made once).  A forward call given
    ``out=`` a slice of ``local`` and ``out_peers=`` the matching addresses in the peers leaves this rank's rows in
    all copies; after :meth:`wait` every copy holds every rank's rows.  No TMA or multicast load ever touches a
    peer buffer: the kernels only STORE into them.
    """

    def __init__(self, shape, dtype, device, group=None):
        import ctypes as C

        from . import _cabi

        if not dist.is_initialized():
            raise RuntimeError("ReplicatedOutput needs an initialised process group")
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.local = torch.empty(shape, dtype=dtype, device=device)
        lib = _cabi.lib()
        mine = _cabi.IpcHandle()
        with torch.cuda.device(device):
            rc = lib.nb200_ipc_export(C.c_void_p(self.local.data_ptr()), C.byref(mine))
        if rc != _cabi.OK:
            raise RuntimeError(f"nb200_ipc_export failed: {_cabi.last_error()}")
        blobs = [None] * self.world
        dist.all_gather_object(blobs, bytes(mine.bytes), group=group)
        self.peer_ptrs = []
        self._opened = []
        with torch.cuda.device(device):
            for r, blob in enumerate(blobs):
                if r == self.rank:
                    continue
                h = _cabi.IpcHandle()
                C.memmove(h.bytes, blob, len(blob))
                ptr = C.c_void_p(0)
                rc = lib.nb200_ipc_open(C.byref(h), C.byref(ptr))
                if rc != _cabi.OK:
                    raise RuntimeError(f"nb200_ipc_open (rank {r}) failed: {_cabi.last_error()}")
                self.peer_ptrs.append(int(ptr.value))
                self._opened.append(int(ptr.value))
        self._flag = torch.zeros(1, dtype=torch.int32, device=device)

    def peers_of(self, view: torch.Tensor):
        """Addresses, in the peers' buffers, of the element where ``view`` (a slice of ``local``) starts."""
        off = view.data_ptr() - self.local.data_ptr()
        return [p + off for p in self.peer_ptrs]

    def wait(self) -> None:
        """Orders the current stream after every rank's forward: a one-element all-reduce enqueued behind this
        rank's kernels completes only when every rank has enqueued (and the device has reached) its own."""
        dist.all_reduce(self._flag, group=self.group)

    def close(self) -> None:
        import ctypes as C

        from . import _cabi

        torch.cuda.synchronize(self.local.device)
        dist.barrier(group=self.group)     # nobody unmaps while a peer may still be storing
        for p in self._opened:
            _cabi.lib().nb200_ipc_close(C.c_void_p(p))
        self._opened = []
        self.peer_ptrs = []


class _GatheredAttention(torch.autograd.Function):
    """Attention on this rank's (batch, head) shard whose output lands, already gathered, in every rank's copy."""

    @staticmethod
    def forward(ctx, q, k, v, bias, mask, scale, causal, rep, dim, lo):
        from .nn import attention as att

        n = q.shape[dim]
        view = rep.local.narrow(dim, lo, n)
        out, lse = att.sdpa_forward(q, k, v, bias, mask, scale=scale, causal=causal, out=view,
                                    out_peers=rep.peers_of(view))
        rep.wait()
        ctx.save_for_backward(q, k, v, bias, mask, out, lse)
        ctx.scale, ctx.causal, ctx.dim, ctx.lo, ctx.n = scale, causal, dim, lo, n
        return rep.local.view(rep.local.shape)     # a fresh alias: autograd attaches this call's graph to it

    @staticmethod
    def backward(ctx, g):
        from .nn import attention as att

        q, k, v, bias, mask, out, lse = ctx.saved_tensors
        g_local = g.narrow(ctx.dim, ctx.lo, ctx.n)      # a replicated consumer: this rank's rows of its cotangent
        want_dbias = bias is not None and ctx.needs_input_grad[3]
        dq, dk, dv, dbias = att.sdpa_backward(q, k, v, bias, mask, out, lse, g_local, scale=ctx.scale,
                                              causal=ctx.causal, want_dbias=want_dbias)
        return dq, dk, dv, dbias, None, None, None, None, None, None


def attention_gathered(q, k, v, *, rep: ReplicatedOutput, axis: str, bias=None, mask=None, scale=None,
                       causal: bool = False) -> torch.Tensor:
    """Attention on this rank's shard ``q, k, v`` (4-D, sliced along ``axis`` with :func:`local_slice`) with the
    output all-gather fused into the forward kernel: returns the full ``(B, H, S, Dv)`` result, identical on every
    rank, without a separate collective over the output.  ``bias`` / ``mask`` are this rank's 4-D slices (extents 1
    or local).  Differentiable: the backward takes this rank's rows of the cotangent."""
    if axis not in ("batch", "heads"):
        raise ValueError(f"attention_gathered: axis must be 'batch' or 'heads', got {axis!r}")
    dim = 0 if axis == "batch" else 1
    full = rep.local.shape[dim]
    lo, hi = bh_partition(full, rep.world, rep.rank)
    if hi - lo != q.shape[dim]:
        raise ValueError(f"attention_gathered: shard has {q.shape[dim]} along {axis}, rank {rep.rank} owns {hi - lo}")
    scale = (q.shape[-1] ** -0.5) if scale is None else float(scale)
    return _GatheredAttention.apply(q, k, v, bias, mask, scale, bool(causal), rep, dim, lo)
