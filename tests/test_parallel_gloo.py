"""Multi-rank host logic on CPU ranks (gloo, world size 2): the batch x heads partition, the optional
output all-gather with its gradient, and the max-over-ranks timing reduction.  No kernel runs here."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, axis):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nitrix_b200 import parallel as P

        B, H, S, D = 4, 6, 5, 3
        full = torch.arange(B * H * S * D, dtype=torch.float32).reshape(B, H, S, D)
        local = P.local_slice(full, axis, world, rank).clone().requires_grad_(True)
        assert local.shape[0 if axis == "batch" else 1] == (B if axis == "batch" else H) // world
        # a broadcast operand (extent 1 on the sharded axis) is kept whole
        shared = torch.zeros(1, 1, S, S)
        assert P.local_slice(shared, axis, world, rank) is shared
        # stand-in for the kernels: out_local = 2 * local; gather replicates it on every rank
        gathered = P.all_gather_output(local * 2, axis)
        assert torch.equal(gathered, full * 2)
        # replicated consumer: every rank differentiates the same loss; its gradient is the local slice
        w = torch.arange(gathered.numel(), dtype=torch.float32).reshape(gathered.shape)
        (gathered * w).sum().backward()
        assert torch.equal(local.grad, 2 * P.local_slice(w, axis, world, rank))
        assert P.max_over_ranks(float(rank + 1)) == float(world)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("axis", ["batch", "heads"])
def test_partition_and_gather_two_ranks(axis):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), axis), nprocs=world, join=True)
