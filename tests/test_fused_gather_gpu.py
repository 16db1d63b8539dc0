"""Fused output all-gather on real GPUs (needs at least two): the forward kernel of each rank stores its output rows
into every rank's copy of the result over NVLink.  Compared with (a) the unsharded call and (b) the NCCL all-gather
of the sharded outputs; gradients of a replicated consumer are compared with the unsharded backward.

Runs as one child process per GPU (NCCL for the rendezvous of the IPC handles and the closing barrier); the kernels
only store into peer memory -- no TMA load, multicast or library kernel is ever given a peer pointer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, axis, dtype_name, D, causal):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from nitrix_b200 import _cabi
        from nitrix_b200 import parallel as P
        from nitrix_b200.nn import attention as att

        dtype = getattr(torch, dtype_name)
        B, H, S, T = 2, 4, 256, 384
        g = torch.Generator().manual_seed(0)          # same operands on every rank
        q = torch.randn(B, H, S, D, generator=g).to(dtype).to(dev)
        k = torch.randn(B, H, T, D, generator=g).to(dtype).to(dev)
        v = torch.randn(B, H, T, D, generator=g).to(dtype).to(dev)
        bias = torch.randn(1, H, S, T, generator=g).to(dtype).to(dev)
        w = torch.randn(B, H, S, D, generator=g).to(dev)
        scale = D ** -0.5

        # unsharded reference on this GPU
        leaves = [x.clone().requires_grad_(True) for x in (q, k, v)]
        whole = att.scaled_dot_product_attention(*leaves, bias=bias, causal=causal, scale=scale)
        gw = torch.autograd.grad((whole.float() * w).sum(), leaves)

        # sharded, output gathered by the forward kernel itself
        rep = P.ReplicatedOutput((B, H, S, D), dtype, dev)
        rep.local.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        loc = [P.local_slice(x, axis, world, rank).clone().requires_grad_(True) for x in (q, k, v)]
        bias_loc = P.local_slice(bias, axis, world, rank)
        full = P.attention_gathered(*loc, rep=rep, axis=axis, bias=bias_loc, causal=causal, scale=scale)
        torch.cuda.synchronize()
        assert _cabi.lib().nb200_device_status(rank) == 0, _cabi.last_error()
        assert not torch.isnan(full.float()).any()                  # every rank's rows arrived
        assert torch.equal(full, whole.detach())                    # same kernels on the same (batch, head) problems
        gl = torch.autograd.grad((full.float() * w).sum(), loc)
        for a, b in zip(gl, gw):
            ref = P.local_slice(b, axis, world, rank)
            assert float((a.float() - ref.float()).abs().max()) <= 2e-2 * max(1.0, float(ref.float().abs().max()))

        # and the NCCL all-gather of the sharded outputs gives the same tensor
        out_loc = att.scaled_dot_product_attention(*[x.detach() for x in loc], bias=bias_loc, causal=causal, scale=scale)
        gathered = P.all_gather_output(out_loc, axis)
        assert torch.equal(gathered, full)
        rep.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("axis,dtype_name,D,causal", [("heads", "bfloat16", 128, True), ("batch", "float16", 64, False)])
def test_fused_all_gather_two_gpus(axis, dtype_name, D, causal):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), axis, dtype_name, D, causal), nprocs=world, join=True)
