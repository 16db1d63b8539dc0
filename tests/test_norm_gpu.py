"""Fused LayerNorm on the GPU against the CPU oracle: forward and all gradients, through the C ABI.

fp32 within 2e-5 of max |reference| (the reductions run in fp32 on both sides; the orders of summation differ),
16-bit within half an output ulp of the fp32 recipe plus that.  Shapes cover both row mappings of the vector
kernels (one warp / one CTA per row), every per-thread chunk count, partial last chunks, and the scalar kernels
(channels not a multiple of 16 bytes, more than 8192 channels, an unaligned view).
"""
import numpy as np
import pytest
import torch

from oracle import norm_oracle as N

pytestmark = pytest.mark.gpu


def _run(shape, dtype, weight=True, bias=True, out_scale=0.5, eps=1e-5, seed=0, view=None):
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import norm

    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(shape, generator=g) * 1.5 + 0.3).to(dtype)
    dy = torch.randn(shape, generator=g).to(dtype)
    xd = x.cuda()
    if view is not None:
        xd = view(xd)
        x, dy = view(x), view(dy)
    c = x.shape[-1]
    w = (torch.randn(c, generator=g) * 0.5 + 1.0).to(dtype) if weight else None
    b = (torch.randn(c, generator=g) * 0.5).to(dtype) if bias else None
    xd = xd.detach().requires_grad_(True)
    wd = None if w is None else w.cuda().requires_grad_(True)
    bd = None if b is None else b.cuda().requires_grad_(True)
    y = norm.layer_norm(xd, wd, bd, eps=eps, out_scale=out_scale)
    leaves = [t for t in (xd, wd, bd) if t is not None]
    grads = list(torch.autograd.grad(y, leaves, grad_outputs=dy.cuda()))
    torch.cuda.synchronize()
    assert _cabi.lib().nb200_device_status(0) == 0
    xf = x.float().numpy()
    want = N.layer_norm(xf, None if w is None else w.float().numpy(), None if b is None else b.float().numpy(),
                        eps=eps, out_scale=out_scale)
    rdx, rdw, rdb = N.layer_norm_grads(xf, None if w is None else w.float().numpy(), dy.float().numpy(), eps=eps,
                                       out_scale=out_scale)
    refs = [rdx] + ([rdw] if w is not None else []) + ([rdb] if b is not None else [])
    tol = 2e-5 if dtype == torch.float32 else (1e-2 if dtype == torch.bfloat16 else 2e-3)
    assert y.dtype == dtype and y.shape == x.shape
    err = float(np.abs(y.detach().float().cpu().numpy() - want).max() / np.abs(want).max())
    assert err <= tol, ("y", err)
    for name, a, r in zip(("dx", "dweight", "dbias"), grads, refs):
        assert a.dtype == dtype
        err = float(np.abs(a.float().cpu().numpy().astype(np.float64) - r).max() / np.abs(r).max())
        assert err <= tol, (name, err)


def test_reference_golden_vector_on_the_gpu():
    import pathlib

    from nitrix_b200.nn import norm

    z = np.load(pathlib.Path(__file__).resolve().parent / "golden" / "layer_norm_float32.npz")
    y = norm.layer_norm(torch.from_numpy(z["x"]).cuda(), torch.from_numpy(z["weight"]).cuda(),
                        torch.from_numpy(z["bias"]).cuda(), out_scale=0.5)
    np.testing.assert_allclose(y.cpu().numpy(), z["out"], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("c", [8, 64, 200, 256, 520, 1024, 2048, 4096, 8192])
def test_vector_kernels_every_row_mapping(c, dtype):
    _run((3, 37, c), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("c", [5, 30, 515, 8200, 12000])
def test_scalar_kernels_take_every_other_row_length(c, dtype):
    _run((2, 9, c), dtype)


@pytest.mark.parametrize("weight,bias", [(False, False), (True, False), (False, True)])
def test_optional_affine_parameters(weight, bias):
    _run((4, 33, 768), torch.bfloat16, weight=weight, bias=bias, out_scale=1.0)
    _run((4, 33, 768), torch.float32, weight=weight, bias=bias, out_scale=2.5, eps=1e-3)


def test_a_strided_view_and_many_rows():
    _run((4, 50, 260), torch.float32, view=lambda t: t[..., 1:257])          # a strided view: the host layer hands over a dense copy
    _run((64, 1024, 128), torch.bfloat16)                                     # 65536 rows: grid-stride column sums


def test_dweight_is_summed_in_a_fixed_order():
    from nitrix_b200.nn import norm

    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(4096, 1024, device="cuda", generator=g, dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(1024, device="cuda", generator=g, dtype=torch.bfloat16, requires_grad=True)
    dy = torch.randn(4096, 1024, device="cuda", generator=g, dtype=torch.bfloat16)
    outs = []
    for _ in range(3):
        y = norm.layer_norm(x, w, None)
        outs.append(torch.autograd.grad(y, [x, w], grad_outputs=dy))
    for a in outs[1:]:
        assert torch.equal(a[0], outs[0][0]) and torch.equal(a[1], outs[0][1])


def test_empty_input():
    from nitrix_b200.nn import norm

    y = norm.layer_norm(torch.empty(0, 64, device="cuda"), torch.ones(64, device="cuda"))
    assert y.shape == (0, 64)
