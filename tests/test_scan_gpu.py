"""Selective scan on the GPU against the restated recipe: forward and every gradient, through the C ABI.

The comparison runs the recipe in fp64 on the same (quantised) operands on the device and differentiates it with
autograd, as the reference differentiates its own recipe.  fp32 within 2e-5 of max |reference|; 16-bit within an
output ulp of the storage dtype plus that.  Shapes cover every state-count instantiation (up to 16, 32, 64), lengths
on and off the eight-step chunks, a channel count that does not fill the last CTA, leading batch axes, B and C shared
over the batch, and the optional D.
"""
import pathlib

import numpy as np
import pytest
import torch

from oracle import scan_oracle as S

pytestmark = pytest.mark.gpu


def _operands(lead, length, d, n, dtype, with_d, seed, shared_bc=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(lead + (length, d), device="cuda", generator=g)
    delta = torch.rand(lead + (length, d), device="cuda", generator=g) * 0.5 + 0.01
    A = -(torch.rand(d, n, device="cuda", generator=g) * 1.5 + 0.2)
    bc_lead = () if shared_bc else lead
    B = torch.randn(bc_lead + (length, n), device="cuda", generator=g)
    C = torch.randn(bc_lead + (length, n), device="cuda", generator=g)
    D = torch.randn(d, device="cuda", generator=g) if with_d else None
    dy = torch.randn(lead + (length, d), device="cuda", generator=g)
    return [None if t is None else t.to(dtype) for t in (x, delta, A, B, C, D, dy)]


def _run(lead, length, d, n, dtype, with_d=True, seed=0, shared_bc=False):
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import ssm

    x, delta, A, B, C, D, dy = _operands(lead, length, d, n, dtype, with_d, seed, shared_bc)
    leaves = [t.detach().clone().requires_grad_(True) for t in (x, delta, A, B, C) + ((D,) if with_d else ())]
    y = ssm.selective_scan(*leaves[:5], leaves[5] if with_d else None)
    grads = torch.autograd.grad(y, leaves, grad_outputs=dy)
    torch.cuda.synchronize()
    assert _cabi.lib().nb200_device_status(0) == 0, _cabi.last_error()
    ref_leaves = [t.detach().double().requires_grad_(True) for t in (x, delta, A, B, C) + ((D,) if with_d else ())]
    want = S.selective_scan_torch(*ref_leaves[:5], ref_leaves[5] if with_d else None)
    ref_grads = torch.autograd.grad(want, ref_leaves, grad_outputs=dy.double())
    tol = 2e-5 if dtype == torch.float32 else (1.5e-2 if dtype == torch.bfloat16 else 2e-3)
    assert y.dtype == dtype and y.shape == x.shape
    err = float((y.detach().double() - want.detach()).abs().max() / want.detach().abs().max())
    assert err <= tol, ("y", err)
    for name, a, r in zip(("dx", "ddelta", "dA", "dB", "dC", "dD"), grads, ref_grads):
        assert a.dtype == dtype and a.shape == r.shape, name
        err = float((a.double() - r).abs().max() / r.abs().max().clamp_min(1e-6))   # (dA is exactly 0 at length 1)
        assert err <= tol, (name, err)


def test_reference_golden_vector_on_the_gpu():
    from nitrix_b200.nn import ssm

    z = np.load(pathlib.Path(__file__).resolve().parent / "golden" / "selective_scan_float32.npz")
    y = ssm.selective_scan(*(torch.from_numpy(z[k]).cuda() for k in ("x", "delta", "A", "B", "C", "D")))
    np.testing.assert_allclose(y.cpu().numpy(), z["out"], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("length,d,n", [(1, 8, 4), (8, 64, 16), (37, 100, 16), (64, 200, 3), (129, 96, 32),
                                        (50, 70, 64), (256, 256, 16)])
def test_forward_and_gradients(length, d, n, dtype):
    _run((2,), length, d, n, dtype)


def test_without_the_skip_term_and_with_leading_axes():
    _run((2, 3), 40, 48, 8, torch.float32, with_d=False)
    _run((), 33, 130, 16, torch.float32, with_d=True)


def test_projections_shared_over_the_batch_get_summed_gradients():
    _run((3,), 29, 72, 16, torch.float32, shared_bc=True)
