"""Randomised parity of the fp32 attention kernels against an fp64 restatement on the device.

Eighty seeded draws of (batch, heads, S, T, head dims, causal, bias shape, mask shape, bias gradient) in the size
range where the library picks among the plain 3 x TF32 kernels, the in-CTA warp-group splits and the cluster splits
(forward, dq, dk/dv), with lengths on and off the 64-wide tiles.  out and every gradient within the fp32 budget of
1e-4 of max |reference|.  Draws whose rows keep exactly one key are skipped: their dq and dk are exactly zero in
the reference, which leaves nothing to divide by.
"""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

FP32_REL = 1e-4


def _draw(rng):
    B, H = rng.choice([1, 2, 3]), rng.choice([1, 2, 4, 6])
    S = rng.choice([7, 63, 64, 65, 100, 128, 150, 200, 256, 257, 300, 344, 400, 512, 520])
    T = rng.choice([5, 64, 65, 100, 128, 130, 193, 200, 256, 257, 320, 344, 384, 512, 520, 600])
    D = rng.choice([32, 64])
    Dv = rng.choice([D, D, D, 32, 64])
    causal = (rng.random() < 0.3 and S == T) or rng.random() < 0.15
    bias_shape = rng.choice([None, None, (B, H, S, T), (1, H, S, T), (B, 1, S, T), (1, 1, 1, T), (1, H, 1, T)])
    mask_shape = rng.choice([None, None, None, (B, H, S, T), (B, 1, 1, T), (1, 1, S, T), (B, 1, S, T)])
    want_dbias = bias_shape is not None and rng.random() < 0.6
    return B, H, S, T, D, Dv, causal, bias_shape, mask_shape, want_dbias


@pytest.mark.parametrize("seed", range(80))
def test_random_fp32_problem_matches_fp64(seed):
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import attention as att

    rng = random.Random(seed)
    B, H, S, T, D, Dv, causal, bias_shape, mask_shape, want_dbias = _draw(rng)
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, S, D, device="cuda", generator=g)
    k = torch.randn(B, H, T, D, device="cuda", generator=g)
    v = torch.randn(B, H, T, Dv, device="cuda", generator=g)
    dout = torch.randn(B, H, S, Dv, device="cuda", generator=g)
    bias = None if bias_shape is None else torch.randn(bias_shape, device="cuda", generator=g)
    mask = None
    if mask_shape is not None:
        mask = torch.rand(mask_shape, device="cuda", generator=g) > 0.2
        mask[..., 0] = True                      # every row keeps key 0 (also under causal): no empty rows here
    scale = D ** -0.5
    out, lse = att.sdpa_forward(q, k, v, bias, mask, scale=scale, causal=causal)
    dq, dk, dv, db = att.sdpa_backward(q, k, v, bias, mask, out, lse, dout, scale=scale, causal=causal,
                                       want_dbias=want_dbias)
    torch.cuda.synchronize()
    assert _cabi.lib().nb200_device_status(0) == 0, _cabi.last_error()

    qd, kd, vd = (x.double().requires_grad_() for x in (q, k, v))
    bd = None if bias is None else bias.double().requires_grad_()
    s = qd @ kd.transpose(-1, -2) * scale
    if bd is not None:
        s = s + bd
    keep = torch.ones(S, T, dtype=torch.bool, device="cuda")
    if causal:
        keep = keep & torch.tril(keep)
    if mask is not None:
        keep = keep & mask
    ref = torch.softmax(s.masked_fill(~keep, float("-inf")), -1) @ vd
    leaves = [qd, kd, vd] + ([bd] if want_dbias else [])
    grads = torch.autograd.grad(ref, leaves, grad_outputs=dout.double())
    got = [dq, dk, dv] + ([db] if want_dbias else [])
    names = ["dq", "dk", "dv", "dbias"]
    err = float((out.double() - ref.detach()).abs().max() / ref.detach().abs().max())
    assert err <= FP32_REL, ("out", err)
    for name, a, r in zip(names, got, grads):
        err = float((a.double() - r.reshape(a.shape)).abs().max() / r.abs().max())
        assert err <= FP32_REL, (name, err, (B, H, S, T, D, Dv, causal, bias_shape, mask_shape))
