"""Randomised parity of the bf16 / fp16 attention kernels against an fp64 restatement on the device.

Sixty seeded draws of (dtype, batch, heads, S, T, head dim 64 / 128, causal, bias shape, mask shape, bias gradient)
with lengths the reference's callers have (28, 111, 197, 217, 344 tokens) next to multiples of the 128-wide tiles:
the tcgen05 forward, the one-kernel backwards, the query- / key-major pair, broadcast-bias gradients, staged
operands.  out and every gradient within 3e-2 (bf16) / 6e-3 (fp16) of max |reference| -- an output ulp of the
16-bit storage plus the fp32 accumulation.
"""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(60))
def test_random_sixteen_bit_problem_matches_fp64(seed):
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import attention as att

    rng = random.Random(1000 + seed)
    dt = rng.choice([torch.bfloat16, torch.float16])
    B, H = rng.choice([1, 2, 3]), rng.choice([1, 2, 4])
    S = rng.choice([28, 64, 111, 128, 197, 200, 217, 256, 344, 512, 640, 1000, 1024])
    T = rng.choice([28, 64, 111, 128, 197, 200, 217, 256, 344, 512, 640, 1000, 1024, 1500])
    D = rng.choice([64, 128])
    causal = (rng.random() < 0.3 and S == T) or rng.random() < 0.1
    bias_shape = rng.choice([None, None, (B, H, S, T), (1, H, S, T), (B, 1, S, T), (1, 1, 1, T), (1, H, 1, T)])
    mask_shape = rng.choice([None, None, None, (B, H, S, T), (B, 1, 1, T), (1, 1, S, T), (B, 1, S, T)])
    want_dbias = bias_shape is not None and rng.random() < 0.6
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, H, S, D, device="cuda", generator=g).to(dt)
    k = torch.randn(B, H, T, D, device="cuda", generator=g).to(dt)
    v = torch.randn(B, H, T, D, device="cuda", generator=g).to(dt)
    dout = torch.randn(B, H, S, D, device="cuda", generator=g).to(dt)
    bias = None if bias_shape is None else torch.randn(bias_shape, device="cuda", generator=g).to(dt)
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
    grads = torch.autograd.grad(ref, [qd, kd, vd] + ([bd] if want_dbias else []), grad_outputs=dout.double())
    tol = 3e-2 if dt == torch.bfloat16 else 6e-3
    err = float((out.double() - ref.detach()).abs().max() / ref.detach().abs().max())
    assert err <= tol, ("out", err)
    for name, a, r in zip(("dq", "dk", "dv", "dbias"), [dq, dk, dv] + ([db] if want_dbias else []), grads):
        err = float((a.double() - r.reshape(a.shape)).abs().max() / r.abs().max())
        assert err <= tol, (name, err, (dt, B, H, S, T, D, causal, bias_shape, mask_shape))
