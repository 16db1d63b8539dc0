"""CPU restatement of the reference's selective-scan recipe -- TEST INFRASTRUCTURE ONLY.

Only ``tests/`` may import this module.  It follows ``reference_selective_scan`` with the canonical sequential driver
(reference ``src/nitrix/nn/ssm/_reference.py``): accumulation dtype = promote(result dtype of the operands, float32)
(:262-279); ``dA = exp(delta[..., None] * A)``, ``dBx = delta[..., None] * B[..., None, :] * x[..., None]`` (:60-69);
``h_t = dA_t * h_{t-1} + dBx_t`` from ``h = 0`` (:84-98); ``y = (H * C[..., None, :]).sum(-1) (+ D * x)`` (:72-81); cast
back.  Pinned by ``tests/test_scan_oracle_golden.py`` against the reference's own stored vector
``tests/golden/selective_scan_float32.npz`` (reference ``tests/test_nn_ssm.py:69-83``).

``selective_scan_torch`` is the same recipe on torch tensors (any device, any float dtype); autograd through it
gives the gradients the GPU tests compare with -- the reference differentiates its recipe the same way
(``_reference.py:24-25``: "Differentiated by ordinary XLA autodiff").
"""
from __future__ import annotations

import numpy as np


def selective_scan(x, delta, A, B, C, D=None):
    """numpy, sequential; ``x, delta (..., l, d)``, ``A (d, n)``, ``B, C (..., l, n)``, ``D (d,)`` or None."""
    io = np.result_type(x, delta, A, B, C) if D is None else np.result_type(x, delta, A, B, C, D)
    acc = np.promote_types(io, np.float32)
    x, delta, A, B, C = (a.astype(acc) for a in (x, delta, A, B, C))
    dA = np.exp(delta[..., None] * A)                                   # (..., l, d, n)
    dBx = delta[..., None] * B[..., None, :] * x[..., None]
    h = np.zeros(dA.shape[:-3] + dA.shape[-2:], dtype=acc)
    ys = []
    for t in range(x.shape[-2]):
        h = dA[..., t, :, :] * h + dBx[..., t, :, :]
        ys.append((h * C[..., t, None, :]).sum(-1))
    y = np.stack(ys, axis=-2) if ys else np.zeros_like(x)
    if D is not None:
        y = y + D.astype(acc) * x
    return y.astype(io)


def selective_scan_torch(x, delta, A, B, C, D=None):
    """The same recipe on torch tensors; differentiable."""
    import torch

    dA = torch.exp(delta[..., None] * A)
    dBx = delta[..., None] * B[..., None, :] * x[..., None]
    h = torch.zeros(dA.shape[:-3] + dA.shape[-2:], dtype=x.dtype, device=x.device)
    ys = []
    for t in range(x.shape[-2]):
        h = dA[..., t, :, :] * h + dBx[..., t, :, :]
        ys.append((h * C[..., t, None, :]).sum(-1))
    y = torch.stack(ys, dim=-2)
    if D is not None:
        y = y + D * x
    return y
