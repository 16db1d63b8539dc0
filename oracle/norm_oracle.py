"""CPU restatement of the reference's LayerNorm recipe -- TEST INFRASTRUCTURE ONLY.

Only ``tests/`` may import this module: it is the checker the CUDA kernels are compared with, never a code path of
the library.  It follows ``reference_layer_norm`` (reference ``src/nitrix/nn/norm/_reference.py:88-110``) step by
step in numpy: accumulation dtype = promote(input dtype, float32); mean and BIASED variance over the trailing axis;
``x_hat = (x - mean) * rsqrt(var + eps)``; ``* weight`` and ``+ bias`` in the accumulation dtype when given; times
``out_scale``; cast back to the input dtype.  Pinned by ``tests/test_norm_oracle_golden.py`` against the reference's
own stored vector ``tests/golden/layer_norm_float32.npz`` (x, weight, bias, out with ``out_scale = 0.5``;
reference ``tests/test_nn_norm.py:51-62``).

``layer_norm_grads`` gives the gradients autodiff derives from that recipe, in closed form, in float64; the test file
checks the closed form against finite differences of the forward (the reference has no stored gradient vectors:
``tests/test_nn_norm.py:183-210`` checks its autodiff against finite differences the same way).
"""
from __future__ import annotations

import numpy as np


def layer_norm(x, weight=None, bias=None, *, eps=1e-5, out_scale=1.0, acc_dtype=None):
    """``reference_layer_norm`` (``_reference.py:88-110``).  ``x``: ndarray (..., c); returns the same dtype."""
    io_dtype = x.dtype
    acc = np.dtype(acc_dtype or np.promote_types(io_dtype, np.float32))          # :95-98
    xa = x.astype(acc)
    mean = xa.mean(axis=-1, keepdims=True)                                       # :99
    var = ((xa - mean) ** 2).mean(axis=-1, keepdims=True)                        # :100 (jnp.var: biased, about the mean)
    x_hat = (xa - mean) / np.sqrt(var + acc.type(eps))                           # :101
    if weight is not None:
        x_hat = x_hat * weight.astype(acc)                                       # :102-103
    if bias is not None:
        x_hat = x_hat + bias.astype(acc)                                         # :104-105
    return (acc.type(out_scale) * x_hat).astype(io_dtype)                        # :106-107


def layer_norm_grads(x, weight, dy, *, eps=1e-5, out_scale=1.0):
    """(dx, dweight, dbias) of ``sum(layer_norm(x, weight, bias) * dy)`` in float64 (closed form)."""
    x = x.astype(np.float64)
    dy = dy.astype(np.float64)
    c = x.shape[-1]
    w = np.ones(c) if weight is None else weight.astype(np.float64)
    mean = x.mean(-1, keepdims=True)
    var = ((x - mean) ** 2).mean(-1, keepdims=True)
    rstd = 1.0 / np.sqrt(var + eps)
    xh = (x - mean) * rstd
    gy = out_scale * dy
    dxh = gy * w
    dx = rstd * (dxh - dxh.mean(-1, keepdims=True) - xh * (dxh * xh).mean(-1, keepdims=True))
    axes = tuple(range(x.ndim - 1))
    return dx, (gy * xh).sum(axes), gy.sum(axes)
