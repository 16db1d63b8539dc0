"""``nitrix.nn.selective_scan`` on the B200 library: the reference's dispatcher surface over the CUDA kernels.

Mirrors the reference's public function (``src/nitrix/nn/ssm/__init__.py:127-``): the same operands --
``x, delta (..., l, d)``, ``A (d, n)``, ``B, C (..., l, n)``, optional ``D (d,)`` -- the same ``ValueError`` texts of
its ``_validate`` (``:40-77``), and the recipe of ``reference_selective_scan``
(``src/nitrix/nn/ssm/_reference.py:60-98``): ``h_t = exp(delta_t A) h_{t-1} + (delta_t B_t) x_t``,
``y_t = sum_n C_{t,n} h_{t,n} (+ D x_t)``, fp32 recurrence for any storage dtype.  Forward and backward run the
library's kernels (``nb200_selective_scan_fwd`` / ``_bwd``); there is no host path.  The reference's ``driver``
argument chooses among XLA formulations of the same recurrence and has no counterpart here.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _cabi
from ..backend import resolve_backend

__all__ = ["selective_scan"]

_DTYPES = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


def _validate(x, delta, A, B, C_, D) -> None:
    """Same checks and texts as the reference's ``_validate`` (``nn/ssm/__init__.py:40-77``)."""
    if x.shape != delta.shape:
        raise ValueError(f"selective_scan: x and delta must match; got x.shape={tuple(x.shape)}, "
                         f"delta.shape={tuple(delta.shape)}.")
    if x.dim() < 2:
        raise ValueError(f"selective_scan: x must be at least (l, d); got ndim {x.dim()}.")
    d, length = x.shape[-1], x.shape[-2]
    if A.dim() != 2 or A.shape[0] != d:
        raise ValueError(f"selective_scan: A must be (d, n) with d={d}; got A.shape={tuple(A.shape)}.")
    n = A.shape[1]
    if B.shape[-1] != n or C_.shape[-1] != n:
        raise ValueError(f"selective_scan: B/C last dim must be n={n}; got B.shape={tuple(B.shape)}, "
                         f"C.shape={tuple(C_.shape)}.")
    if B.shape[-2] != length or C_.shape[-2] != length:
        raise ValueError(f"selective_scan: B/C sequence dim must be l={length}; got "
                         f"B.shape={tuple(B.shape)}, C.shape={tuple(C_.shape)}.")
    if D is not None and tuple(D.shape) != (d,):
        raise ValueError(f"selective_scan: D must be (d,) with d={d}; got D.shape={tuple(D.shape)}.")


def _check(rc: int, what: str) -> None:
    if rc != _cabi.OK:
        raise RuntimeError(f"{what} failed (status {rc}): {_cabi.last_error()}")


def _params(x3, A) -> "_cabi.SelectiveScanParams":
    p = _cabi.SelectiveScanParams()
    p.struct_size = C.sizeof(_cabi.SelectiveScanParams)
    p.batch, p.length, p.channels, p.states = x3.shape[0], x3.shape[1], x3.shape[2], A.shape[1]
    p.dtype = _DTYPES[x3.dtype]
    return p


def _bytes(fn, p) -> int:
    need = C.c_size_t(0)
    _check(fn(C.byref(p), C.byref(need)), fn.__name__)
    return int(need.value)


def selective_scan_forward(x3, delta3, A, B3, C3, D, want_checkpoints: bool):
    """Enqueue the forward on the current stream: ``(y, checkpoints_or_None)`` for dense 3-D operands."""
    y = torch.empty_like(x3)
    p = _params(x3, A)
    p.x, p.delta, p.A, p.B, p.C, p.y = (t.data_ptr() for t in (x3, delta3, A, B3, C3, y))
    p.D = None if D is None else D.data_ptr()
    ck = None
    if want_checkpoints:
        n = _bytes(_cabi.lib().nb200_selective_scan_checkpoint_bytes, p)
        ck = torch.empty(max(n // 4, 1), dtype=torch.float32, device=x3.device)
        p.checkpoints = ck.data_ptr()
    with torch.cuda.device(x3.device):
        _check(_cabi.lib().nb200_selective_scan_fwd(C.byref(p), torch.cuda.current_stream().cuda_stream),
               "nb200_selective_scan_fwd")
    return y, ck


def selective_scan_backward(x3, delta3, A, B3, C3, D, ck, dy3):
    """Enqueue the backward on the current stream: ``(dx, ddelta, dA, dB, dC, dD_or_None)``."""
    p = _params(x3, A)
    dx, ddelta = torch.empty_like(x3), torch.empty_like(x3)
    dA, dB, dC = torch.empty_like(A), torch.empty_like(B3), torch.empty_like(C3)
    dD = None if D is None else torch.empty_like(D)
    p.x, p.delta, p.A, p.B, p.C, p.dy = (t.data_ptr() for t in (x3, delta3, A, B3, C3, dy3))
    p.D = None if D is None else D.data_ptr()
    p.checkpoints = None if ck is None else ck.data_ptr()
    p.dx, p.ddelta, p.dA, p.dB, p.dC = (t.data_ptr() for t in (dx, ddelta, dA, dB, dC))
    p.dD = None if dD is None else dD.data_ptr()
    need = _bytes(_cabi.lib().nb200_selective_scan_workspace_bytes, p)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=x3.device)
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    with torch.cuda.device(x3.device):
        _check(_cabi.lib().nb200_selective_scan_bwd(C.byref(p), torch.cuda.current_stream().cuda_stream),
               "nb200_selective_scan_bwd")
    return dx, ddelta, dA, dB, dC, dD


class _SelectiveScan(torch.autograd.Function):
    """The differentiation rule of the fused op: saves the operands and the forward's checkpoints."""

    @staticmethod
    def forward(ctx, x, delta, A, B, C_, D):
        dt = x.dtype
        lead = x.shape[:-2]
        x3 = x.reshape((-1,) + tuple(x.shape[-2:])).contiguous()
        delta3 = delta.to(dt).reshape(x3.shape).contiguous()
        B3 = B.to(dt).expand(lead + tuple(B.shape[-2:])).reshape((-1,) + tuple(B.shape[-2:])).contiguous()
        C3 = C_.to(dt).expand(lead + tuple(C_.shape[-2:])).reshape((-1,) + tuple(C_.shape[-2:])).contiguous()
        A2 = A.to(dt).contiguous()
        D1 = None if D is None else D.to(dt).contiguous()
        need_grad = any(ctx.needs_input_grad)
        y, ck = selective_scan_forward(x3, delta3, A2, B3, C3, D1, need_grad)
        ctx.save_for_backward(x3, delta3, A2, B3, C3, D1 if D1 is not None else x3.new_empty(0),
                              ck if ck is not None else x3.new_empty(0, dtype=torch.float32))
        ctx.has_D = D is not None
        ctx.shapes = (x.shape, delta.shape, B.shape, C_.shape)
        ctx.dtypes = (delta.dtype, A.dtype, B.dtype, C_.dtype, None if D is None else D.dtype)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x3, delta3, A2, B3, C3, D1, ck = ctx.saved_tensors
        dy3 = dy.to(x3.dtype).reshape(x3.shape).contiguous()
        dx, ddelta, dA, dB, dC, dD = selective_scan_backward(x3, delta3, A2, B3, C3, D1 if ctx.has_D else None,
                                                              ck if ck.numel() else None, dy3)
        xs, ds, bs, cs = ctx.shapes
        lead = xs[:-2]

        def back_to(g3, shape):   # gradient of an operand that was broadcast over the leading axes
            g = g3.reshape(lead + tuple(g3.shape[-2:]))
            while g.dim() > len(shape):
                g = g.sum(0)
            for ax, extent in enumerate(shape):
                if extent == 1 and g.shape[ax] != 1:
                    g = g.sum(ax, keepdim=True)
            return g

        dl_t, a_t, b_t, c_t, d_t = ctx.dtypes
        return (dx.reshape(xs), ddelta.reshape(ds).to(dl_t), dA.to(a_t), back_to(dB, bs).to(b_t),
                back_to(dC, cs).to(c_t), None if dD is None else dD.to(d_t))


def selective_scan(x: torch.Tensor, delta: torch.Tensor, A: torch.Tensor, B: torch.Tensor, C: torch.Tensor,  # noqa: N803
                   D: Optional[torch.Tensor] = None, *, backend: str = "auto") -> torch.Tensor:
    """Mamba / S6 selective scan (reference ``nn/ssm/__init__.py:127-``): ``x, delta (..., l, d)``, ``A (d, n)``,
    ``B, C (..., l, n)``, optional ``D (d,)``; returns ``(..., l, d)`` in ``x``'s dtype.  CUDA tensors of fp32, bf16
    or fp16; at most 64 states per channel.  Differentiable in every operand."""
    _validate(x, delta, A, B, C, D)
    resolve_backend(backend)   # raises without a Blackwell device: there is no host path
    if not x.is_cuda or x.dtype not in _DTYPES:
        raise TypeError(f"selective_scan: x must be a CUDA tensor of float32, bfloat16 or float16; got {x.dtype} on {x.device}")
    if A.shape[1] > 64:
        raise ValueError(f"selective_scan: at most 64 states per channel are supported; got n={A.shape[1]}.")
    if x.numel() == 0:
        return torch.empty_like(x)
    return _SelectiveScan.apply(x, delta, A, B, C, D)
