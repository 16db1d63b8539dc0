"""``nitrix.nn.layer_norm`` on the B200 library: the reference's dispatcher surface over the fused CUDA kernels.

Mirrors the reference's public function (``src/nitrix/nn/norm/__init__.py:110-176``): same arguments, the same
``ValueError`` for a mis-shaped ``weight`` / ``bias`` (``:44-54``), normalisation over the trailing axis with the
biased variance, the optional affine transform and the ``out_scale`` hook (``src/nitrix/nn/norm/_reference.py:88-110``).
Where the reference's fused module declines every shape and its dispatcher falls back to XLA, this one always runs
the library's kernels -- forward and backward (``nb200_layer_norm_fwd`` / ``nb200_layer_norm_bwd``) -- and there is
no host path: without a CUDA device or without the built library the call raises.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import _cabi
from ..backend import resolve_backend

__all__ = ["layer_norm"]

_DTYPES = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}


def _check_affine(name: str, weight, bias, channels: int) -> None:
    """Same text as the reference's check (``nn/norm/__init__.py:44-54``)."""
    for label, p in (("weight", weight), ("bias", bias)):
        if p is not None and tuple(p.shape) != (channels,):
            raise ValueError(f"{name}: {label} must have shape ({channels},); got {tuple(p.shape)}.")


def _check(rc: int, what: str) -> None:
    if rc != _cabi.OK:
        raise RuntimeError(f"{what} failed (status {rc}): {_cabi.last_error()}")


def _params(x2: torch.Tensor, eps: float, out_scale: float) -> "_cabi.LayerNormParams":
    p = _cabi.LayerNormParams()
    p.struct_size = C.sizeof(_cabi.LayerNormParams)
    p.rows, p.channels = x2.shape[0], x2.shape[1]
    p.dtype = _DTYPES[x2.dtype]
    p.eps, p.out_scale = float(eps), float(out_scale)
    p.x = x2.data_ptr()
    return p


def layer_norm_forward(x2: torch.Tensor, weight, bias, eps: float, out_scale: float):
    """Enqueue the forward on the current stream: ``(y, mean, rstd)`` for dense ``x2`` of shape (rows, channels)."""
    y = torch.empty_like(x2)
    mean = torch.empty(x2.shape[0], dtype=torch.float32, device=x2.device)
    rstd = torch.empty_like(mean)
    p = _params(x2, eps, out_scale)
    p.weight = None if weight is None else weight.data_ptr()
    p.bias = None if bias is None else bias.data_ptr()
    p.y, p.mean, p.rstd = y.data_ptr(), mean.data_ptr(), rstd.data_ptr()
    with torch.cuda.device(x2.device):
        _check(_cabi.lib().nb200_layer_norm_fwd(C.byref(p), torch.cuda.current_stream().cuda_stream),
               "nb200_layer_norm_fwd")
    return y, mean, rstd


def layer_norm_backward(x2, weight, dy2, mean, rstd, eps: float, out_scale: float, want_weight: bool, want_bias: bool):
    """Enqueue the backward on the current stream: ``(dx, dweight_or_None, dbias_or_None)``."""
    dx = torch.empty_like(x2)
    p = _params(x2, eps, out_scale)
    p.weight = None if weight is None else weight.data_ptr()
    p.dy, p.dx, p.mean, p.rstd = dy2.data_ptr(), dx.data_ptr(), mean.data_ptr(), rstd.data_ptr()
    dw = torch.empty(x2.shape[1], dtype=x2.dtype, device=x2.device) if want_weight else None
    db = torch.empty(x2.shape[1], dtype=x2.dtype, device=x2.device) if want_bias else None
    ws = None
    if want_weight or want_bias:
        need = C.c_size_t(0)
        _check(_cabi.lib().nb200_layer_norm_workspace_bytes(C.byref(p), C.byref(need)),
               "nb200_layer_norm_workspace_bytes")
        ws = torch.empty(max(int(need.value), 16), dtype=torch.uint8, device=x2.device)
        p.workspace, p.workspace_bytes = ws.data_ptr(), int(need.value)
        p.dweight = None if dw is None else dw.data_ptr()
        p.dbias = None if db is None else db.data_ptr()
    with torch.cuda.device(x2.device):
        _check(_cabi.lib().nb200_layer_norm_bwd(C.byref(p), torch.cuda.current_stream().cuda_stream),
               "nb200_layer_norm_bwd")
    return dx, dw, db


class _LayerNorm(torch.autograd.Function):
    """The differentiation rule of the fused op: saves (x, weight, mean, rstd), returns (dx, dweight, dbias)."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, out_scale):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        w = None if weight is None else weight.to(x.dtype).contiguous()
        b = None if bias is None else bias.to(x.dtype).contiguous()
        y, mean, rstd = layer_norm_forward(x2, w, b, eps, out_scale)
        ctx.save_for_backward(x2, w if w is not None else x2.new_empty(0), mean, rstd)
        ctx.has_weight, ctx.has_bias = weight is not None, bias is not None
        ctx.eps, ctx.out_scale, ctx.shape = eps, out_scale, x.shape
        ctx.param_dtypes = (None if weight is None else weight.dtype, None if bias is None else bias.dtype)
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).to(x2.dtype).contiguous()
        need_w = ctx.has_weight and ctx.needs_input_grad[1]
        need_b = ctx.has_bias and ctx.needs_input_grad[2]
        dx, dw, db = layer_norm_backward(x2, w if ctx.has_weight else None, dy2, mean, rstd, ctx.eps, ctx.out_scale,
                                         need_w, need_b)
        if dw is not None:
            dw = dw.to(ctx.param_dtypes[0])
        if db is not None:
            db = db.to(ctx.param_dtypes[1])
        return dx.reshape(ctx.shape), dw, db, None, None


def layer_norm(x: torch.Tensor, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None, *,
               eps: float = 1e-5, out_scale: float = 1.0, backend: str = "auto") -> torch.Tensor:
    """LayerNorm over the trailing axis: ``out_scale * (xhat * weight + bias)`` (reference
    ``nn/norm/__init__.py:110-176``).  ``x`` is a CUDA tensor of fp32, bf16 or fp16; ``weight`` and ``bias`` have
    shape ``(c,)``.  Differentiable in ``x``, ``weight`` and ``bias``."""
    _check_affine("layer_norm", weight, bias, x.shape[-1])
    resolve_backend(backend)   # raises without a Blackwell device: there is no host path
    if not x.is_cuda or x.dtype not in _DTYPES:
        raise TypeError(f"layer_norm: x must be a CUDA tensor of float32, bfloat16 or float16; got {x.dtype} on {x.device}")
    if x.numel() == 0:
        return torch.empty_like(x)
    return _LayerNorm.apply(x, weight, bias, float(eps), float(out_scale))
