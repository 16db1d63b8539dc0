"""Scaled-dot-product / flash attention on B200, PyTorch-hosted.

Drop-in for the reference's public entry
``nitrix.nn.attention.scaled_dot_product_attention``
(reference ``src/nitrix/nn/attention/__init__.py:126-230``): same positional
and keyword surface ``(q, k, v, *, bias, mask, scale, causal, qk_norm,
backend)``, same validation errors (``:40-60``), same differentiation contract
as its ``custom_vjp`` (reference ``src/nitrix/_kernels/cuda/attention.py:661-700``):
residuals ``(q, k, v, bias, mask, out, lse)``, cotangents
``(dq, dk, dv, dbias-or-None, None)`` with ``scale`` and ``causal`` static.

Differences, all on purpose:

* tensors are ``torch`` CUDA tensors (device memory, streams); the arithmetic
  is done by the CUDA library behind ``include/nitrix_b200_attention.h``;
* bias and mask are passed by stride, never broadcast-materialised, and q/k/v
  stay in ``(..., h, s, d)`` layout (the reference transposes and materialises,
  ``attention.py:507-514,560-569``);
* ``dbias`` is produced only when ``bias.requires_grad`` (the reference always
  produces it when a bias is present, ``attention.py:408,437``);
* there is no host fallback: a problem the fused kernels decline runs on the
  CUDA-core family of the same library, with the reference's warn-once
  contract.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from .. import _cabi
from ..backend import fallback, resolve_backend

__all__ = ["scaled_dot_product_attention", "default_scale", "qk_rms_norm", "sdpa_forward", "sdpa_backward"]

_QK_RMS_EPS = 1e-6  # reference _reference.py:32

_DTYPES = {torch.float32: _cabi.F32, torch.bfloat16: _cabi.BF16, torch.float16: _cabi.F16}
_KERNELS = {"cuda-sm100": _cabi.KERNEL_AUTO, "cuda-simt": _cabi.KERNEL_SIMT}


def default_scale(head_dim: int) -> float:
    """``1/sqrt(d)`` (reference ``_reference.py:35-49``)."""
    return 1.0 / math.sqrt(float(head_dim))


def qk_rms_norm(z: torch.Tensor) -> torch.Tensor:
    """RMS-normalise over the head dim, no learnable scale (reference ``_reference.py:52-77``).

    Runs outside the fused kernels' differentiation rule, as in the reference
    (``nn/attention/__init__.py:193-197``), so autograd chains its gradient.
    """
    acc = torch.promote_types(z.dtype, torch.float32)
    zf = z.to(acc)
    return (zf * torch.rsqrt(zf.square().mean(-1, keepdim=True) + _QK_RMS_EPS)).to(z.dtype)


def _norm_desc(x: torch.Tensor, y: torch.Tensor, g: Optional[torch.Tensor] = None) -> "_cabi.QkNormTensor":
    """Describes ``x`` viewed as (B, H, N, D) -- leading dims flattened -- for the fused pre-op."""
    t = _cabi.QkNormTensor()
    h, n = x.shape[-3], x.shape[-2]
    x4 = x.reshape((-1, h, n, x.shape[-1])) if x.dim() != 4 else x
    t.x, t.y, t.g = x4.data_ptr(), y.data_ptr(), (g.data_ptr() if g is not None else None)
    t.xs[0], t.xs[1], t.xs[2] = x4.stride(0), x4.stride(1), x4.stride(2)
    t.B, t.H, t.N = x4.shape[0], h, n
    return t


def _qk_norm_fusable(q: torch.Tensor, k: torch.Tensor) -> bool:
    """Both on one CUDA device, same supported dtype and head dim, rows the kernel can read with 16-byte loads."""
    if not (q.is_cuda and k.is_cuda and q.device == k.device and q.dtype == k.dtype and q.dtype in _DTYPES):
        return False
    d = q.shape[-1]
    vec = 16 // q.element_size()
    if q.dim() < 3 or k.dim() < 3 or k.shape[-1] != d or d % vec or d > 256:
        return False
    for z in (q, k):
        if z.stride(-1) != 1 or z.data_ptr() % 16:
            return False
        z4 = z if z.dim() == 4 else (z.reshape((-1,) + tuple(z.shape[-3:])) if z.is_contiguous() else None)
        if z4 is None or any(st % vec for st in z4.stride()[:3]):
            return False
    return True


class _QkRmsNorm(torch.autograd.Function):
    """``(q, k) -> (qk_rms_norm(q), qk_rms_norm(k))`` as one kernel launch each way (``nb200_qk_rms_norm`` /
    ``nb200_qk_rms_norm_grad``) instead of a chain of element-wise passes.  Same place in the call sequence as the
    reference's pre-op (``nn/attention/__init__.py:193-197``): outside the attention kernels' own differentiation
    rule, so autograd chains the two."""

    @staticmethod
    def forward(ctx, q, k):
        qn, kn = torch.empty(q.shape, dtype=q.dtype, device=q.device), torch.empty(k.shape, dtype=k.dtype, device=k.device)
        with torch.cuda.device(q.device):
            rc = _cabi.lib().nb200_qk_rms_norm(_norm_desc(q, qn), _norm_desc(k, kn), q.shape[-1], _DTYPES[q.dtype],
                                                torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError("nb200_qk_rms_norm: " + _cabi.last_error())
        ctx.save_for_backward(q, k)
        return qn, kn

    @staticmethod
    def backward(ctx, gq, gk):
        q, k = ctx.saved_tensors
        gq, gk = gq.contiguous().to(q.dtype), gk.contiguous().to(k.dtype)
        dq, dk = torch.empty(q.shape, dtype=q.dtype, device=q.device), torch.empty(k.shape, dtype=k.dtype, device=k.device)
        with torch.cuda.device(q.device):
            rc = _cabi.lib().nb200_qk_rms_norm_grad(_norm_desc(q, dq, gq), _norm_desc(k, dk, gk), q.shape[-1],
                                                     _DTYPES[q.dtype], torch.cuda.current_stream().cuda_stream)
        if rc != 0:
            raise RuntimeError("nb200_qk_rms_norm_grad: " + _cabi.last_error())
        return dq, dk


def qk_rms_norm_pair(q: torch.Tensor, k: torch.Tensor):
    """``qk_rms_norm`` of q and k: the fused CUDA pre-op where its layout rules hold, else the element-wise form."""
    if _qk_norm_fusable(q, k):
        return _QkRmsNorm.apply(q, k)
    return qk_rms_norm(q), qk_rms_norm(k)


def _validate(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
    # reference nn/attention/__init__.py:40-60
    if q.ndim < 3 or k.ndim < 3 or v.ndim < 3:
        raise ValueError(
            "scaled_dot_product_attention: q, k, v must have at least 3 dims (..., h, s, d); "
            f"got ndim {q.ndim}, {k.ndim}, {v.ndim}."
        )
    if q.shape[-1] != k.shape[-1]:
        raise ValueError(
            f"scaled_dot_product_attention: q/k head-dim mismatch (q d={q.shape[-1]}, k d={k.shape[-1]})."
        )
    if k.shape[-2] != v.shape[-2]:
        raise ValueError(
            f"scaled_dot_product_attention: k/v key-length mismatch (k t={k.shape[-2]}, v t={v.shape[-2]})."
        )


# ---------------------------------------------------------------------------
# shape canonicalisation: everything becomes 4-D (B, H, rows, cols)
# ---------------------------------------------------------------------------

def _to_bhxd(x: torch.Tensor, lead: Tuple[int, ...], h: int) -> torch.Tensor:
    """(..., h, n, d) -> (B, h, n, d) with the leading dims broadcast to ``lead``."""
    n, d = x.shape[-2], x.shape[-1]
    x = x.expand(*lead, h, n, d) if tuple(x.shape[:-3]) != lead or x.shape[-3] != h else x
    x = x.reshape(-1, h, n, d) if x.ndim != 4 else x
    if x.stride(-1) != 1 or _has_expanded_axis(x):
        # the tensor-core kernels address q, k, v by absolute (batch, head): an expanded view is materialised
        x = x.contiguous()
    return x


def _has_expanded_axis(x: torch.Tensor) -> bool:
    return any(st == 0 and n > 1 for st, n in zip(x.stride(), x.shape))


def _to_own_extent(x: torch.Tensor, lead: Tuple[int, ...], h: int, s: int, t: int) -> torch.Tensor:
    """bias / mask broadcastable to (*lead, h, s, t) -> 4-D (Bb, Hb, Sb, Tb), each extent 1 or full.

    Only differentiable view/expand ops are used, so a bias gradient of this
    4-D shape flows back to the caller's bias shape through autograd.  Leading
    dims are merged without copying whenever they are all broadcast or all
    present; a partially broadcast multi-dim batch is expanded over the batch.
    """
    full = (*lead, h, s, t)
    if x.ndim > len(full):
        raise ValueError(f"bias/mask of shape {tuple(x.shape)} has more dims than (..., h, s, t) = {full}")
    x = x.reshape((1,) * (len(full) - x.ndim) + tuple(x.shape))
    for have, want in zip(x.shape, full):
        if have != 1 and have != want:
            raise ValueError(f"bias/mask of shape {tuple(x.shape)} does not broadcast to {full}")
    nl = len(lead)
    lead_have = tuple(x.shape[:nl])
    if all(a == 1 for a in lead_have):
        x = x.reshape(1, *x.shape[nl:])
    elif lead_have == lead:
        x = x.reshape(-1, *x.shape[nl:])
    else:
        x = x.expand(*lead, *x.shape[nl:]).reshape(-1, *x.shape[nl:])
    return x


def _strides4(x: Optional[torch.Tensor], full: Tuple[int, int, int, int]):
    """Element strides with 0 on every broadcast (extent-1) axis."""
    arr = (C.c_int64 * 4)()
    if x is not None:
        for a in range(4):
            arr[a] = 0 if (x.shape[a] == 1 and full[a] != 1) else x.stride(a)
    return arr


class PackedMask:
    """A boolean mask bit-packed once by ``nb200_mask_pack`` for one problem shape and reused by the forward, the
    backward and later calls.  ``level`` 1: packed without the key-major copy; 2: with it (what the backward of a
    mask with a query axis reads).  ``like`` is the 4-D byte mask it was packed from (strides tell the library
    which axes the mask broadcasts over)."""

    def __init__(self, blob: torch.Tensor, level: int, like: torch.Tensor):
        self.blob, self.level, self.like = blob, int(level), like


def _fill_common(p, q, k, v, out, lse, bias, mask, scale, causal, kernel, bh_range):
    B, H, S, D = q.shape
    T, Dv = k.shape[2], v.shape[3]
    p.dtype = _DTYPES[q.dtype]
    p.B, p.H, p.S, p.T, p.D, p.Dv = B, H, S, T, D, Dv
    p.q, p.k, p.v, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    full = (B, H, S, T)
    for name, ten in (("q_stride", q), ("k_stride", k), ("v_stride", v), ("out_stride", out)):
        getattr(p, name)[:] = list(ten.stride())
    if bias is not None:
        p.bias = bias.data_ptr()
        p.bias_dtype = _DTYPES[bias.dtype]
        p.bias_stride = _strides4(bias, full)
    if isinstance(mask, PackedMask):
        p.mask = mask.blob.data_ptr()
        p.mask_stride = _strides4(mask.like, full)
        p.mask_is_bitpacked = mask.level
    elif mask is not None:
        p.mask = mask.data_ptr()
        p.mask_stride = _strides4(mask, full)
    p.scale = float(scale)
    p.causal = int(bool(causal))
    p.kernel = int(kernel)
    lo, hi = (0, B * H) if bh_range is None else bh_range
    p.bh_begin, p.bh_end = int(lo), int(hi)


def _check(rc: int, what: str) -> None:
    if rc != _cabi.OK:
        raise RuntimeError(f"{what} failed (status {rc}): {_cabi.last_error()}")


def _workspace(p, which: int, device) -> Optional[torch.Tensor]:
    need = C.c_size_t(0)
    _check(_cabi.lib().nb200_sdpa_workspace_bytes(C.byref(p), which, C.byref(need)), "nb200_sdpa_workspace_bytes")
    if need.value == 0:
        return None
    ws = torch.empty(need.value, dtype=torch.uint8, device=device)
    p.workspace = ws.data_ptr()
    p.workspace_bytes = need.value
    return ws


def _launch(fn, p, device, what: str) -> None:
    """Call a library entry point on `device`'s current stream (the device is switched only when it is not current)."""
    stream = torch.cuda.current_stream(device).cuda_stream
    if device.index is None or device.index == torch.cuda.current_device():
        _check(fn(C.byref(p), C.c_void_p(stream)), what)
    else:
        with torch.cuda.device(device):
            _check(fn(C.byref(p), C.c_void_p(stream)), what)


def _mask_bytes(mask):
    if mask is None or isinstance(mask, PackedMask):
        return mask
    if mask.dtype == torch.bool:
        return mask.view(torch.uint8)
    if mask.dtype == torch.uint8:
        return mask
    return (mask != 0).view(torch.uint8)


def planned_kernel(q, k, v, bias=None, mask=None, *, scale=1.0, causal=False, which=_cabi.PASS_FWD,
                   kernel=_cabi.KERNEL_AUTO, want_dbias=False) -> int:
    """Kernel family the library would run for these 4-D operands (no launch)."""
    p = _cabi.new_params()
    B, H, S, _ = q.shape
    out = q  # pointers are not dereferenced by the planner
    lse = q
    _fill_common(p, q, k, v, out, lse, bias, _mask_bytes(mask), scale, causal, kernel, None)
    p.dout = p.dq = p.dk = p.dv = q.data_ptr()
    p.dout_stride = p.dq_stride = p.out_stride
    p.dk_stride, p.dv_stride = p.k_stride, p.v_stride
    if want_dbias and bias is not None and which == _cabi.PASS_BWD:
        p.want_dbias = 1   # the planner needs no dbias buffer
        p.dbias_stride[:] = [bias.shape[1] * bias.shape[2] * bias.shape[3], bias.shape[2] * bias.shape[3], bias.shape[3], 1]
    chosen = C.c_int(0)
    _check(_cabi.lib().nb200_sdpa_plan(C.byref(p), which, C.byref(chosen)), "nb200_sdpa_plan")
    return chosen.value


def pack_mask(q, k, v, mask, *, with_transpose: bool = True) -> PackedMask:
    """Bit-pack a 4-D boolean / byte mask for these operands' shape (enqueued on the current stream)."""
    mask_b = _mask_bytes(mask)
    p = _cabi.new_params()
    _fill_common(p, q, k, v, q, q, None, mask_b, 1.0, False, _cabi.KERNEL_AUTO, None)
    need = C.c_size_t(0)
    _check(_cabi.lib().nb200_mask_pack_bytes(C.byref(p), int(with_transpose), C.byref(need)), "nb200_mask_pack_bytes")
    blob = torch.empty(max(int(need.value), 1), dtype=torch.uint8, device=q.device)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        _check(_cabi.lib().nb200_mask_pack(C.byref(p), int(with_transpose), C.c_void_p(blob.data_ptr()),
                                           C.c_size_t(blob.numel()), C.c_void_p(stream)), "nb200_mask_pack")
    return PackedMask(blob, 2 if with_transpose else 1, mask_b)


_plan_cache: dict = {}


def _meta(x: Optional[torch.Tensor]):
    # everything the planner looks at: dtype, extents, strides and the 16-byte alignment of the base address
    return None if x is None else (x.dtype, tuple(x.shape), x.stride(), x.data_ptr() & 15)


def _planned_kernel_cached(q, k, v, bias, mask, scale, causal, which=_cabi.PASS_FWD, kernel=_cabi.KERNEL_AUTO,
                           want_dbias=False) -> int:
    """Plan for these operands, remembered by their layout (the planner is pure in it)."""
    key = (_meta(q), _meta(k), _meta(v), _meta(bias), _meta(mask), scale > 0.0, bool(causal), q.device.index,
           which, kernel, bool(want_dbias))
    chosen = _plan_cache.get(key)
    if chosen is None:
        chosen = planned_kernel(q, k, v, bias, mask, scale=scale, causal=causal, which=which, kernel=kernel,
                                want_dbias=want_dbias)
        if len(_plan_cache) >= 512:
            _plan_cache.clear()
        _plan_cache[key] = chosen
    return chosen


def sdpa_forward(q, k, v, bias=None, mask=None, *, scale: float, causal: bool = False,
                 kernel: int = _cabi.KERNEL_AUTO, bh_range=None, out=None, lse=None, out_peers=()):
    """Enqueue the forward on the current stream; 4-D operands.  Returns ``(out, lse)``.

    ``q`` (B,H,S,D), ``k`` (B,H,T,D), ``v`` (B,H,T,Dv); ``bias`` / ``mask`` 4-D
    with each extent 1 (broadcast) or full.  ``lse`` is fp32 (B,H,S), base 2.
    ``out_peers``: device addresses (ints) of further buffers with ``out``'s shape and strides that receive every
    output row as well (the fused all-gather of :mod:`nitrix_b200.parallel`).
    """
    B, H, S, _ = q.shape
    Dv = v.shape[3]
    if out is None:
        out = torch.empty((B, H, S, Dv), dtype=q.dtype, device=q.device)
    if lse is None:
        lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    p = _cabi.new_params()
    mask_b = _mask_bytes(mask)
    _fill_common(p, q, k, v, out, lse, bias, mask_b, scale, causal, kernel, bh_range)
    p.n_out_peers = len(out_peers)
    for i, ptr in enumerate(out_peers):
        p.out_peers[i] = int(ptr)
    ws = _workspace(p, _cabi.PASS_FWD, q.device)
    _launch(_cabi.lib().nb200_sdpa_fwd, p, q.device, "nb200_sdpa_fwd")
    del ws  # same-stream reuse is ordered by the caching allocator
    return out, lse


def sdpa_backward(q, k, v, bias, mask, out, lse, dout, *, scale: float, causal: bool = False,
                  want_dbias: bool = False, kernel: int = _cabi.KERNEL_AUTO, bh_range=None, grads=None):
    """Enqueue the backward on the current stream; returns ``(dq, dk, dv, dbias_or_None)``.

    ``dbias`` has the bias' own 4-D extent (broadcast axes already reduced) and dtype.  ``grads`` = existing
    ``(dq, dk, dv, dbias_or_None)`` buffers to write into (several ``bh_range`` calls filling one set of buffers).
    """
    if dout.stride(-1) != 1 or _has_expanded_axis(dout):
        dout = dout.contiguous()   # e.g. the cotangent of out.sum() or out.mean(0) arrives as an expanded view
    if grads is not None:
        dq, dk, dv, dbias_buf = grads
    else:
        dq = torch.empty_like(q, memory_format=torch.contiguous_format)
        dk = torch.empty_like(k, memory_format=torch.contiguous_format)
        dv = torch.empty_like(v, memory_format=torch.contiguous_format)
        dbias_buf = None
    dbias = None
    p = _cabi.new_params()
    mask_b = _mask_bytes(mask)
    _fill_common(p, q, k, v, out, lse, bias, mask_b, scale, causal, kernel, bh_range)
    p.dout, p.dq, p.dk, p.dv = dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    p.dout_stride[:] = list(dout.stride())
    p.dq_stride[:] = list(dq.stride())
    p.dk_stride[:] = list(dk.stride())
    p.dv_stride[:] = list(dv.stride())
    if want_dbias:
        if bias is None:
            raise ValueError("want_dbias without a bias")
        dbias = dbias_buf if dbias_buf is not None else torch.empty(bias.shape, dtype=bias.dtype, device=bias.device)
        p.dbias = dbias.data_ptr()
        p.dbias_stride[:] = list(dbias.stride())
    ws = _workspace(p, _cabi.PASS_BWD, q.device)
    _launch(_cabi.lib().nb200_sdpa_bwd, p, q.device, "nb200_sdpa_bwd")
    del ws  # same-stream reuse is ordered by the caching allocator
    return dq, dk, dv, dbias


class _SDPA(torch.autograd.Function):
    """Differentiation rule of the fused path (reference ``attention.py:661-700``)."""

    @staticmethod
    def forward(ctx, q, k, v, bias, mask, scale, causal, kernel, fused):
        # On the fused (tensor-core) path the mask is bit-packed ONCE, with the key-major copy, and the same bits
        # serve the forward and the backward; otherwise each pass reads the byte mask.
        packed = None
        if fused and mask is not None:
            want_dbias = bias is not None and ctx.needs_input_grad[3]
            if _planned_kernel_cached(q, k, v, bias, mask, scale, causal, _cabi.PASS_BWD, kernel,
                                      want_dbias) == _cabi.KERNEL_TCGEN05:
                packed = pack_mask(q, k, v, mask, with_transpose=True)
        out, lse = sdpa_forward(q, k, v, bias, mask if packed is None else packed, scale=scale, causal=causal,
                                kernel=kernel)
        ctx.save_for_backward(q, k, v, bias, mask, out, lse)
        ctx.packed = packed
        ctx.scale, ctx.causal, ctx.kernel = scale, causal, kernel
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, dout, _dlse):
        q, k, v, bias, mask, out, lse = ctx.saved_tensors
        want_dbias = bias is not None and ctx.needs_input_grad[3]
        dq, dk, dv, dbias = sdpa_backward(q, k, v, bias, mask if ctx.packed is None else ctx.packed, out, lse, dout,
                                          scale=ctx.scale, causal=ctx.causal, want_dbias=want_dbias, kernel=ctx.kernel)
        return dq, dk, dv, dbias, None, None, None, None, None


def scaled_dot_product_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    bias: Optional[torch.Tensor] = None,
    mask: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    causal: bool = False,
    qk_norm: bool = False,
    backend: str = "auto",
    return_lse: bool = False,
):
    """``softmax(scale * q k^T + bias [masked]) v`` over the key axis, differentiable.

    Parameters follow the reference entry point: ``q`` ``(..., h, s, d)``, ``k``
    ``(..., h, t, d)``, ``v`` ``(..., h, t, d_v)``; ``bias`` (additive, applied
    after scaling) and ``mask`` (boolean, ``True`` keeps) broadcast to
    ``(..., h, s, t)``; ``causal`` keeps keys ``j <= i`` with indices aligned at
    zero and is AND-ed with ``mask``; ``scale`` defaults to ``1/sqrt(d)``;
    ``qk_norm`` RMS-normalises q and k first.  The result has shape
    ``(..., h, s, d_v)`` and the common dtype of q, k, v.  Computation is fp32
    (accumulators, softmax) whatever the storage dtype.  A query row with no
    kept key yields NaN, like the reference's ``jnp`` path.

    ``backend``: ``'auto'`` | ``'cuda-sm100'`` (alias ``'pallas-cuda'``) |
    ``'cuda-simt'``; see :mod:`nitrix_b200.backend`.
    """
    _validate(q, k, v)
    resolved_scale = default_scale(q.shape[-1]) if scale is None else float(scale)
    resolved = resolve_backend(backend)
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("scaled_dot_product_attention: q, k, v must be CUDA tensors (no host path exists)")
    out_dtype = torch.promote_types(torch.promote_types(q.dtype, k.dtype), v.dtype)
    if out_dtype not in _DTYPES:
        raise ValueError(f"scaled_dot_product_attention: dtype {out_dtype} is not supported (fp32, bf16, fp16)")
    q, k, v = q.to(out_dtype), k.to(out_dtype), v.to(out_dtype)
    if qk_norm:
        q, k = qk_rms_norm_pair(q, k)

    h, s, d = q.shape[-3:]
    t, dv = k.shape[-2], v.shape[-1]
    lq, lk, lv = tuple(q.shape[:-3]), tuple(k.shape[:-3]), tuple(v.shape[:-3])
    lead = lq if (lq == lk and lq == lv) else tuple(torch.broadcast_shapes(lq, lk, lv))
    if k.shape[-3] != h or v.shape[-3] != h:
        raise ValueError(f"scaled_dot_product_attention: head-count mismatch (q {h}, k {k.shape[-3]}, v {v.shape[-3]})")
    q4, k4, v4 = _to_bhxd(q, lead, h), _to_bhxd(k, lead, h), _to_bhxd(v, lead, h)
    bias4 = None
    if bias is not None:
        if bias.dtype not in _DTYPES:
            bias = bias.to(torch.float32)
        bias4 = _to_own_extent(bias, lead, h, s, t)
    mask4 = None if mask is None else _to_own_extent(mask, lead, h, s, t)

    kernel = _KERNELS[resolved]
    fused = False
    if resolved == "cuda-sm100":
        chosen = _planned_kernel_cached(q4, k4, v4, bias4, mask4, resolved_scale, causal)
        fused = chosen == _cabi.KERNEL_TCGEN05
        # fp32 operands on the 3 x TF32 tensor kernels are a fused path too (fp32 is the one dtype the reference's
        # fused kernels accept, attention.py:736-744): only a problem that leaves the tensor paths altogether warns
        if chosen not in (_cabi.KERNEL_TCGEN05, _cabi.KERNEL_MMA_TF32X3):
            fallback(
                function="scaled_dot_product_attention",
                requested="cuda-sm100",
                resolved="cuda-simt",
                reason=(
                    "the fused tcgen05 kernels take bf16/fp16 with d == d_v in {64, 128} (any query/key lengths); "
                    "the fused 3xTF32 kernels take fp32 with d, d_v in {32, 64, 128}"
                ),
                shapes=(tuple(q.shape), tuple(k.shape), tuple(v.shape)),
                dtype=out_dtype,
            )
    needs_grad = torch.is_grad_enabled() and (
        q4.requires_grad or k4.requires_grad or v4.requires_grad or (bias4 is not None and bias4.requires_grad))
    if needs_grad:
        out4, lse4 = _SDPA.apply(q4, k4, v4, bias4, mask4, resolved_scale, bool(causal), kernel, fused)
    else:   # nothing to differentiate: skip the autograd bookkeeping
        out4, lse4 = sdpa_forward(q4, k4, v4, bias4, mask4, scale=resolved_scale, causal=bool(causal), kernel=kernel)
    out = out4.reshape(*lead, h, s, dv)
    if return_lse:
        return out, lse4.reshape(*lead, h, s)
    return out
