"""JAX binding of the B200 attention library: ``jax.ffi`` custom calls under a ``jax.custom_vjp``.

This is the module a maintainer of the reference drops in place of its fused-kernel module: it provides
``scaled_dot_product_attention_sm100(q, k, v, *, scale, bias=None, mask=None, causal=False)`` with the signature of
the reference's private fused entry ``scaled_dot_product_attention_pallas`` (reference
``src/nitrix/_kernels/cuda/attention.py:768-824``) and the differentiation contract of its ``_sdpa_p`` /
``_sdpa_p_fwd`` / ``_sdpa_p_bwd`` (``:661-700``): ``custom_vjp`` with ``scale`` and ``causal`` static
(``nondiff_argnums=(5, 6)``), residuals ``(q, k, v, bias, mask, out, lse)``, cotangents
``(dq, dk, dv, dbias-or-None, None)``.  ``NotCovered`` plays the role of the reference's ``PallasNotTileable``
(``:71-77``): the dispatcher (``nn/attention/__init__.py:63-123``) catches it and runs its ``jnp`` path with the
warn-once fallback.

Two shared objects are involved: ``libnitrix_b200_attention.so`` (the kernels and the C ABI; its planner and
workspace query are called here through ctypes at trace time, when shapes are static) and
``libnitrix_b200_ffi.so`` (``ffi/nb200_ffi.cc`` compiled against jaxlib's XLA FFI headers), whose two handler
symbols are registered as custom-call targets.

NOT EXECUTED in this repository: neither ``jax`` nor the XLA FFI headers are installed where it is built and
tested.  The module imports without jax (every jax use is inside a function); a CPU test compiles it and checks
the handler names and attributes against ``ffi/nb200_ffi.cc``.
"""
from __future__ import annotations

import ctypes as C
import functools
import math
import os
import pathlib
import numpy as np

from . import _cabi

FWD_TARGET = "nb200_sdpa_fwd"
BWD_TARGET = "nb200_sdpa_bwd"
FWD_SYMBOL = "nb200_sdpa_fwd_ffi"
BWD_SYMBOL = "nb200_sdpa_bwd_ffi"
FWD_ATTRS = ("scale", "causal", "has_bias", "has_mask")
BWD_ATTRS = ("scale", "causal", "has_bias", "has_mask", "want_dbias")

_FFI_LIB_ENV = "NITRIX_B200_FFI_LIB"
_registered = False


class NotCovered(Exception):
    """The library declines this problem (dtype or head dims no kernel covers); the caller runs its own path."""


def _jax():
    try:
        import jax  # noqa: PLC0415
    except ImportError as exc:  # pragma: no cover - jax is absent where this repository is tested
        raise ImportError("nitrix_b200.jax_ffi needs jax (>= 0.4.38, with jax.ffi) and jaxlib built for CUDA") from exc
    return jax


def ffi_library_path() -> pathlib.Path:
    """Where the compiled FFI shim is looked for: ``$NITRIX_B200_FFI_LIB`` or next to the kernel library."""
    env = os.environ.get(_FFI_LIB_ENV)
    if env:
        return pathlib.Path(env)
    from . import _build  # noqa: PLC0415

    return _build.LIBDIR / "libnitrix_b200_ffi.so"


def register() -> None:
    """Register the two custom-call targets with XLA (idempotent)."""
    global _registered
    if _registered:
        return
    jax = _jax()
    _cabi.lib()  # the kernel library first: the shim links against it
    shim = C.CDLL(str(ffi_library_path()), mode=C.RTLD_GLOBAL)
    jax.ffi.register_ffi_target(FWD_TARGET, jax.ffi.pycapsule(getattr(shim, FWD_SYMBOL)), platform="CUDA")
    jax.ffi.register_ffi_target(BWD_TARGET, jax.ffi.pycapsule(getattr(shim, BWD_SYMBOL)), platform="CUDA")
    _registered = True


# ---------------------------------------------------------------------------
# trace-time queries through the C ABI (shapes are static; pointers are placeholders the planner only checks for
# alignment, and XLA's device buffers are aligned far beyond the 16 bytes the kernels need)
# ---------------------------------------------------------------------------
_DTYPE_CODES = {"float32": _cabi.F32, "bfloat16": _cabi.BF16, "float16": _cabi.F16}
_ALIGNED = 1 << 20


def _dense(*dims):
    strides, acc = [], 1
    for d in reversed(dims):
        strides.append(acc)
        acc *= d
    return list(reversed(strides))


def _own_extent_strides(shape4, full4):
    dense = _dense(*shape4)
    return [0 if (n == 1 and f != 1) else s for n, f, s in zip(shape4, full4, dense)]


def _params(q_shape, k_shape, v_shape, dtype_name, bias_shape4, bias_dtype_name, mask_shape4, scale, causal, want_dbias):
    p = _cabi.new_params()
    lead = q_shape[:-3]
    B = int(math.prod(lead)) if lead else 1
    H, S, D = q_shape[-3:]
    T, Dv = k_shape[-2], v_shape[-1]
    if dtype_name not in _DTYPE_CODES:
        raise NotCovered(f"dtype {dtype_name} is not one of float32, bfloat16, float16")
    p.dtype = _DTYPE_CODES[dtype_name]
    p.B, p.H, p.S, p.T, p.D, p.Dv = B, H, S, T, D, Dv
    for name in ("q", "k", "v", "out", "lse", "dout", "dq", "dk", "dv"):
        setattr(p, name, _ALIGNED)
    p.q_stride[:] = p.dq_stride[:] = [H * S * D, S * D, D, 1]
    p.k_stride[:] = p.dk_stride[:] = [H * T * D, T * D, D, 1]
    p.v_stride[:] = p.dv_stride[:] = [H * T * Dv, T * Dv, Dv, 1]
    p.out_stride[:] = p.dout_stride[:] = [H * S * Dv, S * Dv, Dv, 1]
    full = (B, H, S, T)
    if bias_shape4 is not None:
        p.bias = _ALIGNED
        p.bias_dtype = _DTYPE_CODES[bias_dtype_name]
        p.bias_stride[:] = _own_extent_strides(bias_shape4, full)
        if want_dbias:
            p.want_dbias = 1
            p.dbias_stride[:] = _dense(*bias_shape4)
    if mask_shape4 is not None:
        p.mask = _ALIGNED
        p.mask_stride[:] = _own_extent_strides(mask_shape4, full)
    p.scale = float(scale)
    p.causal = int(bool(causal))
    p.kernel = _cabi.KERNEL_AUTO
    p.bh_begin, p.bh_end = 0, B * H
    return p


@functools.lru_cache(maxsize=512)
def _workspace_bytes(which, *key) -> int:
    p = _params(*key)
    need = C.c_size_t(0)
    rc = _cabi.lib().nb200_sdpa_workspace_bytes(C.byref(p), which, C.byref(need))
    if rc == _cabi.ERR_UNSUPPORTED:
        raise NotCovered(_cabi.last_error())
    if rc != _cabi.OK:
        raise ValueError(f"nb200_sdpa_workspace_bytes failed (status {rc}): {_cabi.last_error()}")
    return max(int(need.value), 1)


def _to_own_extent(x, lead, h, s, t):
    """bias / mask broadcastable to (*lead, h, s, t) -> 4-D (Bb, Hb, Sb, Tb) with each extent 1 or full."""
    jnp = _jax().numpy
    full = (*lead, h, s, t)
    x = jnp.reshape(x, (1,) * (len(full) - x.ndim) + tuple(x.shape))
    nl = len(lead)
    lead_have = tuple(x.shape[:nl])
    if all(a == 1 for a in lead_have):
        return jnp.reshape(x, (1, *x.shape[nl:]))
    if lead_have != tuple(lead):
        x = jnp.broadcast_to(x, (*lead, *x.shape[nl:]))   # a partially broadcast multi-dim batch: expand the batch
    return jnp.reshape(x, (-1, *x.shape[nl:]))


def _key(q, k, v, bias4, mask4, scale, causal, want_dbias):
    return (tuple(q.shape), tuple(k.shape), tuple(v.shape), str(q.dtype),
            None if bias4 is None else tuple(bias4.shape), None if bias4 is None else str(bias4.dtype),
            None if mask4 is None else tuple(mask4.shape), float(scale), bool(causal), bool(want_dbias))


# ---------------------------------------------------------------------------
# the primitive pair and its differentiation rule
# ---------------------------------------------------------------------------
def _placeholder(dtype):
    return _jax().numpy.zeros((1, 1, 1, 1), dtype)


def _call_fwd(q, k, v, bias4, mask4, scale, causal):
    jax = _jax()
    jnp = jax.numpy
    register()
    scratch = _workspace_bytes(_cabi.PASS_FWD, *_key(q, k, v, bias4, mask4, scale, causal, False))
    out_t = jax.ShapeDtypeStruct(tuple(q.shape[:-1]) + (v.shape[-1],), q.dtype)
    lse_t = jax.ShapeDtypeStruct(tuple(q.shape[:-1]), jnp.float32)
    scratch_t = jax.ShapeDtypeStruct((scratch,), jnp.uint8)
    call = jax.ffi.ffi_call(FWD_TARGET, (out_t, lse_t, scratch_t), vmap_method="broadcast_all")
    out, lse, _ = call(q, k, v,
                       bias4 if bias4 is not None else _placeholder(q.dtype),
                       mask4 if mask4 is not None else _placeholder(jnp.bool_),
                       scale=np.float32(scale),      # a float32 attribute, as the handler's Attr<float> decodes it
                       causal=bool(causal), has_bias=bias4 is not None, has_mask=mask4 is not None)
    return out, lse


def _call_bwd(q, k, v, bias4, mask4, out, lse, dout, scale, causal, want_dbias):
    jax = _jax()
    jnp = jax.numpy
    register()
    scratch = _workspace_bytes(_cabi.PASS_BWD, *_key(q, k, v, bias4, mask4, scale, causal, want_dbias))
    dbias_t = (jax.ShapeDtypeStruct(tuple(bias4.shape), bias4.dtype) if want_dbias
               else jax.ShapeDtypeStruct((1,), q.dtype))
    types = (jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct(k.shape, k.dtype),
             jax.ShapeDtypeStruct(v.shape, v.dtype), dbias_t, jax.ShapeDtypeStruct((scratch,), jnp.uint8))
    call = jax.ffi.ffi_call(BWD_TARGET, types, vmap_method="broadcast_all")
    dq, dk, dv, dbias, _ = call(q, k, v,
                                bias4 if bias4 is not None else _placeholder(q.dtype),
                                mask4 if mask4 is not None else _placeholder(jnp.bool_),
                                out, lse, dout, scale=np.float32(scale), causal=bool(causal), has_bias=bias4 is not None,
                                has_mask=mask4 is not None, want_dbias=bool(want_dbias))
    return dq, dk, dv, (dbias if want_dbias else None)


def _build_sdpa_p():
    """The ``custom_vjp`` function (built on first use, so that importing this module needs no jax)."""
    jax = _jax()
    jnp = jax.numpy

    @functools.partial(jax.custom_vjp, nondiff_argnums=(5, 6))
    def sdpa_p(q, k, v, bias4, mask4, scale, causal):
        return _call_fwd(q, k, v, bias4, mask4, scale, causal)[0]

    def sdpa_p_fwd(q, k, v, bias4, mask4, scale, causal):
        # symbolic_zeros=True: every differentiable argument arrives as a (value, perturbed) pair
        qv, kv, vv = q.value, k.value, v.value
        bv = None if bias4 is None else bias4.value
        mv = None if mask4 is None else mask4.value
        out, lse = _call_fwd(qv, kv, vv, bv, mv, scale, causal)
        # whether the bias is being differentiated is static information; it travels in the residual pytree's
        # STRUCTURE (None or an empty tuple), not as a traced value
        dbias_wanted = () if (bias4 is not None and bias4.perturbed) else None
        return out, (qv, kv, vv, bv, mv, out, lse, dbias_wanted)      # the reference's residual tuple (:684) + the flag

    def sdpa_p_bwd(scale, causal, res, g):
        q, k, v, bias4, mask4, out, lse, dbias_wanted = res
        if isinstance(g, jax.custom_derivatives.SymbolicZero):
            g = jnp.zeros(g.shape, g.dtype)
        want_dbias = dbias_wanted is not None
        dq, dk, dv, dbias = _call_bwd(q, k, v, bias4, mask4, out, lse, g.astype(q.dtype), scale, causal, want_dbias)
        if bias4 is not None and dbias is None:
            dbias = jnp.zeros(bias4.shape, bias4.dtype)   # an unperturbed bias: its cotangent is never used
        return dq, dk, dv, dbias, None                      # (dq, dk, dv, dbias | None, None) as the reference (:687-697)

    sdpa_p.defvjp(sdpa_p_fwd, sdpa_p_bwd, symbolic_zeros=True)
    return sdpa_p


_sdpa_p = None


def scaled_dot_product_attention_sm100(q, k, v, *, scale: float, bias=None, mask=None, causal: bool = False):
    """Fused attention through the B200 library; raises :class:`NotCovered` when the library declines.

    Same arguments as the reference's fused entry (``attention.py:768-777``): ``q`` ``(..., h, s, d)``, ``k``
    ``(..., h, t, d)``, ``v`` ``(..., h, t, d_v)``; ``bias`` / ``mask`` broadcastable to ``(..., h, s, t)``
    (never materialised: they reach the kernels as 4-D arrays with extent-1 broadcast axes).
    """
    global _sdpa_p
    jax = _jax()
    jnp = jax.numpy
    if _sdpa_p is None:
        _sdpa_p = _build_sdpa_p()
    lead = tuple(jnp.broadcast_shapes(q.shape[:-3], k.shape[:-3], v.shape[:-3]))
    h, s, d = q.shape[-3:]
    t = k.shape[-2]
    dtype = jnp.result_type(q, k, v)
    q, k, v = (jnp.broadcast_to(x.astype(dtype), (*lead, *x.shape[-3:])) for x in (q, k, v))
    bias4 = None if bias is None else _to_own_extent(bias, lead, h, s, t)
    mask4 = None if mask is None else _to_own_extent(mask.astype(jnp.bool_), lead, h, s, t)
    # ask the planner now, at trace time, so that a declined problem surfaces as NotCovered before any custom call
    _workspace_bytes(_cabi.PASS_FWD, *_key(q, k, v, bias4, mask4, scale, causal, False))
    return _sdpa_p(q, k, v, bias4, mask4, float(scale), bool(causal))


__all__ = ["scaled_dot_product_attention_sm100", "NotCovered", "register", "ffi_library_path",
           "FWD_TARGET", "BWD_TARGET", "FWD_SYMBOL", "BWD_SYMBOL"]
