"""JAX binding of the fused LayerNorm: ``jax.ffi`` custom calls under a ``jax.custom_vjp``.

The module a maintainer of the reference points its norm dispatcher at: ``layer_norm_sm100(x, weight, bias, *, eps,
out_scale)`` has the signature the dispatcher calls its fused-norm module with (``layer_norm_pallas``, reference
``src/nitrix/nn/norm/__init__.py:57-95``), returns what ``reference_layer_norm`` returns
(``src/nitrix/nn/norm/_reference.py:44-110``) and is differentiable in ``x``, ``weight`` and ``bias``: ``custom_vjp``
with ``eps`` and ``out_scale`` static, residuals ``(x, weight, mean, rstd)``, cotangents ``(dx, dweight, dbias)``.

Two shared objects are involved: ``libnitrix_b200_attention.so`` (kernels and C ABI; its workspace query is called
here through ctypes at trace time, when shapes are static) and ``libnitrix_b200_norm_ffi.so``
(``ffi/nb200_norm_ffi.cc`` compiled against jaxlib's XLA FFI headers), whose two handler symbols are registered as
custom-call targets.

NOT EXECUTED in this repository: neither ``jax`` nor the XLA FFI headers are installed where it is built and tested.
The module imports without jax (every jax use is inside a function); a CPU test compiles it and checks the handler
names and attributes against ``ffi/nb200_norm_ffi.cc``.
"""
from __future__ import annotations

import ctypes as C
import functools
import math
import os
import pathlib

import numpy as np

from . import _cabi

FWD_TARGET = "nb200_layer_norm_fwd"
BWD_TARGET = "nb200_layer_norm_bwd"
FWD_SYMBOL = "nb200_layer_norm_fwd_ffi"
BWD_SYMBOL = "nb200_layer_norm_bwd_ffi"
FWD_ATTRS = ("eps", "out_scale", "has_weight", "has_bias")
BWD_ATTRS = ("eps", "out_scale", "has_weight", "want_dweight", "want_dbias")

_FFI_LIB_ENV = "NITRIX_B200_NORM_FFI_LIB"
_DTYPE_CODES = {"float32": _cabi.F32, "bfloat16": _cabi.BF16, "float16": _cabi.F16}
_registered = False


def _jax():
    try:
        import jax  # noqa: PLC0415
    except ImportError as exc:  # pragma: no cover - jax is absent where this repository is tested
        raise ImportError("nitrix_b200.jax_norm_ffi needs jax (>= 0.4.38, with jax.ffi) and jaxlib built for CUDA") from exc
    return jax


def ffi_library_path() -> pathlib.Path:
    """Where the compiled FFI shim is looked for: ``$NITRIX_B200_NORM_FFI_LIB`` or next to the kernel library."""
    env = os.environ.get(_FFI_LIB_ENV)
    if env:
        return pathlib.Path(env)
    from . import _build  # noqa: PLC0415

    return _build.LIBDIR / "libnitrix_b200_norm_ffi.so"


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


@functools.lru_cache(maxsize=256)
def workspace_bytes(rows: int, channels: int, dtype_name: str) -> int:
    """Size of the backward's column-sum scratch for this shape (trace time; shapes are static under jit)."""
    p = _cabi.LayerNormParams()
    p.struct_size = C.sizeof(_cabi.LayerNormParams)
    p.rows, p.channels, p.dtype = int(rows), int(channels), _DTYPE_CODES[dtype_name]
    need = C.c_size_t(0)
    rc = _cabi.lib().nb200_layer_norm_workspace_bytes(C.byref(p), C.byref(need))
    if rc != _cabi.OK:
        raise RuntimeError(f"nb200_layer_norm_workspace_bytes failed ({rc}): {_cabi.last_error()}")
    return max(int(need.value), 16)


def _placeholder(dtype):
    jax = _jax()
    return jax.numpy.zeros((1,), dtype)


def _call_fwd(x, weight, bias, eps, out_scale):
    jax = _jax()
    register()
    rows = math.prod(x.shape[:-1])
    out_types = (jax.ShapeDtypeStruct(x.shape, x.dtype), jax.ShapeDtypeStruct((rows,), np.float32),
                 jax.ShapeDtypeStruct((rows,), np.float32))
    call = jax.ffi.ffi_call(FWD_TARGET, out_types)
    return call(x, weight if weight is not None else _placeholder(x.dtype),
                bias if bias is not None else _placeholder(x.dtype),
                eps=np.float32(eps), out_scale=np.float32(out_scale),     # float32 attributes, as Attr<float> decodes them
                has_weight=weight is not None, has_bias=bias is not None)


def _call_bwd(x, weight, mean, rstd, dy, eps, out_scale, want_dweight, want_dbias):
    jax = _jax()
    register()
    rows, c = math.prod(x.shape[:-1]), x.shape[-1]
    need = workspace_bytes(rows, c, str(x.dtype)) if (want_dweight or want_dbias) else 16
    out_types = (jax.ShapeDtypeStruct(x.shape, x.dtype),
                 jax.ShapeDtypeStruct((c,) if want_dweight else (1,), x.dtype),
                 jax.ShapeDtypeStruct((c,) if want_dbias else (1,), x.dtype),
                 jax.ShapeDtypeStruct((need,), np.uint8))
    call = jax.ffi.ffi_call(BWD_TARGET, out_types)
    dx, dw, db, _ = call(x, weight if weight is not None else _placeholder(x.dtype), mean, rstd, dy,
                         eps=np.float32(eps), out_scale=np.float32(out_scale), has_weight=weight is not None,
                         want_dweight=bool(want_dweight), want_dbias=bool(want_dbias))
    return dx, (dw if want_dweight else None), (db if want_dbias else None)


@functools.lru_cache(maxsize=1)
def _build_layer_norm_p():
    jax = _jax()

    @functools.partial(jax.custom_vjp, nondiff_argnums=(3, 4))
    def layer_norm_p(x, weight, bias, eps, out_scale):
        return _call_fwd(x, weight, bias, eps, out_scale)[0]

    def layer_norm_p_fwd(x, weight, bias, eps, out_scale):
        y, mean, rstd = _call_fwd(x, weight, bias, eps, out_scale)
        return y, (x, weight, bias is not None, mean, rstd)

    def layer_norm_p_bwd(eps, out_scale, res, g):
        x, weight, has_bias, mean, rstd = res
        dx, dw, db = _call_bwd(x, weight, mean, rstd, g.astype(x.dtype), eps, out_scale, weight is not None, has_bias)
        return dx, dw, db

    layer_norm_p.defvjp(layer_norm_p_fwd, layer_norm_p_bwd)
    return layer_norm_p


def layer_norm_sm100(x, weight=None, bias=None, *, eps: float = 1e-5, out_scale: float = 1.0):
    """``out_scale * (x_hat * weight + bias)`` over the trailing axis on the B200 kernels (jax arrays on a CUDA
    device; float32, bfloat16 or float16; ``weight`` / ``bias`` of shape ``(c,)`` are cast to ``x``'s dtype)."""
    if str(x.dtype) not in _DTYPE_CODES:
        raise TypeError(f"layer_norm_sm100: unsupported dtype {x.dtype}")
    w = None if weight is None else weight.astype(x.dtype)
    b = None if bias is None else bias.astype(x.dtype)
    return _build_layer_norm_p()(x, w, b, float(eps), float(out_scale))
