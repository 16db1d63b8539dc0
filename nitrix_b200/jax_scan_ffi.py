"""JAX binding of the selective scan: ``jax.ffi`` custom calls under a ``jax.custom_vjp``.

The module a maintainer of the reference points its scan dispatcher at: ``selective_scan_sm100(x, delta, A, B, C, D)``
takes what the dispatcher passes its fused scan module (``_selective_scan_pallas``, reference
``src/nitrix/nn/ssm/__init__.py:80-125``), returns what ``reference_selective_scan`` returns
(``src/nitrix/nn/ssm/_reference.py:193-``) and is differentiable in every operand: ``custom_vjp`` with residuals
``(x, delta, A, B, C, D, checkpoints)`` and cotangents ``(dx, ddelta, dA, dB, dC, dD)``.

Two shared objects are involved: ``libnitrix_b200_attention.so`` (kernels and C ABI; its size queries are called
here through ctypes at trace time, when shapes are static) and ``libnitrix_b200_scan_ffi.so``
(``ffi/nb200_scan_ffi.cc`` compiled against jaxlib's XLA FFI headers), whose two handler symbols are registered as
custom-call targets.

NOT EXECUTED in this repository: neither ``jax`` nor the XLA FFI headers are installed where it is built and tested.
The module imports without jax (every jax use is inside a function); a CPU test compiles it and checks the handler
names and attributes against ``ffi/nb200_scan_ffi.cc``.
"""
from __future__ import annotations

import ctypes as C
import functools
import math
import os
import pathlib

import numpy as np

from . import _cabi

FWD_TARGET = "nb200_selective_scan_fwd"
BWD_TARGET = "nb200_selective_scan_bwd"
FWD_SYMBOL = "nb200_selective_scan_fwd_ffi"
BWD_SYMBOL = "nb200_selective_scan_bwd_ffi"
FWD_ATTRS = ("has_d",)
BWD_ATTRS = ("has_d",)

_FFI_LIB_ENV = "NITRIX_B200_SCAN_FFI_LIB"
_DTYPE_CODES = {"float32": _cabi.F32, "bfloat16": _cabi.BF16, "float16": _cabi.F16}
_registered = False


def _jax():
    try:
        import jax  # noqa: PLC0415
    except ImportError as exc:  # pragma: no cover - jax is absent where this repository is tested
        raise ImportError("nitrix_b200.jax_scan_ffi needs jax (>= 0.4.38, with jax.ffi) and jaxlib built for CUDA") from exc
    return jax


def ffi_library_path() -> pathlib.Path:
    """Where the compiled FFI shim is looked for: ``$NITRIX_B200_SCAN_FFI_LIB`` or next to the kernel library."""
    env = os.environ.get(_FFI_LIB_ENV)
    if env:
        return pathlib.Path(env)
    from . import _build  # noqa: PLC0415

    return _build.LIBDIR / "libnitrix_b200_scan_ffi.so"


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
def scratch_bytes(batch: int, length: int, channels: int, states: int, dtype_name: str):
    """``(checkpoint_bytes, workspace_bytes)`` for this shape (trace time; shapes are static under jit)."""
    p = _cabi.SelectiveScanParams()
    p.struct_size = C.sizeof(_cabi.SelectiveScanParams)
    p.batch, p.length, p.channels, p.states = int(batch), int(length), int(channels), int(states)
    p.dtype = _DTYPE_CODES[dtype_name]
    out = []
    for fn in (_cabi.lib().nb200_selective_scan_checkpoint_bytes, _cabi.lib().nb200_selective_scan_workspace_bytes):
        need = C.c_size_t(0)
        rc = fn(C.byref(p), C.byref(need))
        if rc != _cabi.OK:
            raise RuntimeError(f"selective-scan size query failed ({rc}): {_cabi.last_error()}")
        out.append(max(int(need.value), 16))
    return tuple(out)


def _fold(a, tail):
    """Fold every leading axis of ``a`` into one batch axis, keeping the last ``tail`` axes."""
    return a.reshape((math.prod(a.shape[:-tail]),) + tuple(a.shape[-tail:]))


def _call_fwd(x3, delta3, A, B3, C3, D):
    jax = _jax()
    register()
    ck_bytes, _ = scratch_bytes(x3.shape[0], x3.shape[1], x3.shape[2], A.shape[1], str(x3.dtype))
    out_types = (jax.ShapeDtypeStruct(x3.shape, x3.dtype), jax.ShapeDtypeStruct((ck_bytes // 4,), np.float32))
    call = jax.ffi.ffi_call(FWD_TARGET, out_types)
    return call(x3, delta3, A, B3, C3, D if D is not None else jax.numpy.zeros((1,), x3.dtype), has_d=D is not None)


def _call_bwd(x3, delta3, A, B3, C3, D, ck, dy3):
    jax = _jax()
    register()
    _, ws_bytes = scratch_bytes(x3.shape[0], x3.shape[1], x3.shape[2], A.shape[1], str(x3.dtype))
    dt = x3.dtype
    out_types = (jax.ShapeDtypeStruct(x3.shape, dt), jax.ShapeDtypeStruct(x3.shape, dt),
                 jax.ShapeDtypeStruct(A.shape, dt), jax.ShapeDtypeStruct(B3.shape, dt),
                 jax.ShapeDtypeStruct(C3.shape, dt), jax.ShapeDtypeStruct(D.shape if D is not None else (1,), dt),
                 jax.ShapeDtypeStruct((ws_bytes,), np.uint8))
    call = jax.ffi.ffi_call(BWD_TARGET, out_types)
    dx, ddelta, dA, dB, dC, dD, _ = call(x3, delta3, A, B3, C3,
                                          D if D is not None else jax.numpy.zeros((1,), dt), ck, dy3,
                                          has_d=D is not None)
    return dx, ddelta, dA, dB, dC, (dD if D is not None else None)


@functools.lru_cache(maxsize=1)
def _build_scan_p():
    jax = _jax()

    @jax.custom_vjp
    def scan_p(x3, delta3, A, B3, C3, D):
        return _call_fwd(x3, delta3, A, B3, C3, D)[0]

    def scan_p_fwd(x3, delta3, A, B3, C3, D):
        y, ck = _call_fwd(x3, delta3, A, B3, C3, D)
        return y, (x3, delta3, A, B3, C3, D, ck)

    def scan_p_bwd(res, g):
        x3, delta3, A, B3, C3, D, ck = res
        return _call_bwd(x3, delta3, A, B3, C3, D, ck, g.astype(x3.dtype))

    scan_p.defvjp(scan_p_fwd, scan_p_bwd)
    return scan_p


def selective_scan_sm100(x, delta, A, B, C, D=None):  # noqa: N803
    """The selective scan on the B200 kernels (jax arrays on a CUDA device; float32, bfloat16 or float16; every
    operand is cast to ``x``'s dtype; B and C are broadcast over the leading axes of ``x``; at most 64 states)."""
    jax = _jax()
    if str(x.dtype) not in _DTYPE_CODES:
        raise TypeError(f"selective_scan_sm100: unsupported dtype {x.dtype}")
    lead = x.shape[:-2]
    dt = x.dtype
    b3 = jax.numpy.broadcast_to(B.astype(dt), lead + B.shape[-2:])
    c3 = jax.numpy.broadcast_to(C.astype(dt), lead + C.shape[-2:])
    y = _build_scan_p()(_fold(x, 2), _fold(delta.astype(dt), 2), A.astype(dt), _fold(b3, 2), _fold(c3, 2),
                        None if D is None else D.astype(dt))
    return y.reshape(x.shape)
