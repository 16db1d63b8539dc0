"""ctypes binding of ``include/nitrix_b200_attention.h``.

The library is mandatory: when the shared object is missing the import of this
module raises, it never degrades to another implementation.
"""
from __future__ import annotations

import ctypes as C
import functools

from . import _build

ABI_VERSION = 2

F32, BF16, F16 = 0, 1, 2
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_WORKSPACE, ERR_LAUNCH, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5, -6
KERNEL_AUTO, KERNEL_SIMT, KERNEL_TCGEN05, KERNEL_MMA_TF32X3 = 0, 1, 2, 3
PASS_FWD, PASS_BWD = 0, 1
STATIC_SCRATCH_BYTES = 8 << 20

_I64x4 = C.c_int64 * 4


class SdpaParams(C.Structure):
    """Mirror of ``nb200_sdpa_params`` (field order and types must match the header)."""

    _fields_ = [
        ("struct_size", C.c_uint32),
        ("dtype", C.c_int32),
        ("bias_dtype", C.c_int32),
        ("B", C.c_int32), ("H", C.c_int32), ("S", C.c_int32), ("T", C.c_int32),
        ("D", C.c_int32), ("Dv", C.c_int32),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("out", C.c_void_p), ("lse", C.c_void_p),
        ("bias", C.c_void_p), ("mask", C.c_void_p),
        ("dout", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dbias", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("q_stride", _I64x4), ("k_stride", _I64x4), ("v_stride", _I64x4), ("out_stride", _I64x4),
        ("dout_stride", _I64x4), ("dq_stride", _I64x4), ("dk_stride", _I64x4), ("dv_stride", _I64x4),
        ("bias_stride", _I64x4), ("mask_stride", _I64x4), ("dbias_stride", _I64x4),
        ("scale", C.c_float),
        ("causal", C.c_int32),
        ("kernel", C.c_int32),
        ("bh_begin", C.c_int32), ("bh_end", C.c_int32),
        ("want_dbias", C.c_int32),
        ("mask_is_bitpacked", C.c_int32),
        ("n_out_peers", C.c_int32),
        ("reserved0", C.c_int32),
        ("out_peers", C.c_void_p * 7),
    ]


class IpcHandle(C.Structure):
    """Mirror of ``nb200_ipc_handle``: 128 opaque bytes that name a device allocation to another process."""

    _fields_ = [("bytes", C.c_ubyte * 128)]


class QkNormTensor(C.Structure):
    """``nb200_qk_norm_tensor``: one operand of the fused QK-norm pre-op (include/nitrix_b200_attention.h)."""

    _fields_ = [("x", C.c_void_p), ("g", C.c_void_p), ("y", C.c_void_p), ("xs", C.c_int64 * 3),
                ("B", C.c_int32), ("H", C.c_int32), ("N", C.c_int32), ("reserved", C.c_int32)]


class LayerNormParams(C.Structure):
    """``nb200_layer_norm_params`` (include/nitrix_b200_norm.h)."""

    _fields_ = [("struct_size", C.c_size_t), ("x", C.c_void_p), ("weight", C.c_void_p), ("bias", C.c_void_p),
                ("y", C.c_void_p), ("mean", C.c_void_p), ("rstd", C.c_void_p), ("dy", C.c_void_p), ("dx", C.c_void_p),
                ("dweight", C.c_void_p), ("dbias", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t), ("rows", C.c_int64), ("channels", C.c_int32), ("dtype", C.c_int32),
                ("eps", C.c_float), ("out_scale", C.c_float)]


class SelectiveScanParams(C.Structure):
    """``nb200_selective_scan_params`` (include/nitrix_b200_scan.h)."""

    _fields_ = [("struct_size", C.c_size_t), ("x", C.c_void_p), ("delta", C.c_void_p), ("A", C.c_void_p),
                ("B", C.c_void_p), ("C", C.c_void_p), ("D", C.c_void_p), ("y", C.c_void_p),
                ("checkpoints", C.c_void_p), ("dy", C.c_void_p), ("dx", C.c_void_p), ("ddelta", C.c_void_p),
                ("dA", C.c_void_p), ("dB", C.c_void_p), ("dC", C.c_void_p), ("dD", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("batch", C.c_int32),
                ("length", C.c_int32), ("channels", C.c_int32), ("states", C.c_int32), ("dtype", C.c_int32),
                ("reserved", C.c_int32)]


EXPORTS = (
    "nb200_version",
    "nb200_last_error",
    "nb200_sdpa_plan",
    "nb200_sdpa_workspace_bytes",
    "nb200_sdpa_fwd",
    "nb200_sdpa_bwd",
    "nb200_sdpa_bwd_static_scratch",
    "nb200_launch_count",
    "nb200_profile",
    "nb200_profile_read",
    "nb200_device_status",
    "nb200_selftest_bounded_wait",
    "nb200_mask_pack_bytes",
    "nb200_mask_pack",
    "nb200_ipc_export",
    "nb200_ipc_open",
    "nb200_ipc_close",
    "nb200_qk_rms_norm",
    "nb200_qk_rms_norm_grad",
    "nb200_layer_norm_fwd",
    "nb200_layer_norm_bwd",
    "nb200_layer_norm_workspace_bytes",
    "nb200_selective_scan_fwd",
    "nb200_selective_scan_bwd",
    "nb200_selective_scan_workspace_bytes",
    "nb200_selective_scan_checkpoint_bytes",
)


class NativeLibraryError(ImportError):
    """The CUDA shared library is missing, stale or has the wrong ABI."""


@functools.lru_cache(maxsize=1)
def lib() -> C.CDLL:
    path = _build.lib_path()
    if not path.exists():
        raise NativeLibraryError(
            f"{path} is missing: build it with `python -m nitrix_b200._build` (needs nvcc). "
            "There is no other implementation to fall back to."
        )
    L = C.CDLL(str(path))
    for name in EXPORTS:
        if not hasattr(L, name):
            raise NativeLibraryError(f"{path} does not export {name}")
    L.nb200_version.restype = C.c_int
    L.nb200_last_error.restype = C.c_char_p
    L.nb200_launch_count.restype = C.c_uint64
    L.nb200_device_status.argtypes = [C.c_int]
    L.nb200_profile.argtypes = [C.c_int]
    L.nb200_profile_read.argtypes = [C.c_char_p, C.c_size_t]
    L.nb200_profile_read.restype = C.c_size_t
    L.nb200_sdpa_plan.argtypes = [C.POINTER(SdpaParams), C.c_int, C.POINTER(C.c_int)]
    L.nb200_sdpa_workspace_bytes.argtypes = [C.POINTER(SdpaParams), C.c_int, C.POINTER(C.c_size_t)]
    L.nb200_sdpa_fwd.argtypes = [C.POINTER(SdpaParams), C.c_void_p]
    L.nb200_sdpa_bwd.argtypes = [C.POINTER(SdpaParams), C.c_void_p]
    L.nb200_sdpa_bwd_static_scratch.argtypes = [C.POINTER(SdpaParams), C.c_void_p]
    L.nb200_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_void_p]
    L.nb200_mask_pack_bytes.argtypes = [C.POINTER(SdpaParams), C.c_int, C.POINTER(C.c_size_t)]
    L.nb200_mask_pack.argtypes = [C.POINTER(SdpaParams), C.c_int, C.c_void_p, C.c_size_t, C.c_void_p]
    L.nb200_ipc_export.argtypes = [C.c_void_p, C.POINTER(IpcHandle)]
    L.nb200_ipc_open.argtypes = [C.POINTER(IpcHandle), C.POINTER(C.c_void_p)]
    L.nb200_ipc_close.argtypes = [C.c_void_p]
    L.nb200_qk_rms_norm.argtypes = [C.POINTER(QkNormTensor), C.POINTER(QkNormTensor), C.c_int, C.c_int, C.c_void_p]
    L.nb200_qk_rms_norm_grad.argtypes = [C.POINTER(QkNormTensor), C.POINTER(QkNormTensor), C.c_int, C.c_int, C.c_void_p]
    L.nb200_layer_norm_fwd.argtypes = [C.POINTER(LayerNormParams), C.c_void_p]
    L.nb200_layer_norm_bwd.argtypes = [C.POINTER(LayerNormParams), C.c_void_p]
    L.nb200_layer_norm_workspace_bytes.argtypes = [C.POINTER(LayerNormParams), C.POINTER(C.c_size_t)]
    L.nb200_selective_scan_fwd.argtypes = [C.POINTER(SelectiveScanParams), C.c_void_p]
    L.nb200_selective_scan_bwd.argtypes = [C.POINTER(SelectiveScanParams), C.c_void_p]
    L.nb200_selective_scan_workspace_bytes.argtypes = [C.POINTER(SelectiveScanParams), C.POINTER(C.c_size_t)]
    L.nb200_selective_scan_checkpoint_bytes.argtypes = [C.POINTER(SelectiveScanParams), C.POINTER(C.c_size_t)]
    if L.nb200_version() != ABI_VERSION:
        raise NativeLibraryError(f"{path}: ABI {L.nb200_version()} != expected {ABI_VERSION}")
    return L


def last_error() -> str:
    return lib().nb200_last_error().decode("utf-8", "replace")


def new_params() -> SdpaParams:
    p = SdpaParams()
    p.struct_size = C.sizeof(SdpaParams)
    return p


def kernel_times() -> dict:
    """Per-kernel ``{name: (launches, total_ms)}`` recorded since ``lib().nb200_profile(1)``."""
    L = lib()
    need = L.nb200_profile_read(None, 0)
    buf = C.create_string_buffer(int(need) + 16)
    L.nb200_profile_read(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split("\t")
        out[name] = (int(n), float(ms))
    return out
