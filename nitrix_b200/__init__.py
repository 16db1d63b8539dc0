"""B200-native flash attention with additive bias and boolean mask.

One path of hypercoil/nitrix -- ``nitrix.nn.scaled_dot_product_attention`` and
its forward/backward kernels -- rebuilt as hand-written sm_100a CUDA behind a C
ABI (``include/nitrix_b200_attention.h``).  The shared library is mandatory: the first
call into it raises ``NativeLibraryError`` when it has not been built; there is
no other implementation to fall back to (``python -m nitrix_b200._build`` builds it).
"""
from . import _cabi
from .backend import (
    NitrixBackendError,
    NitrixBackendFallback,
    reproducible,
    reset_fallback_state,
    resolve_backend,
)

from .nn import scaled_dot_product_attention


def require_native() -> None:
    """Load the CUDA library now (raises ``NativeLibraryError`` when it is missing)."""
    _cabi.lib()


__all__ = [
    "scaled_dot_product_attention",
    "require_native",
    "NitrixBackendError",
    "NitrixBackendFallback",
    "reproducible",
    "reset_fallback_state",
    "resolve_backend",
]
