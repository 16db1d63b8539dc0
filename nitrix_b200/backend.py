"""Backend resolution and loud-fallback bookkeeping for the B200 attention path.

Mirrors the reference's dispatch vocabulary (reference
``src/nitrix/_internal/backend.py``: types ``:34-60``, env knobs ``:141-162``,
``auto_backend`` ``:170-198``, ``resolve_backend`` ``:227-267``, ``fallback`` /
``reset_fallback_state`` ``:307-383``) with the same three-level rule
(keyword > ``NITRIX_BACKEND`` > autodetect), the same environment variable
names and the same warn-once / strict / silence behaviour.

What differs is what the names resolve to.  There is no host implementation
behind this package: both resolved engines are CUDA kernel families of the same
shared library.

``'cuda-sm100'``
    the fused TMA + tcgen05 kernels (the counterpart of the reference's
    ``'pallas-cuda'``, which is accepted as an alias);
``'cuda-simt'``
    CUDA-core kernels in true fp32 arithmetic.  They take every shape and dtype
    and are what a problem the fused kernels decline falls back to, with one
    ``NitrixBackendFallback`` warning per (function, shapes, dtype, backend).
    Reproducibility mode resolves ``'auto'`` to this family, as the reference
    resolves it to its non-tensor-core engine (``backend.py:192-195``).

``'jax'`` (the reference's host path) is not shipped; asking for it raises
``NitrixBackendError``.
"""
from __future__ import annotations

import contextlib
import contextvars
import os
import threading
import warnings
from typing import Any, Iterator, Literal, Optional

Backend = Literal["auto", "cuda-sm100", "cuda-simt", "pallas-cuda", "jax"]
ResolvedBackend = Literal["cuda-sm100", "cuda-simt"]

_VALID_BACKENDS = ("auto", "cuda-sm100", "cuda-simt", "pallas-cuda", "jax")


class NitrixBackendFallback(UserWarning):
    """A requested engine could not take the problem and another one ran.

    Raised once per ``(function, shape-signature, dtype, backend)`` per process.
    ``NITRIX_SILENCE_FALLBACK=1`` silences it, ``NITRIX_STRICT_BACKEND=1`` turns
    it into :class:`NitrixBackendError`.
    """


class NitrixBackendError(RuntimeError):
    """A backend cannot be honoured on this host, or strict mode forbade a fallback."""


def _env_flag(name: str) -> bool:
    return os.environ.get(name, "0").lower() in ("1", "true", "yes", "on")


def silence_fallback() -> bool:
    return _env_flag("NITRIX_SILENCE_FALLBACK")


def strict_backend() -> bool:
    return _env_flag("NITRIX_STRICT_BACKEND")


def env_backend() -> Optional[str]:
    value = os.environ.get("NITRIX_BACKEND")
    if value is None:
        return None
    value = value.strip().lower()
    if value not in _VALID_BACKENDS:
        raise NitrixBackendError(f"NITRIX_BACKEND={value!r} not in {_VALID_BACKENDS!r}")
    return value


# --- reproducibility switch (reference _internal/config.py:78-149) -----------
_reproducible: contextvars.ContextVar[Optional[bool]] = contextvars.ContextVar("nitrix_b200_reproducible", default=None)


def reproducible_enabled() -> bool:
    override = _reproducible.get()
    if override is not None:
        return override
    return _env_flag("NITRIX_REPRODUCIBLE")


@contextlib.contextmanager
def reproducible(enabled: bool = True) -> Iterator[None]:
    """Within the block ``backend='auto'`` resolves to the fp32 CUDA-core family."""
    token = _reproducible.set(bool(enabled))
    try:
        yield
    finally:
        _reproducible.reset(token)


_sm100_by_device: dict = {}


def has_sm100_device() -> bool:
    """True when the current CUDA device is a compute-capability 10.x part (remembered per device index)."""
    try:
        import torch

        if not torch.cuda.is_available():
            return False
        dev = torch.cuda.current_device()
        known = _sm100_by_device.get(dev)
        if known is None:
            known = torch.cuda.get_device_capability(dev)[0] == 10
            _sm100_by_device[dev] = known
        return known
    except Exception:
        return False


def auto_backend() -> ResolvedBackend:
    if reproducible_enabled():
        return "cuda-simt"
    return "cuda-sm100"


def resolve_backend(backend: str) -> ResolvedBackend:
    """Three-level resolution: keyword > ``NITRIX_BACKEND`` > auto."""
    if backend not in _VALID_BACKENDS:
        raise NitrixBackendError(f"backend={backend!r} not in {_VALID_BACKENDS!r}")
    if backend == "auto":
        env = env_backend()
        if env is not None and env != "auto":
            backend = env
        else:
            backend = auto_backend()
    if backend == "jax":
        raise NitrixBackendError(
            "backend='jax' (the reference's host implementation) is not part of this library; "
            "use 'auto', 'cuda-sm100' or 'cuda-simt'."
        )
    if backend == "pallas-cuda":
        backend = "cuda-sm100"
    if not has_sm100_device():
        raise NitrixBackendError(
            f"backend={backend!r} needs a Blackwell (sm_100) CUDA device and none is visible; "
            "this library has no host fallback."
        )
    return backend  # type: ignore[return-value]


_warned_keys: set[tuple[str, str, str, str]] = set()
_warned_lock = threading.Lock()


def _shape_signature(*shapes: Any) -> str:
    parts = []
    for s in shapes:
        if s is None:
            parts.append("None")
        elif isinstance(s, (tuple, list)):
            parts.append("x".join(str(d) for d in s))
        else:
            parts.append(str(s))
    return ";".join(parts)


def fallback(*, function: str, requested: str, resolved: str, reason: str,
             shapes: tuple = (), dtype: Any = None) -> str:
    """Warn once (or raise under strict mode) that ``resolved`` runs instead of ``requested``."""
    if requested == resolved:
        return resolved
    if strict_backend():
        raise NitrixBackendError(
            f"{function}: requested backend={requested!r} but would fall back to {resolved!r} "
            f"({reason}). NITRIX_STRICT_BACKEND=1 converted this to an error."
        )
    if silence_fallback():
        return resolved
    key = (function, _shape_signature(*shapes), str(dtype), requested)
    with _warned_lock:
        if key in _warned_keys:
            return resolved
        _warned_keys.add(key)
    warnings.warn(
        f"{function}: falling back to backend={resolved!r} from {requested!r}: {reason}. "
        "Set NITRIX_SILENCE_FALLBACK=1 to suppress this warning, or NITRIX_STRICT_BACKEND=1 "
        "to convert it to an error.",
        category=NitrixBackendFallback,
        stacklevel=3,
    )
    return resolved


def reset_fallback_state() -> None:
    with _warned_lock:
        _warned_keys.clear()


__all__ = [
    "Backend", "ResolvedBackend", "NitrixBackendFallback", "NitrixBackendError", "auto_backend",
    "env_backend", "fallback", "resolve_backend", "reset_fallback_state", "silence_fallback",
    "strict_backend", "reproducible", "reproducible_enabled", "has_sm100_device",
]
