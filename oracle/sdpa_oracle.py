"""CPU oracle for scaled-dot-product attention -- TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the test-suite, the smoke
entry and the benchmark's CPU-baseline / reference arm may import it.  The
shipped package (``nitrix_b200``) never imports anything from ``oracle``.

It restates, operation for operation, the reference's own ``jnp`` attention
path ``reference_scaled_dot_product_attention``
(reference ``src/nitrix/nn/attention/_reference.py:80-181``):

* up-cast rule (``:140-150``): output dtype is the common result type of q, k, v;
  the accumulation dtype is that type promoted with float32, so bf16/fp16 inputs
  are computed entirely in float32 and cast back once at the end, fp64 stays fp64;
* optional QK-norm (``:52-77``, eps 1e-6 ``:32``) on the up-cast q and k;
* ``logits = einsum('...hsd,...htd->...hst', q, k)`` (``:155-160``), then
  ``* scale`` (``:161``), then ``+ bias`` in the accumulation dtype (``:162-163``);
* ``keep = mask & causal`` with ``causal_keep[i, j] = i >= j``, indices aligned at
  zero even when ``s != t`` (``:165-170``); excluded logits become ``-inf`` (``:171-172``);
* ``softmax`` over keys as max-subtracted ``exp`` divided by its sum (``:174``,
  ``jax.nn.softmax``); a fully masked row gives NaN exactly like the reference;
* ``einsum('...hst,...htd->...hsd', weights, v)`` and the final cast (``:175-181``).

The arithmetic the reference delegates to a third-party library (``jnp.einsum``,
``jnp.where``, ``jax.nn.softmax`` of jax >= 0.10.0, the floor pinned by the
reference's ``pyproject.toml:34``; no lock file is in its tree) is restated from
its published definition.  jax cannot be imported where this code runs, so the
oracle is pinned by the reference's own stored vectors instead: the five
``tests/golden/attention_*_float32.npz`` fixtures (forward only).  Four of them
are reproduced to <= 5e-7 max-abs; ``attention_cross`` carries TF32 matmul
rounding from the GPU it was generated on and is reproduced to 1e-3 in true
fp32 and to ~2e-7 once q, k, v and the softmax weights are rounded to TF32
(see :func:`round_to_tf32`).  Gradients have no stored vectors in the
reference: gradient parity is "unpinned by stored values" and rests on autograd
of this restatement cross-checked against the closed form
(:func:`analytic_grads_numpy`) and central finite differences in fp64, which
is the same evidence the reference's own test-suite uses
(``tests/test_nn_attention.py:227-253``).

Two implementations are kept on purpose:

* :func:`reference_sdpa_numpy` -- NumPy, the line-by-line restatement;
* :func:`reference_sdpa_torch` -- the same operations with ``torch`` on the CPU,
  which gives reverse-mode gradients (the reference differentiates its ``jnp``
  path by ordinary autodiff, ``_reference.py:10-13``) and is the timed CPU
  baseline.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple

import numpy as np

QK_RMS_EPS = 1e-6  # reference _reference.py:32
LOG2E = 1.4426950408889634  # reference _kernels/cuda/attention.py:59


def default_scale(head_dim: int) -> float:
    """``1/sqrt(d)`` -- reference ``_reference.py:35-49``."""
    return 1.0 / math.sqrt(float(head_dim))


def _acc_dtype_numpy(*arrays) -> Tuple[np.dtype, np.dtype]:
    """(out_dtype, acc_dtype) following ``_reference.py:140-141``."""
    out = np.result_type(*[a.dtype for a in arrays])
    acc = np.promote_types(out, np.float32)
    return out, acc


def qk_rms_norm_numpy(z: np.ndarray) -> np.ndarray:
    """``z * rsqrt(mean(z^2, -1) + eps)`` -- reference ``_reference.py:52-77``."""
    ms = np.mean(np.square(z), axis=-1, keepdims=True)
    return z * (1.0 / np.sqrt(ms + np.asarray(QK_RMS_EPS, z.dtype))).astype(z.dtype)


def round_to_tf32(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to the 10-bit TF32 mantissa (round-to-nearest-even).

    Only used to show that the reference's ``attention_cross`` fixture was
    produced by TF32 matmuls; it is not part of the oracle's arithmetic.
    """
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 13) & 1
    bits = (bits + 0xFFF + lsb) & ~np.uint64(0x1FFF)
    return bits.astype(np.uint32).view(np.float32).reshape(x.shape)


def reference_sdpa_numpy(
    q: np.ndarray,
    k: np.ndarray,
    v: np.ndarray,
    *,
    bias: Optional[np.ndarray] = None,
    mask: Optional[np.ndarray] = None,
    scale: Optional[float] = None,
    causal: bool = False,
    qk_norm: bool = False,
    tf32_matmul: bool = False,
    return_lse: bool = False,
):
    """Line-by-line NumPy restatement of ``_reference.py:137-181``.

    ``tf32_matmul`` rounds both matmuls' operands to TF32 (diagnostic for the
    ``cross`` fixture only).  With ``return_lse`` the base-2 log-sum-exp of the
    masked logits, ``m + log2(l)`` as the fused reference kernel stores it
    (``_kernels/cuda/attention.py:156``), is returned as well.
    """
    if scale is None:
        scale = default_scale(q.shape[-1])
    out_dtype, acc = _acc_dtype_numpy(q, k, v)
    q = q.astype(acc)
    k = k.astype(acc)
    v = v.astype(acc)
    if qk_norm:
        q = qk_rms_norm_numpy(q)
        k = qk_rms_norm_numpy(k)
    qm, km = (round_to_tf32(q), round_to_tf32(k)) if tf32_matmul else (q, k)
    logits = np.einsum("...hsd,...htd->...hst", qm, km).astype(acc)
    logits = logits * np.asarray(scale, acc)
    if bias is not None:
        logits = logits + bias.astype(acc)
    keep = mask
    if causal:
        s, t = logits.shape[-2], logits.shape[-1]
        causal_keep = np.arange(s)[:, None] >= np.arange(t)[None, :]
        keep = causal_keep if keep is None else (keep & causal_keep)
    if keep is not None:
        logits = np.where(keep, logits, np.asarray(-np.inf, acc))
    with np.errstate(invalid="ignore"):
        m = np.max(logits, axis=-1, keepdims=True)
        e = np.exp(logits - m)
        l = np.sum(e, axis=-1, keepdims=True)
        weights = e / l
    wm, vm = (round_to_tf32(weights), round_to_tf32(v)) if tf32_matmul else (weights, v)
    out = np.einsum("...hst,...htd->...hsd", wm, vm).astype(acc).astype(out_dtype)
    if return_lse:
        with np.errstate(divide="ignore", invalid="ignore"):
            lse2 = (m + np.log(l))[..., 0] * LOG2E
        return out, lse2.astype(np.float32)
    return out


def naive_rowwise_numpy(q, k, v, *, bias=None, mask=None, scale=None, causal=False):
    """Independent per-row fp64 loop (the shape of the reference's own naive
    oracle, ``tests/test_nn_attention.py:76-111``).  Small inputs only."""
    q64, k64, v64 = (np.asarray(a, np.float64) for a in (q, k, v))
    *lead, h, s, d = q64.shape
    t = k64.shape[-2]
    dv = v64.shape[-1]
    if scale is None:
        scale = default_scale(d)
    full = (*lead, h, s, t)
    b_full = None if bias is None else np.broadcast_to(np.asarray(bias, np.float64), full)
    m_full = None if mask is None else np.broadcast_to(np.asarray(mask, bool), full)
    out = np.zeros((*lead, h, s, dv))
    for idx in np.ndindex(*lead, h):
        for i in range(s):
            row = np.empty(t)
            for j in range(t):
                z = float(np.dot(q64[idx][i], k64[idx][j])) * scale
                if b_full is not None:
                    z += b_full[idx][i, j]
                drop = (m_full is not None and not m_full[idx][i, j]) or (causal and j > i)
                row[j] = -np.inf if drop else z
            w = np.exp(row - row.max())
            w /= w.sum()
            out[idx][i] = w @ v64[idx]
    return out


def analytic_grads_numpy(q, k, v, dout, *, bias=None, mask=None, scale=None, causal=False,
                         acc=np.float64):
    """Closed-form gradients of the restatement (no autodiff), in ``acc``.

    With ``P = softmax(S)``: ``dV = P^T dO``; ``dP = dO V^T``;
    ``dS = P * (dP - rowsum(P*dP))``; ``dQ = scale * dS K``; ``dK = scale * dS^T Q``;
    ``dBias = dS`` summed over the axes the bias was broadcast along (the rule
    of the reference's ``_unbroadcast``, ``_kernels/cuda/attention.py:517-544``).
    Returns ``(out, dq, dk, dv, dbias_or_None)`` as ``acc`` arrays.
    """
    if scale is None:
        scale = default_scale(q.shape[-1])
    q_, k_, v_, do_ = (np.asarray(a, acc) for a in (q, k, v, dout))
    logits = np.einsum("...hsd,...htd->...hst", q_, k_) * scale
    if bias is not None:
        logits = logits + np.asarray(bias, acc)
    keep = None if mask is None else np.asarray(mask, bool)
    if causal:
        s, t = logits.shape[-2:]
        ck = np.arange(s)[:, None] >= np.arange(t)[None, :]
        keep = ck if keep is None else (keep & ck)
    if keep is not None:
        logits = np.where(keep, logits, -np.inf)
    m = logits.max(-1, keepdims=True)
    e = np.exp(logits - m)
    p = e / e.sum(-1, keepdims=True)
    out = np.einsum("...hst,...htd->...hsd", p, v_)
    dv = np.einsum("...hst,...hsd->...htd", p, do_)
    dp = np.einsum("...hsd,...htd->...hst", do_, v_)
    ds = p * (dp - np.sum(p * dp, -1, keepdims=True))
    dq = np.einsum("...hst,...htd->...hsd", ds, k_) * scale
    dk = np.einsum("...hst,...hsd->...htd", ds, q_) * scale
    dbias = None
    if bias is not None:
        dbias = unbroadcast_numpy(ds, np.shape(bias))
    # reduce broadcast leading dims of k/v (e.g. shared K across batch) the same way
    dq = unbroadcast_numpy(dq, np.shape(q))
    dk = unbroadcast_numpy(dk, np.shape(k))
    dv = unbroadcast_numpy(dv, np.shape(v))
    return out, dq, dk, dv, dbias


def unbroadcast_numpy(full: np.ndarray, shape: Sequence[int]) -> np.ndarray:
    """Sum ``full`` over the axes along which ``shape`` was broadcast
    (reference ``_kernels/cuda/attention.py:517-544``)."""
    shape = tuple(shape)
    extra = full.ndim - len(shape)
    if extra:
        full = full.sum(axis=tuple(range(extra)))
    axes = tuple(i for i, (a, b) in enumerate(zip(full.shape, shape)) if b == 1 and a != 1)
    if axes:
        full = full.sum(axis=axes, keepdims=True)
    return full.reshape(shape)


# ----------------------------------------------------------------------------
# torch-CPU twin: same operations, differentiable, multi-threaded (CPU baseline)
# ----------------------------------------------------------------------------

def reference_sdpa_torch(q, k, v, *, bias=None, mask=None, scale=None, causal=False,
                         qk_norm=False, acc_dtype=None):
    """The same recipe with torch ops (any device the tensors live on; the
    oracle uses the CPU).  ``acc_dtype`` overrides the accumulation dtype
    (``torch.float64`` for the gradient oracle)."""
    import torch

    if scale is None:
        scale = default_scale(q.shape[-1])
    out_dtype = torch.promote_types(torch.promote_types(q.dtype, k.dtype), v.dtype)
    acc = acc_dtype or torch.promote_types(out_dtype, torch.float32)
    q_, k_, v_ = q.to(acc), k.to(acc), v.to(acc)
    if qk_norm:
        q_ = q_ * torch.rsqrt(q_.square().mean(-1, keepdim=True) + QK_RMS_EPS)
        k_ = k_ * torch.rsqrt(k_.square().mean(-1, keepdim=True) + QK_RMS_EPS)
    logits = torch.einsum("...hsd,...htd->...hst", q_, k_)
    logits = logits * scale
    if bias is not None:
        logits = logits + bias.to(acc)
    keep = mask
    if causal:
        s, t = logits.shape[-2], logits.shape[-1]
        ck = torch.arange(s, device=logits.device)[:, None] >= torch.arange(t, device=logits.device)[None, :]
        keep = ck if keep is None else (keep & ck)
    if keep is not None:
        logits = torch.where(keep, logits, torch.tensor(-math.inf, dtype=acc, device=logits.device))
    weights = torch.softmax(logits, dim=-1)
    out = torch.einsum("...hst,...htd->...hsd", weights, v_)
    return out.to(out_dtype if acc_dtype is None else acc)


def reference_grads_torch(q, k, v, dout, *, bias=None, mask=None, scale=None, causal=False,
                          qk_norm=False, acc_dtype=None, want_dbias=True):
    """Forward + reverse-mode gradients of :func:`reference_sdpa_torch` for the
    upstream cotangent ``dout`` (CPU tensors).  Returns
    ``(out, dq, dk, dv, dbias_or_None)`` in the accumulation dtype (fp32 unless
    ``acc_dtype`` says otherwise), i.e. the reference's fp32 result that
    reduced-precision outputs are compared with."""
    import torch

    acc = acc_dtype or torch.float32
    leaves = [t.detach().to(acc).requires_grad_(True) for t in (q, k, v)]
    b = None
    if bias is not None:
        b = bias.detach().to(acc).requires_grad_(bool(want_dbias))
    out = reference_sdpa_torch(*leaves, bias=b, mask=mask, scale=scale, causal=causal,
                               qk_norm=qk_norm, acc_dtype=acc)
    wrt = leaves + ([b] if (b is not None and want_dbias) else [])
    grads = torch.autograd.grad(out, wrt, grad_outputs=dout.to(acc))
    dq, dk, dv = grads[:3]
    dbias = grads[3] if len(grads) > 3 else None
    return out.detach(), dq, dk, dv, dbias
