"""Seeded attention problems shared by the parity tests, the smoke entry and the benchmark.

Small cases follow the reference's kernel test fixtures
(``tests/test_nn_attention_kernel.py:46-81``: per-tensor ``RandomState`` seeds
0..4 for q, k, v, bias, mask; mask ``rand > 0.3`` with key 0 kept).  The
``config*`` builders produce the five benchmark workloads, optionally shrunk.
"""
from __future__ import annotations

import numpy as np
import torch


def _randn(shape, seed, std=1.0):
    return torch.from_numpy((np.random.RandomState(seed).standard_normal(shape) * std).astype(np.float32))


def kernel_case(name, *, b=2, h=2, s=128, t=None, d=64, dv=None):
    """(q, k, v, kwargs) on the CPU in fp32; names as in the reference kernel tests plus extras."""
    if t is None:
        t = 256 if name == "cross" else s
    dv = d if dv is None else dv
    q, k, v = _randn((b, h, s, d), 0), _randn((b, h, t, d), 1), _randn((b, h, t, dv), 2)
    kw = {}
    if name in ("bias", "bias_causal", "bias_mask"):
        kw["bias"] = _randn((h, s, t), 3)  # shared over batch, as in the reference test
    if name in ("full_bias", "full_bias_mask"):
        kw["bias"] = _randn((b, h, s, t), 3)
    if name in ("causal", "bias_causal"):
        kw["causal"] = True
    if name in ("mask", "bias_mask", "full_bias_mask"):
        m = np.random.RandomState(4).rand(b, h, s, t) > 0.3
        m[..., 0] = True
        kw["mask"] = torch.from_numpy(m)
    if name == "mask_b1st":  # (B, 1, S, T): shared over heads
        m = np.random.RandomState(4).rand(b, 1, s, t) > 0.1
        m[..., 0] = True
        kw["mask"] = torch.from_numpy(m)
    if name == "key_padding":
        lens = np.random.RandomState(4).randint(max(1, t // 8), t + 1, size=b)
        kw["mask"] = torch.from_numpy(np.arange(t)[None, :] < lens[:, None]).reshape(b, 1, 1, t)
    if name == "key_bias":  # per-key bias (1, H, 1, T)
        kw["bias"] = _randn((1, h, 1, t), 3)
    return q, k, v, kw


def config1():
    """fp32 B=2 H=4 L=256 D=64, bias (B,H,L,L), key mask with the last 32 keys of batch 1 masked.
    One RandomState(0) stream drawn in the order q, k, v, bias."""
    rng = np.random.RandomState(0)
    B, H, L, D = 2, 4, 256, 64
    draw = lambda *shape: torch.from_numpy(rng.standard_normal(shape).astype(np.float32))
    q, k, v, bias = draw(B, H, L, D), draw(B, H, L, D), draw(B, H, L, D), draw(B, H, L, L)
    mask = torch.ones(B, 1, 1, L, dtype=torch.bool)
    mask[1, ..., -32:] = False
    return q, k, v, dict(bias=bias, mask=mask, scale=1.0 / 8.0)


def alibi_bias(H, L, dtype=torch.float32, device="cpu"):
    """-slope_h * |i - j| with slope_h = 2^(-8 (h+1) / H), shape (1, H, L, L)."""
    slopes = torch.pow(2.0, -8.0 * (torch.arange(H, device=device, dtype=torch.float32) + 1) / H)
    idx = torch.arange(L, device=device, dtype=torch.float32)
    dist = (idx[:, None] - idx[None, :]).abs()
    return (-slopes[:, None, None] * dist[None]).unsqueeze(0).to(dtype)


def config2(B=8, H=16, L=2048, D=64, dtype=torch.bfloat16, device="cpu", seed=0):
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda: torch.randn(B, H, L, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    return mk(), mk(), mk(), dict(bias=alibi_bias(H, L, dtype, device), causal=True)


def config3(B=4, H=32, L=4096, D=128, dtype=torch.bfloat16, device="cpu", seed=0):
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda: torch.randn(B, H, L, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    q, k, v = mk(), mk(), mk()
    bias = torch.empty(B, H, L, L, device=device, dtype=dtype)
    for b in range(B):  # chunked so the fp32 temporary stays small
        bias[b] = (torch.randn(H, L, L, generator=g, device=device, dtype=torch.float32) * 0.5).to(dtype)
    mask = torch.rand(B, 1, L, L, generator=g, device=device) >= 0.1
    mask |= torch.eye(L, dtype=torch.bool, device=device)
    return q, k, v, dict(bias=bias, mask=mask)


def config4(B=32, H=8, L=1024, D=64, dtype=torch.float16, device="cpu", seed=0):
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda: torch.randn(B, H, L, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    lens = torch.from_numpy(np.random.RandomState(4).randint(max(1, L // 8), L + 1, size=B)).to(device)
    mask = (torch.arange(L, device=device)[None, :] < lens[:, None]).reshape(B, 1, 1, L)
    return mk(), mk(), mk(), dict(mask=mask)


def config5(B=1, H=16, L=65536, D=128, dtype=torch.bfloat16, device="cpu", seed=0):
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda: torch.randn(B, H, L, D, generator=g, device=device, dtype=torch.float32).to(dtype)
    bias = torch.randn(1, H, 1, L, generator=g, device=device, dtype=torch.float32).to(dtype)
    return mk(), mk(), mk(), dict(bias=bias, causal=True)
