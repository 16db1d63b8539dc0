"""The backward entry point for callers that cannot allocate device memory.

``nb200_sdpa_bwd_static_scratch`` serves hosts that own all device memory
themselves and give the library no way to get scratch (a plug-in under a
framework without a scratch allocator, code running while allocation is
forbidden).  It must give what ``nb200_sdpa_bwd`` gives, from a scratch array
built into the library.  Driven here through the C ABI with ctypes, twice in a
row on different problems, so that contents left behind by the first call
cannot leak into the second; collected last on purpose.
"""
import ctypes as C

import pytest
import torch

import _cases

pytestmark = pytest.mark.gpu


def _backward_both(name, dtype, want_dbias, **shape):
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import attention as att

    lib = _cabi.lib()
    q, k, v, kw = _cases.kernel_case(name, **shape)
    b, h, s, d = q.shape
    t = k.shape[2]
    q, k, v = (x.to(dtype).cuda() for x in (q, k, v))
    bias = kw.get("bias")
    mask = kw.get("mask")
    bias4 = None if bias is None else att._to_own_extent(bias.to(dtype).cuda(), (b,), h, s, t)
    mask4 = None if mask is None else att._to_own_extent(mask.cuda(), (b,), h, s, t)
    causal = bool(kw.get("causal", False))
    scale = d ** -0.5
    out, lse = att.sdpa_forward(q, k, v, bias4, mask4, scale=scale, causal=causal)
    dout = torch.randn(out.shape, generator=torch.Generator().manual_seed(5)).to(dtype).cuda()
    want = att.sdpa_backward(q, k, v, bias4, mask4, out, lse, dout, scale=scale, causal=causal,
                             want_dbias=want_dbias)

    # the same call, but through the no-allocation entry point; no workspace is passed
    p = _cabi.new_params()
    att._fill_common(p, q, k, v, out, lse, bias4, att._mask_bytes(mask4), scale, causal, _cabi.KERNEL_AUTO, None)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    p.dout, p.dq, p.dk, p.dv = dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    for field, ten in (("dout_stride", dout), ("dq_stride", dq), ("dk_stride", dk), ("dv_stride", dv)):
        getattr(p, field)[:] = list(ten.stride())
    dbias = None
    if want_dbias:
        dbias = torch.empty_like(bias4)
        p.dbias = dbias.data_ptr()
        p.dbias_stride[:] = list(dbias.stride())
    before = torch.cuda.memory_allocated()
    rc = lib.nb200_sdpa_bwd_static_scratch(C.byref(p), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0, _cabi.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    return (dq, dk, dv, dbias), want


def _close(got, want, dtype):
    for a, b in zip(got, want):
        if b is None:
            assert a is None
            continue
        err = float((a.double() - b.double()).abs().max())
        ref = float(b.double().abs().max()) + 1e-30
        if dtype == torch.float32:
            assert err / ref < 1e-4, err / ref       # the fp32 budget of the parity tests
        else:
            assert err < 2e-2 * max(1.0, ref), err   # the bf16 / fp16 budget of the parity tests


def test_static_scratch_backward_matches_regular_backward_twice():
    # first call: broadcast bias -> both the delta rows and the fp32 dbias accumulator live in the array
    got, want = _backward_both("bias_mask", torch.float32, True, s=96, t=160, d=32)
    _close(got, want, torch.float32)
    # second call, smaller and different: stale contents of the first must not matter
    got, want = _backward_both("bias_causal", torch.bfloat16, True, s=64, t=64, d=64)
    _close(got, want, torch.bfloat16)


def test_static_scratch_with_tensor_core_backwards_after_a_larger_call():
    """The tensor-core backwards keep more in the array than delta: packed mask words (row-major, key-major and the
    per-sequence key counts) and, at head dim 64 without a bias gradient, the fp32 dq sums -- all of which must start
    from zero although the array still holds an earlier, larger call's contents."""
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import attention as att

    def plans_tc(name, dtype, want_dbias, **shape):
        q, k, v, kw = _cases.kernel_case(name, **shape)
        b, h, s, _ = q.shape
        t = k.shape[2]
        bias, mask = kw.get("bias"), kw.get("mask")
        b4 = None if bias is None else att._to_own_extent(bias.to(dtype).cuda(), (b,), h, s, t)
        m4 = None if mask is None else att._to_own_extent(mask.cuda(), (b,), h, s, t)
        return att.planned_kernel(q.to(dtype).cuda(), k.to(dtype).cuda(), v.to(dtype).cuda(), b4, m4,
                                  causal=bool(kw.get("causal", False)), which=_cabi.PASS_BWD,
                                  want_dbias=want_dbias) == _cabi.KERNEL_TCGEN05

    # a larger call first: it leaves dq sums and mask words all over the array
    big = dict(b=2, h=4, s=512, t=512, d=64)
    assert plans_tc("mask", torch.bfloat16, False, **big)
    got, want = _backward_both("mask", torch.bfloat16, False, **big)
    _close(got, want, torch.bfloat16)
    # merged backward (head dim 64, 4-D mask, no bias gradient): dq accumulator + both mask copies
    small = dict(b=2, h=2, s=128, t=256, d=64)
    assert plans_tc("mask", torch.bfloat16, False, **small)
    got, want = _backward_both("mask", torch.bfloat16, False, **small)
    _close(got, want, torch.bfloat16)
    # key padding at head dim 64: the per-sequence key counts are formed by atomicMax and must start at zero
    assert plans_tc("key_padding", torch.float16, False, **small)
    got, want = _backward_both("key_padding", torch.float16, False, **small)
    _close(got, want, torch.float16)
    # head dim 128 with a per-batch bias gradient and a mask: query-major + key-major kernels
    d128 = dict(b=2, h=2, s=256, t=128, d=128)
    assert plans_tc("full_bias_mask", torch.bfloat16, True, **d128)
    got, want = _backward_both("full_bias_mask", torch.bfloat16, True, **d128)
    _close(got, want, torch.bfloat16)
    # a bias shared by the batch, gradient summed in the array's fp32 accumulator by the tensor-core kernels
    assert plans_tc("bias_causal", torch.bfloat16, True, **small)
    got, want = _backward_both("bias_causal", torch.bfloat16, True, **small)
    _close(got, want, torch.bfloat16)


def test_static_scratch_rejects_oversized_problems():
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import attention as att

    # delta alone needs B*H*S*4 bytes: 4 * 16 * 65536 * 4 = 16 MiB > the 8 MiB array
    B, H, S, D = 4, 16, 65536, 64
    x = torch.empty(1, device="cuda", dtype=torch.bfloat16)
    p = _cabi.new_params()
    p.dtype = _cabi.BF16
    p.B, p.H, p.S, p.T, p.D, p.Dv = B, H, S, 128, D, D
    for f in ("q", "k", "v", "out", "lse", "dout", "dq", "dk", "dv"):
        setattr(p, f, x.data_ptr())
    for f in ("q_stride", "out_stride", "dout_stride", "dq_stride"):
        getattr(p, f)[:] = [H * S * D, S * D, D, 1]
    for f in ("k_stride", "v_stride", "dk_stride", "dv_stride"):
        getattr(p, f)[:] = [H * 128 * D, 128 * D, D, 1]
    p.scale, p.bh_end = 0.125, B * H
    rc = _cabi.lib().nb200_sdpa_bwd_static_scratch(C.byref(p), None)
    assert rc == _cabi.ERR_WORKSPACE
    assert "built-in scratch" in _cabi.last_error()
