"""The multi-GPU slice of the C ABI on the tensor-core family: ``bh_begin / bh_end``.

A rank of an N-GPU job runs the ordinary kernels on a contiguous range of the flattened ``b * H + h`` axis of
shared, full-size buffers.  Here the ranges are run one after the other on one GPU, forward and backward, and must
reproduce one whole-range call exactly (same kernels, same (batch, head) problems; only the merged backward's dq
goes through fp32 reductions whose order may differ in the last bit).
"""
import pytest
import torch

import _cases

pytestmark = pytest.mark.gpu


def _prep(name, dtype, **shape):
    from nitrix_b200.nn import attention as att

    q, k, v, kw = _cases.kernel_case(name, **shape)
    b, h, s, _ = q.shape
    t = k.shape[2]
    q, k, v = (x.to(dtype).cuda() for x in (q, k, v))
    bias, mask = kw.get("bias"), kw.get("mask")
    bias4 = None if bias is None else att._to_own_extent(bias.to(dtype).cuda(), (b,), h, s, t)
    mask4 = None if mask is None else att._to_own_extent(mask.cuda(), (b,), h, s, t)
    return q, k, v, bias4, mask4, bool(kw.get("causal", False))


def _run_ranges(q, k, v, bias, mask, causal, want_dbias, ranges):
    """Forward + backward over the given bh ranges into one set of buffers; returns (out, lse, dq, dk, dv, dbias)."""
    from nitrix_b200 import _cabi
    from nitrix_b200.nn import attention as att

    scale = q.shape[-1] ** -0.5
    assert att.planned_kernel(q, k, v, bias, mask, scale=scale, causal=causal) == _cabi.KERNEL_TCGEN05
    assert att.planned_kernel(q, k, v, bias, mask, scale=scale, causal=causal, which=_cabi.PASS_BWD,
                              want_dbias=want_dbias) == _cabi.KERNEL_TCGEN05
    out = torch.full(q.shape, float("nan"), dtype=q.dtype, device=q.device)
    lse = torch.full(q.shape[:3], float("nan"), dtype=torch.float32, device=q.device)
    dout = torch.randn(q.shape, generator=torch.Generator().manual_seed(5)).to(q.dtype).cuda()
    nan_like = lambda x: torch.full(x.shape, float("nan"), dtype=x.dtype, device=x.device)
    grads = (nan_like(q), nan_like(k), nan_like(v), nan_like(bias) if want_dbias else None)
    for r in ranges:
        att.sdpa_forward(q, k, v, bias, mask, scale=scale, causal=causal, bh_range=r, out=out, lse=lse)
    for r in ranges:
        att.sdpa_backward(q, k, v, bias, mask, out, lse, dout, scale=scale, causal=causal, want_dbias=want_dbias,
                          bh_range=r, grads=grads)
    torch.cuda.synchronize()
    assert _cabi.lib().nb200_device_status(torch.cuda.current_device()) == 0, _cabi.last_error()
    return (out, lse, *grads)


CASES = [
    # (case, dtype, shape, want_dbias, what it exercises)
    ("bias_causal", torch.bfloat16, dict(b=2, h=4, s=384, t=384, d=64), False),      # merged backward, shared tiled bias
    ("mask", torch.float16, dict(b=2, h=3, s=256, t=256, d=64), False),              # merged backward, 4-D mask
    ("full_bias_mask", torch.bfloat16, dict(b=2, h=3, s=256, t=384, d=128), True),   # query- / key-major, dbias tiles
    ("full_bias", torch.bfloat16, dict(b=3, h=2, s=256, t=256, d=64), True),         # D = 64 with a bias gradient
    ("key_padding", torch.float16, dict(b=8, h=4, s=512, t=512, d=64), False),       # C4-shaped: batches per rank
    ("key_bias", torch.bfloat16, dict(b=1, h=8, s=1024, t=1024, d=128), False),      # C5-shaped: heads per rank
]


@pytest.mark.parametrize("case,dtype,shape,want_dbias", CASES)
def test_bh_ranges_equal_whole_call(case, dtype, shape, want_dbias):
    q, k, v, bias, mask, causal = _prep(case, dtype, **shape)
    if case == "key_bias":
        causal = True
    B, H = q.shape[:2]
    n = B * H
    whole = _run_ranges(q, k, v, bias, mask, causal, want_dbias, [(0, n)])
    if case == "key_padding":      # 8 batches over 4 "ranks": 2 batches each, as the 32 -> 4 per GPU split
        ranges = [(i * 2 * H, (i + 1) * 2 * H) for i in range(4)]
    elif case == "key_bias":       # 8 heads over 4 "ranks": 2 heads each, as the 16 -> 2 per GPU split
        ranges = [(i * 2, (i + 1) * 2) for i in range(4)]
    else:                          # an uneven split that cuts through a batch
        ranges = [(0, n // 2 + 1), (n // 2 + 1, n)]
    parts = _run_ranges(q, k, v, bias, mask, causal, want_dbias, ranges)
    names = ("out", "lse", "dq", "dk", "dv", "dbias")
    merged = True   # dq of the one-kernel backwards (head dim 64 without dbias, head dim 128) goes through fp32 atomics
    for name, a, b in zip(names, parts, whole):
        if b is None:
            assert a is None
            continue
        assert not torch.isnan(a.float()).any(), name      # every (batch, head) was covered by some range
        if name == "dq" and merged:
            # fp32 atomics: the order of the partial sums may differ between the two runs
            assert float((a.float() - b.float()).abs().max()) <= 2e-2 * max(1.0, float(b.float().abs().max())), name
        else:
            assert torch.equal(a, b), name


def test_partial_range_leaves_other_pairs_untouched():
    q, k, v, bias, mask, causal = _prep("bias_causal", torch.bfloat16, b=2, h=2, s=256, t=256, d=64)
    from nitrix_b200.nn import attention as att

    scale = 0.125
    out = torch.full(q.shape, 7.0, dtype=q.dtype, device=q.device)
    lse = torch.full(q.shape[:3], 7.0, dtype=torch.float32, device=q.device)
    att.sdpa_forward(q, k, v, bias, mask, scale=scale, causal=causal, bh_range=(1, 3), out=out, lse=lse)
    torch.cuda.synchronize()
    flat = out.reshape(4, -1)
    assert (flat[0] == 7.0).all() and (flat[3] == 7.0).all()
    assert not (flat[1] == 7.0).all() and not (flat[2] == 7.0).all()
