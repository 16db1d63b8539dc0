"""The benchmark configurations at their full sizes (C2-C5: bf16/fp16, up to L = 65536).

The CPU oracle cannot finish a whole configuration in seconds (C5's score matrix alone is 275 GB), so parity is
checked two ways:

* sampled rows: for a few (batch, head) pairs and a block of query rows the oracle's arithmetic is restated on the
  GPU in fp32 for those rows only (rows x T scores fit easily) and compared with the kernels' ``out`` and ``dq`` rows
  -- the same formula as ``oracle/sdpa_oracle.py`` (scale, + bias, mask / causal -> -inf, softmax, weights @ v and
  the closed-form row gradient);
* sampled key blocks: for three 128-key blocks (first tile, a middle tile, last tile) the same restatement walks all
  query rows in chunks and accumulates ``dv = p^T dO``, ``dk = scale ds^T q`` and the ``dbias`` columns of those keys,
  which are compared by value with the kernels' ``dk``, ``dv`` and ``dbias``;
* size-independent identities over the whole result: softmax rows sum to one, so ``sum_keys dv = sum_queries dout``;
  the score gradient of a row sums to zero, so every dbias row sums to zero; logits are bilinear in (q, k), so
  ``<q, dq> = <k, dk>`` per (batch, head).

Tolerance: the low-precision budget of the path, 2e-2 max-abs (scaled by the reference's magnitude above 1).
"""
import math

import pytest
import torch

import _cases

pytestmark = pytest.mark.gpu

ABS = 2e-2


def _rows_reference(q, k, v, dout, bias, mask, causal, scale, b, h, rows):
    """fp32 restatement of the oracle for query rows `rows` of pair (b, h): returns out rows and dq rows."""
    f = torch.float32
    qr = q[b, h, rows].to(f)
    kk, vv = k[b, h].to(f), v[b, h].to(f)
    s = (qr @ kk.T) * scale
    T = kk.shape[0]
    if bias is not None:
        bb = bias[b if bias.shape[0] > 1 else 0, h if bias.shape[1] > 1 else 0]
        s = s + (bb[rows] if bb.shape[0] > 1 else bb).to(f)
    keep = torch.ones(len(rows), T, dtype=torch.bool, device=q.device)
    if mask is not None:
        mm = mask[b if mask.shape[0] > 1 else 0, h if mask.shape[1] > 1 else 0]
        keep &= mm[rows] if mm.shape[0] > 1 else mm
    if causal:
        keep &= torch.arange(T, device=q.device)[None, :] <= rows[:, None]
    s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    out = p @ vv
    g = dout[b, h, rows].to(f)
    dp = g @ vv.T
    ds = p * (dp - (dp * p).sum(-1, keepdim=True))
    dq = (ds @ kk) * scale
    return out, dq


def _keys_reference(q, k, v, dout, bias, mask, causal, scale, b, h, key_blocks, chunk=2048):
    """fp32 restatement of the oracle's gradients for the keys of `key_blocks` (lists of 128 key indices) of pair
    (b, h): returns per block (dk, dv, dbias columns).  Queries are walked in chunks of `chunk` rows; each chunk
    forms its full score rows (so lse and delta are the restatement's own, not the kernels'), then
    p = softmax, dv += p^T dO, ds = p (dP - delta), dk += scale ds^T q, dbias[:, keys] = ds[:, keys]."""
    f = torch.float32
    dev = q.device
    S, T = q.shape[2], k.shape[2]
    kk, vv = k[b, h].to(f), v[b, h].to(f)
    acc = [dict(dk=torch.zeros(len(kb), kk.shape[1], device=dev), dv=torch.zeros(len(kb), vv.shape[1], device=dev),
                db=torch.zeros(S, len(kb), device=dev)) for kb in key_blocks]
    for r0 in range(0, S, chunk):
        rows = torch.arange(r0, min(r0 + chunk, S), device=dev)
        qr, g = q[b, h, rows].to(f), dout[b, h, rows].to(f)
        s = (qr @ kk.T) * scale
        if bias is not None:
            bb = bias[b if bias.shape[0] > 1 else 0, h if bias.shape[1] > 1 else 0]
            s = s + (bb[rows] if bb.shape[0] > 1 else bb).to(f)
        keep = torch.ones(len(rows), T, dtype=torch.bool, device=dev)
        if mask is not None:
            mm = mask[b if mask.shape[0] > 1 else 0, h if mask.shape[1] > 1 else 0]
            keep &= mm[rows] if mm.shape[0] > 1 else mm
        if causal:
            keep &= torch.arange(T, device=dev)[None, :] <= rows[:, None]
        s = s.masked_fill(~keep, float("-inf"))
        p = torch.softmax(s, dim=-1)
        del s, keep
        delta = ((p @ vv) * g).sum(-1, keepdim=True)
        for kb, a in zip(key_blocks, acc):
            pk = p[:, kb]
            ds = pk * (g @ vv[kb].T - delta)
            a["dv"] += pk.T @ g
            a["dk"] += (ds.T @ qr) * scale
            a["db"][rows] = ds
        del p
    return acc


def _close(got, ref, what):
    err = float((got.detach().float() - ref.detach().float()).abs().max())
    lim = ABS * max(1.0, float(ref.abs().max()))
    assert err < lim, (what, err, lim)


@pytest.mark.parametrize("name", ["config2", "config3", "config4", "config5"])
def test_full_size_configuration(name):
    from nitrix_b200.nn import attention as att

    dev = torch.device("cuda", 0)
    q, k, v, kw = getattr(_cases, name)(device=dev)
    bias, mask, causal = kw.get("bias"), kw.get("mask"), kw.get("causal", False)
    B, H, L, D = q.shape
    scale = 1.0 / math.sqrt(D)
    want_dbias = name == "config3"
    dout = torch.randn(q.shape, generator=torch.Generator(device=dev).manual_seed(11), device=dev).to(q.dtype)
    leaves = [x.requires_grad_(True) for x in (q, k, v)]
    if want_dbias:
        bias = bias.requires_grad_(True)
        leaves.append(bias)
    out = att.scaled_dot_product_attention(q, k, v, bias=bias, mask=mask, causal=causal, scale=scale, backend="cuda-sm100")
    grads = torch.autograd.grad(out, leaves, grad_outputs=dout)
    torch.cuda.synchronize()
    dq, dk, dv = grads[:3]
    from nitrix_b200 import _cabi
    assert _cabi.lib().nb200_device_status(0) == 0
    for t in (out, dq, dk, dv):
        assert torch.isfinite(t).all()

    # ---- sampled rows against the fp32 restatement of the oracle ----
    b4 = None if bias is None else att._to_own_extent(bias.detach(), (B,), H, L, L)
    m4 = None if mask is None else att._to_own_extent(mask, (B,), H, L, L)
    picks = [(0, 0, 0), (B - 1, H - 1, L - 128), (B // 2, H // 3, (L // 2 // 128) * 128 + 64)]
    for (b, h, r0) in picks:
        rows = torch.arange(r0, min(r0 + 128, L), device=dev)
        ref_out, ref_dq = _rows_reference(q.detach(), k.detach(), v.detach(), dout, b4, m4, causal, scale, b, h, rows)
        _close(out[b, h, rows], ref_out, (name, "out", b, h, r0))
        _close(dq[b, h, rows], ref_dq, (name, "dq", b, h, r0))

    # ---- sampled key blocks: dk, dv (and dbias columns) by value ----
    # three 128-key blocks in two (batch, head) pairs: the first tile, a middle tile at an odd offset, the last tile
    torch.backends.cuda.matmul.allow_tf32 = False
    first, mid, last = 0, (L // 2 // 128) * 128 + 128, L - 128
    plan = [((0, 0), [first, mid]), ((B - 1, H - 1), [last])]
    for (b, h), starts in plan:
        blocks = [torch.arange(k0, k0 + 128, device=dev) for k0 in starts]
        refs = _keys_reference(q.detach(), k.detach(), v.detach(), dout, b4, m4, causal, scale, b, h, blocks)
        for kb, r in zip(blocks, refs):
            k0 = int(kb[0])
            _close(dk[b, h, kb], r["dk"], (name, "dk", b, h, k0))
            _close(dv[b, h, kb], r["dv"], (name, "dv", b, h, k0))
            if want_dbias:
                _close(grads[3][b, h][:, kb], r["db"], (name, "dbias", b, h, k0))

    # ---- identities over the whole result ----
    # sum over keys of dv == sum over queries of dout (softmax rows sum to one); fp32 sums of 16-bit values
    _close(dv.float().sum(2), dout.float().sum(2), (name, "sum dv"))  # relative to its own magnitude via _close
    # <q, dq> == <k, dk> per (batch, head)
    lhs = (q.detach().float() * dq.float()).sum((2, 3))
    rhs = (k.detach().float() * dk.float()).sum((2, 3))
    assert float((lhs - rhs).abs().max()) < ABS * max(1.0, float(rhs.abs().max())), (name, "bilinear identity")
    if want_dbias:
        dbias = grads[3]
        assert dbias.shape == bias.shape and dbias.dtype == bias.dtype
        rowsum = dbias.float().sum(-1)
        # a row's score gradient sums to zero; each of its L entries carries a 16-bit rounding error
        assert float(rowsum.abs().max()) < ABS * max(1.0, float(dbias.float().abs().sum(-1).max()) * 2 ** -8), (name, "dbias rows")
        # masked entries get an exactly-zero gradient
        assert int((dbias.detach().masked_fill(m4, 0) != 0).sum()) == 0
