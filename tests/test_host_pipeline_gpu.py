"""The host-operand pipeline (batch chunks over copy-in / kernel / copy-out streams) gives what the direct
device call gives: chunking over the batch changes no (batch, head) pair's result."""
import pytest
import torch

import _cases

pytestmark = pytest.mark.gpu


def _direct(att, q, k, v, dout, bias, mask, causal, scale, want_dbias):
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v)]
    b = bias
    if bias is not None and want_dbias:
        b = bias.clone().requires_grad_(True)
        leaves.append(b)
    out = att.scaled_dot_product_attention(*leaves[:3], bias=b, mask=mask, causal=causal, scale=scale)
    grads = torch.autograd.grad(out, leaves, grad_outputs=dout)
    names = ["dq", "dk", "dv"] + (["dbias"] if len(leaves) == 4 else [])
    return {"out": out.detach(), **dict(zip(names, grads))}


@pytest.mark.parametrize("case,shape,want_dbias,chunks", [
    ("bias_causal", dict(b=4, h=2, s=256, t=256, d=64), False, 4),     # bias shared by the batch: goes up once
    ("full_bias_mask", dict(b=3, h=2, s=256, t=256, d=128), True, 2),  # per-batch bias and mask, dbias, ragged chunks
    ("key_padding", dict(b=2, h=2, s=128, t=256, d=64), False, 8),     # more chunks asked for than batch rows
    ("bias_causal", dict(b=4, h=2, s=128, t=128, d=64), True, 4),      # gradient of a bias shared by the batch: sums over all chunks
])
def test_pipeline_matches_direct_call(case, shape, want_dbias, chunks):
    from nitrix_b200.nn import attention as att
    from nitrix_b200.nn.host_pipeline import HostPipeline

    q, k, v, kw = _cases.kernel_case(case, **shape)
    dt = torch.bfloat16
    dev = torch.device("cuda", 0)
    q, k, v = (x.to(dt) for x in (q, k, v))
    bias, mask, causal = kw.get("bias"), kw.get("mask"), kw.get("causal", False)
    B, H, S, D = q.shape
    T = k.shape[2]
    if bias is not None and not (want_dbias and bias.dim() == 3):
        bias = att._to_own_extent(bias.to(dt), (B,), H, S, T)
    elif bias is not None:
        bias = bias.to(dt)      # stays (H, S, T): a 3-D bias shared by the batch, with a gradient
    if mask is not None:
        mask = att._to_own_extent(mask, (B,), H, S, T)
    dout = torch.randn(q.shape[:-1] + (v.shape[-1],), generator=torch.Generator().manual_seed(3)).to(dt)
    scale = D ** -0.5
    host = {n: t.contiguous().pin_memory() for n, t in (("q", q), ("k", k), ("v", v), ("dout", dout))}
    if bias is not None:
        host["bias"] = bias.contiguous().pin_memory()
    if mask is not None:
        host["mask"] = mask.contiguous().pin_memory()
    pipe = HostPipeline(host, device=dev, causal=causal, scale=scale, want_dbias=want_dbias, chunks=chunks)
    for _ in range(2):          # the second run reuses the staging buffers while the first one's copies drain
        got = pipe.run()
    torch.cuda.synchronize()
    ref = _direct(att, q.to(dev), k.to(dev), v.to(dev), dout.to(dev), None if bias is None else bias.to(dev),
                  None if mask is None else mask.to(dev), causal, scale, want_dbias)
    assert set(got) == set(ref)
    for name, r in ref.items():
        g = got[name]
        assert tuple(g.shape) == tuple(r.shape), name
        # same kernels on the same values; only dq of the merged backward (fp32 reductions) may differ in the last bit
        assert float((g.float() - r.cpu().float()).abs().max()) <= 2e-2 * max(1.0, float(r.float().abs().max())), name
