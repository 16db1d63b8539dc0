"""GPU parity: the CUDA library (through its C ABI) against the CPU oracle.

Structure follows the reference's kernel tests
(``tests/test_nn_attention_kernel.py``: forward parity ``:83-96``, gradient
parity with loss ``sum(out**2)`` and max-relative error ``:102-140``) plus its
golden corpus (``tests/test_nn_attention.py:41-70``).

Tolerances.  fp32: 1e-4 relative (max-abs error over max-abs reference).
bf16 / fp16: 2e-2 max-abs against the oracle's FP32 result on the same
(already quantised) inputs, for outputs and for gradients.
"""
import pathlib
import warnings

import numpy as np
import pytest
import torch

import _cases
from oracle import sdpa_oracle as O

pytestmark = pytest.mark.gpu

GOLD = pathlib.Path(__file__).parent / "golden"
FP32_REL = 1e-4
LOWP_ABS = 2e-2


def _nb():
    import nitrix_b200
    from nitrix_b200.nn import attention

    return nitrix_b200, attention


def relerr(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-30))


def abserr(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max())


def run_both(q, k, v, kw, dtype, backend, dout_seed=5, want_dbias=True):
    """Library result on the GPU and oracle result on the CPU for the same quantised inputs."""
    _, att = _nb()
    kw = dict(kw)
    bias = kw.pop("bias", None)
    mask = kw.pop("mask", None)
    qd, kd, vd = (x.to(dtype) for x in (q, k, v))
    bd = None if bias is None else bias.to(dtype)
    dout = torch.from_numpy(np.random.RandomState(dout_seed).standard_normal(
        (*q.shape[:-1], v.shape[-1])).astype(np.float32)).to(dtype)
    # oracle in fp32 on the quantised values (fp64 for fp32 inputs)
    acc = torch.float64 if dtype == torch.float32 else torch.float32
    ref = O.reference_grads_torch(qd, kd, vd, dout, bias=bd, mask=mask, acc_dtype=acc,
                                  want_dbias=want_dbias and bias is not None, **kw)
    dev = "cuda"
    leaves = [x.to(dev).requires_grad_(True) for x in (qd, kd, vd)]
    bg = None if bd is None else bd.to(dev).requires_grad_(want_dbias)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = att.scaled_dot_product_attention(*leaves, bias=bg, mask=None if mask is None else mask.to(dev),
                                               backend=backend, **kw)
    wrt = leaves + ([bg] if (bg is not None and want_dbias) else [])
    grads = torch.autograd.grad(out, wrt, grad_outputs=dout.to(dev))
    torch.cuda.synchronize()
    got = [out.detach(), *grads] + ([None] if len(grads) == 3 else [])
    return got, list(ref)


def check(got, ref, dtype, names=("out", "dq", "dk", "dv", "dbias")):
    for name, a, b in zip(names, got, ref):
        if b is None:
            assert a is None, name
            continue
        assert a.shape == b.shape, (name, a.shape, b.shape)
        assert a.dtype == dtype, (name, a.dtype)
        assert torch.isfinite(a).all(), name
        if dtype == torch.float32:
            assert relerr(a, b) < FP32_REL, (name, relerr(a, b))
        else:
            assert abserr(a, b) < LOWP_ABS * max(1.0, float(b.abs().max())), (name, abserr(a, b))


# --------------------------------------------------------------------------
# golden corpus of the reference (fp32; the CUDA-core family)
# --------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["dense", "windowed_bias", "causal", "cross", "qk_norm"])
def test_golden_forward(name):
    nb, att = _nb()
    z = np.load(GOLD / f"attention_{name}_float32.npz")
    kw = {"causal": bool(z["causal"])}
    if "bias" in z.files:
        kw["bias"] = torch.from_numpy(z["bias"]).cuda()
    if "qk_norm" in z.files:
        kw["qk_norm"] = bool(z["qk_norm"])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        got = att.scaled_dot_product_attention(*(torch.from_numpy(z[n]).cuda() for n in "qkv"), **kw)
    want = torch.from_numpy(z["out"])
    # `cross` was stored from TF32 matmuls: it only holds to the fused-kernel budget
    tol = 2e-3 if name == "cross" else FP32_REL
    np.testing.assert_allclose(got.cpu().numpy(), want.numpy(), atol=tol, rtol=tol)


# --------------------------------------------------------------------------
# the reference's kernel-test shapes, every operand combination
# --------------------------------------------------------------------------
CASES = ["dense", "bias", "causal", "mask", "cross", "bias_causal", "bias_mask", "full_bias_mask",
         "mask_b1st", "key_padding", "key_bias"]


@pytest.mark.parametrize("name", CASES)
def test_simt_fp32_parity(name):
    q, k, v, kw = _cases.kernel_case(name)
    got, ref = run_both(q, k, v, kw, torch.float32, "cuda-simt")
    check(got, ref, torch.float32)


@pytest.mark.parametrize("d", [32, 64, 128])
@pytest.mark.parametrize("name", ["dense", "bias_causal", "full_bias_mask", "key_padding", "key_bias", "cross"])
def test_fp32_3xtf32_parity(name, d):
    """fp32 operands at a size where the 3 x TF32 mma.sync kernels run forward and backward (grids of >= 96 CTAs of
    64 rows; lengths that do not fill the last tile): the fp32 budget of 1e-4 relative holds for out and all gradients."""
    shape = dict(b=4, h=6, s=344, t=200 if name == "cross" else 344, d=d)
    q, k, v, kw = _cases.kernel_case(name, **shape)
    got, ref = run_both(q, k, v, kw, torch.float32, "auto")
    check(got, ref, torch.float32)


@pytest.mark.parametrize("t", [100, 130, 200, 344, 520])
@pytest.mark.parametrize("name", ["dense", "bias_causal", "full_bias_mask", "key_padding"])
def test_fp32_small_forward_splits_keys_over_warp_groups(name, t):
    """Small fp32 problems: a CTA's groups of warps take the key tiles in turn and merge (m, l, out) at the end -- two,
    three and four groups (2, 3, 4+ key tiles; 100 keys is two tiles of which the second is partial), with causal rows
    whose later groups see no key at all, a random mask, key padding, and a row the mask empties."""
    _, att = _nb()
    s_len = t if name == "bias_causal" else 150
    q, k, v, kw = _cases.kernel_case(name, b=2, h=3, s=s_len, t=t, d=64)
    mask = kw.get("mask")
    if name == "full_bias_mask":
        mask = mask.clone()
        mask[0, 1, 7, :] = False           # one row with no kept key: NaN, as the reference's softmax gives
        kw = dict(kw, mask=mask)
    ref = O.reference_sdpa_torch(q, k, v, bias=kw.get("bias"), mask=kw.get("mask"), causal=kw.get("causal", False),
                                 acc_dtype=torch.float64)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out, lse = att.scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda(),
                                                    bias=None if kw.get("bias") is None else kw["bias"].cuda(),
                                                    mask=None if mask is None else mask.cuda(),
                                                    causal=kw.get("causal", False), return_lse=True)
    _device_ok()
    out = out.cpu().double()
    dead = torch.isnan(ref)
    assert torch.equal(torch.isnan(out), dead)
    assert float((out[~dead] - ref[~dead]).abs().max()) <= FP32_REL * float(ref[~dead].abs().max())


@pytest.mark.parametrize("d", [32, 64])
@pytest.mark.parametrize("s,t", [(100, 100), (150, 344), (344, 130), (520, 200), (256, 256)])
@pytest.mark.parametrize("name", ["dense", "bias_causal", "full_bias_mask", "key_padding"])
def test_fp32_small_backward_splits_tiles_over_groups_and_clusters(name, s, t, d):
    """Small fp32 problems, backward: the dq kernel's groups of warps take the key tiles in turn (two or three groups),
    the dk / dv kernel runs as clusters of two or four CTAs that take the query tiles in turn and sum their partial
    tiles over distributed shared memory -- with partial last tiles on both sides, causal key tiles that have fewer
    query tiles than the cluster has CTAs, a random mask, key padding and a bias gradient."""
    if name == "bias_causal":
        s = t
    q, k, v, kw = _cases.kernel_case(name, b=2, h=3, s=s, t=t, d=d)
    got, ref = run_both(q, k, v, kw, torch.float32, "auto")
    check(got, ref, torch.float32)


@pytest.mark.parametrize("shape", [dict(b=2, h=4, s=512, d=64), dict(b=1, h=2, s=2048, d=128), dict(b=2, h=4, s=344, d=32)])
def test_fp32_operand_split_keeps_the_fp32_budget_at_long_sequences(shape):
    """The 3 x TF32 kernels split every operand as hi = top 19 bits, lo = x - hi (the tensor core reads lo's TF32
    bits): out and all gradients against an fp64 restatement on the device, at lengths where thousands of products
    accumulate -- max error over max |reference| inside the fp32 budget of 1e-4 (measured: 2e-6 .. 3.5e-5)."""
    _, att = _nb()
    b, h, s, d = shape["b"], shape["h"], shape["s"], shape["d"]
    g = torch.Generator(device="cuda").manual_seed(11)
    q, k, v, dout = (torch.randn(b, h, s, d, device="cuda", generator=g) for _ in range(4))
    scale = d ** -0.5
    out, lse = att.sdpa_forward(q, k, v, None, None, scale=scale)
    dq, dk, dv = att.sdpa_backward(q, k, v, None, None, out, lse, dout, scale=scale)[:3]
    _device_ok()
    qd, kd, vd = (x.double().requires_grad_() for x in (q, k, v))
    ref = torch.softmax(qd @ kd.transpose(-1, -2) * scale, -1) @ vd
    ref.backward(dout.double())
    for name, a, r in (("out", out, ref.detach()), ("dq", dq, qd.grad), ("dk", dk, kd.grad), ("dv", dv, vd.grad)):
        err = float((a.double() - r).abs().max() / r.abs().max())
        assert err <= FP32_REL, (name, err)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", ["bias_mask", "causal", "key_padding"])
def test_simt_low_precision_parity(name, dtype):
    q, k, v, kw = _cases.kernel_case(name)
    got, ref = run_both(q, k, v, kw, dtype, "cuda-simt")
    check(got, ref, dtype)


def test_config1_fp32():
    q, k, v, kw = _cases.config1()
    got, ref = run_both(q, k, v, kw, torch.float32, "auto")
    check(got, ref, torch.float32)
    # masked keys get an exactly-zero bias gradient
    assert (got[4][1, :, :, -32:] == 0).all()


@pytest.mark.parametrize("shape", [dict(s=100, t=77, d=40, dv=24), dict(s=28, t=28, d=16), dict(s=1, t=300, d=96),
                                   dict(s=130, t=5, d=256, dv=8)])
def test_simt_ragged_shapes(shape):
    q, k, v, kw = _cases.kernel_case("full_bias_mask", **shape)
    got, ref = run_both(q, k, v, kw, torch.float32, "cuda-simt")
    check(got, ref, torch.float32)


def test_causal_cross_lengths_clamped():
    """causal with s > t and s < t: indices aligned at zero (reference _reference.py:166-170)."""
    for s, t in ((192, 64), (64, 192)):
        q, k, v, kw = _cases.kernel_case("causal", s=s, t=t)
        got, ref = run_both(q, k, v, kw, torch.float32, "cuda-simt")
        check(got, ref, torch.float32)


def test_leading_dims_and_broadcast_bias_grad():
    """(2, 3, h, s, d) batches; bias (h, s, t) shared over both: dbias is reduced over them."""
    _, att = _nb()
    rng = np.random.RandomState(0)
    mk = lambda *s: torch.from_numpy(rng.standard_normal(s).astype(np.float32))
    q, k, v, bias = mk(2, 3, 2, 20, 16), mk(2, 3, 2, 24, 16), mk(2, 3, 2, 24, 16), mk(2, 20, 24)
    dout = mk(2, 3, 2, 20, 16)
    ref = O.reference_grads_torch(q, k, v, dout, bias=bias, acc_dtype=torch.float64)
    leaves = [x.cuda().requires_grad_(True) for x in (q, k, v, bias)]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = att.scaled_dot_product_attention(*leaves[:3], bias=leaves[3])
    grads = torch.autograd.grad(out, leaves, grad_outputs=dout.cuda())
    check([out.detach(), *grads], list(ref), torch.float32)
    assert grads[3].shape == bias.shape


def test_fully_masked_row_is_nan():
    _, att = _nb()
    q = torch.ones(1, 1, 2, 16, device="cuda")
    kv = torch.ones(1, 1, 3, 16, device="cuda")
    mask = torch.tensor([[True, True, True], [False, False, False]], device="cuda")
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = att.scaled_dot_product_attention(q, kv, kv, mask=mask)
    assert torch.isfinite(out[0, 0, 0]).all() and torch.isnan(out[0, 0, 1]).all()


def test_empty_batch_and_empty_queries():
    _, att = _nb()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = att.scaled_dot_product_attention(torch.empty(0, 2, 8, 16, device="cuda"),
                                               torch.empty(0, 2, 8, 16, device="cuda"),
                                               torch.empty(0, 2, 8, 16, device="cuda"))
        assert out.shape == (0, 2, 8, 16)
        out = att.scaled_dot_product_attention(torch.empty(1, 2, 0, 16, device="cuda"),
                                               torch.randn(1, 2, 8, 16, device="cuda"),
                                               torch.randn(1, 2, 8, 16, device="cuda"))
        assert out.shape == (1, 2, 0, 16)


def test_bh_range_partition_matches_whole():
    """Two half-range calls on shared buffers equal one whole call (the multi-GPU slice)."""
    _, att = _nb()
    q, k, v, kw = _cases.kernel_case("bias_mask")
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    bias = kw["bias"].cuda().reshape(1, 2, 128, 128)
    mask = kw["mask"].cuda()
    from nitrix_b200 import _cabi
    whole, lse = att.sdpa_forward(q, k, v, bias, mask, scale=0.125, kernel=_cabi.KERNEL_SIMT)
    out = torch.zeros_like(whole)
    lse2 = torch.zeros_like(lse)
    att.sdpa_forward(q, k, v, bias, mask, scale=0.125, kernel=_cabi.KERNEL_SIMT, bh_range=(0, 3), out=out, lse=lse2)
    att.sdpa_forward(q, k, v, bias, mask, scale=0.125, kernel=_cabi.KERNEL_SIMT, bh_range=(3, 4), out=out, lse=lse2)
    assert torch.equal(out, whole) and torch.equal(lse, lse2)


def test_lse_is_base2_logsumexp():
    _, att = _nb()
    q, k, v, kw = _cases.kernel_case("bias")
    _, lse_ref = O.reference_sdpa_numpy(q.numpy(), k.numpy(), v.numpy(), bias=kw["bias"].numpy(), return_lse=True)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        _, lse = att.scaled_dot_product_attention(q.cuda(), k.cuda(), v.cuda(), bias=kw["bias"].cuda(), return_lse=True)
    np.testing.assert_allclose(lse.cpu().numpy(), lse_ref, atol=1e-4, rtol=1e-5)


def test_backward_workspace_is_far_below_score_matrix():
    """Gross-memory contract (reference tests/test_nn_attention_kernel.py:197-252): scratch << B*H*S*T*4."""
    import ctypes as C
    from nitrix_b200 import _cabi
    _, att = _nb()
    B, H, S, D = 2, 4, 1024, 64
    q = torch.empty(B, H, S, D, device="cuda", dtype=torch.bfloat16)
    p = _cabi.new_params()
    att._fill_common(p, q, q, q, q, q, None, None, 0.125, False, _cabi.KERNEL_AUTO, None)
    p.dout = p.dq = p.dk = p.dv = q.data_ptr()
    for name in ("dout_stride", "dq_stride", "dk_stride", "dv_stride"):
        getattr(p, name)[:] = list(q.stride())
    need = C.c_size_t(0)
    assert _cabi.lib().nb200_sdpa_workspace_bytes(C.byref(p), _cabi.PASS_BWD, C.byref(need)) == 0
    assert need.value < B * H * S * S * 4 // 8


# --------------------------------------------------------------------------
# tensor-core (TMA + tcgen05) family: bf16 / fp16, D in {64, 128}
# --------------------------------------------------------------------------
def _device_ok():
    from nitrix_b200 import _cabi
    torch.cuda.synchronize()
    rc = _cabi.lib().nb200_device_status(torch.cuda.current_device())
    assert rc == 0, _cabi.last_error()


def _assert_plans_tc(q, k, v, kw, dtype, which=0, want_dbias=False):
    from nitrix_b200 import _cabi
    _, att = _nb()
    b, h, s, d = q.shape
    t = k.shape[2]
    lead = (b,)
    bias = kw.get("bias")
    mask = kw.get("mask")
    b4 = None if bias is None else att._to_own_extent(bias.to(dtype).cuda(), lead, h, s, t)
    m4 = None if mask is None else att._to_own_extent(mask.cuda(), lead, h, s, t)
    chosen = att.planned_kernel(q.to(dtype).cuda(), k.to(dtype).cuda(), v.to(dtype).cuda(), b4, m4,
                                causal=kw.get("causal", False), which=which, want_dbias=want_dbias)
    assert chosen == _cabi.KERNEL_TCGEN05


TC_CASES = ["dense", "bias", "causal", "mask", "cross", "bias_causal", "full_bias_mask", "mask_b1st",
            "key_padding", "key_bias"]


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("name", TC_CASES)
def test_tc_parity(name, dtype, d):
    q, k, v, kw = _cases.kernel_case(name, s=256, t=512 if name == "cross" else 384 if "bias" in name else 256, d=d)
    if "causal" in name:
        q, k, v, kw = _cases.kernel_case(name, s=384, t=384, d=d)
    _assert_plans_tc(q, k, v, kw, dtype)
    # the gradient of a bias shared over the batch (or over the queries) is summed in fp32 by the tensor-core
    # backward as well; with and without dbias the backward stays on tensor cores
    bias = kw.get("bias")
    shared_bias = bias is not None and bias.numel() < q.shape[0] * q.shape[1] * q.shape[2] * k.shape[2]
    for want_dbias in ([True, False] if shared_bias else [True]):
        _assert_plans_tc(q, k, v, kw, dtype, which=1, want_dbias=want_dbias and bias is not None)
        got, ref = run_both(q, k, v, kw, dtype, "cuda-sm100", want_dbias=want_dbias)
        _device_ok()
        check(got, ref, dtype)


RAGGED = [dict(s=200, t=200), dict(s=136, t=328), dict(s=392, t=72), dict(s=8, t=8), dict(s=256, t=200)]


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("shape", RAGGED)
@pytest.mark.parametrize("name", ["dense", "bias_causal", "full_bias_mask", "key_padding", "key_bias", "causal"])
def test_tc_ragged_lengths(name, shape, d):
    """Lengths that do not fill whole 128-row tiles (multiples of 8) stay on the tensor-core kernels: rows past the
    end are zero-filled by TMA, keys past T are masked, nothing is stored past S."""
    q, k, v, kw = _cases.kernel_case(name, d=d, **shape)
    dtype = torch.bfloat16
    _assert_plans_tc(q, k, v, kw, dtype)
    want_dbias = kw.get("bias") is not None   # shared biases included: their gradient is summed on tensor cores too
    _assert_plans_tc(q, k, v, kw, dtype, which=1, want_dbias=want_dbias)
    got, ref = run_both(q, k, v, kw, dtype, "cuda-sm100", want_dbias=want_dbias)
    _device_ok()
    check(got, ref, dtype)


def test_tc_ragged_fp16():
    q, k, v, kw = _cases.kernel_case("bias_mask", s=264, t=136, d=64)
    _assert_plans_tc(q, k, v, kw, torch.float16)
    got, ref = run_both(q, k, v, kw, torch.float16, "cuda-sm100", want_dbias=False)
    _device_ok()
    check(got, ref, torch.float16)


# the token counts the reference's documents name as what its callers have (6^3 patches + CLS = 217, 28, ViT's 197,
# 111, 344): none but the last is a multiple of 8, and all must stay on the tensor-core kernels -- bias and dbias rows
# of such lengths go through padded copies, lse / delta through padded rows
ODD = [dict(s=217, t=217), dict(s=28, t=28), dict(s=197, t=197), dict(s=111, t=344), dict(s=344, t=111), dict(s=1, t=77),
       dict(s=130, t=5)]


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("shape", ODD)
@pytest.mark.parametrize("name", ["dense", "bias", "bias_causal", "full_bias_mask", "key_padding", "key_bias", "mask_b1st"])
def test_tc_any_lengths(name, shape, d):
    q, k, v, kw = _cases.kernel_case(name, d=d, **shape)
    dtype = torch.bfloat16
    want_dbias = kw.get("bias") is not None
    _assert_plans_tc(q, k, v, kw, dtype)
    _assert_plans_tc(q, k, v, kw, dtype, which=1, want_dbias=want_dbias)
    got, ref = run_both(q, k, v, kw, dtype, "cuda-sm100", want_dbias=want_dbias)
    _device_ok()
    check(got, ref, dtype)


def test_tc_bias_with_strided_keys_and_odd_row_stride():
    """A bias whose key axis is not contiguous (a transposed view) and one whose rows are an odd number of elements
    apart: both reach the kernels through the padded copy instead of falling off the tensor-core path."""
    from nitrix_b200 import _cabi
    _, att = _nb()
    q, k, v, _ = _cases.kernel_case("dense", s=256, t=256, d=64)
    base = _cases._randn((2, 2, 256, 256), 3).to(torch.bfloat16)
    dt = torch.bfloat16
    qd, kd, vd = (x.to(dt).cuda() for x in (q, k, v))
    wide = torch.zeros(2, 2, 256, 261, dtype=dt)
    wide[..., :256] = base
    for bias_cpu, bias_gpu in ((base.transpose(-1, -2), base.cuda().transpose(-1, -2)), (base, wide.cuda()[..., :256])):
        assert att.planned_kernel(qd, kd, vd, bias_gpu, None, scale=0.125) == _cabi.KERNEL_TCGEN05
        ref = O.reference_sdpa_torch(qd.cpu().float(), kd.cpu().float(), vd.cpu().float(), bias=bias_cpu.float())
        got = att.scaled_dot_product_attention(qd, kd, vd, bias=bias_gpu, backend="cuda-sm100")
        _device_ok()
        assert abserr(got, ref) < LOWP_ABS


def test_tc_backward_full_bias_causal_dbias_zero_past_diagonal():
    """Per-batch bias + causal: dbias comes from the tensor-core backward and is exactly zero above the diagonal."""
    q, k, v, kw = _cases.kernel_case("full_bias", s=256, t=256, d=64)
    kw["causal"] = True
    _assert_plans_tc(q, k, v, kw, torch.bfloat16, which=1, want_dbias=True)
    got, ref = run_both(q, k, v, kw, torch.bfloat16, "cuda-sm100")
    _device_ok()
    check(got, ref, torch.bfloat16)
    upper = torch.triu(torch.ones(256, 256, dtype=torch.bool), diagonal=1)
    assert (got[4].cpu()[..., upper] == 0).all()


@pytest.mark.parametrize("d", [64, 128])
def test_tc_many_tiles_full_bias_mask(d):
    """Long enough (8 key tiles, 64 CTAs) for the rings to wrap many times with both query tiles active."""
    q, k, v, kw = _cases.kernel_case("full_bias_mask", b=2, h=4, s=1024, t=1024, d=d)
    _assert_plans_tc(q, k, v, kw, torch.bfloat16, which=1, want_dbias=True)
    got, ref = run_both(q, k, v, kw, torch.bfloat16, "cuda-sm100")
    _device_ok()
    check(got, ref, torch.bfloat16)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_tc_fully_masked_rows_are_nan_and_the_rest_matches(d, dtype):
    """Rows whose mask drops every key come out NaN (0 * inf, as the reference's softmax gives) on the tensor-core
    kernels too; every masked key contributes exactly zero (also where 2^x is computed on the FMA pipe, which clamps
    its argument instead of seeing -inf), and widely spread logits (bias of +-60) stay inside the budget."""
    _, att = _nb()
    g = torch.Generator().manual_seed(11)
    b, h, s, t = 1, 2, 256, 384
    q = torch.randn(b, h, s, d, generator=g)
    k = torch.randn(b, h, t, d, generator=g)
    v = torch.randn(b, h, t, d, generator=g)
    bias = (torch.randn(b, h, s, t, generator=g) * 20).clamp(-60, 60)
    mask = torch.rand(b, 1, s, t, generator=g) >= 0.3
    dead = torch.tensor([0, 5, 127, 128, 255])
    mask[:, :, dead, :] = False
    mask[:, :, 7, :] = False
    mask[:, :, 7, 300] = True            # a row with one kept key, in the last key tile
    kw = dict(bias=bias, mask=mask)
    _assert_plans_tc(q, k, v, kw, dtype)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = att.scaled_dot_product_attention(q.to(dtype).cuda(), k.to(dtype).cuda(), v.to(dtype).cuda(),
                                               bias=bias.to(dtype).cuda(), mask=mask.cuda())
    _device_ok()
    out = out.float().cpu()
    assert torch.isnan(out[:, :, dead]).all()
    live = torch.ones(s, dtype=torch.bool)
    live[dead] = False
    assert torch.isfinite(out[:, :, live]).all()
    ref = O.reference_sdpa_torch(q.to(dtype).float(), k.to(dtype).float(), v.to(dtype).float(),
                                 bias=bias.to(dtype).float(), mask=mask)
    assert relerr(out[:, :, live], ref[:, :, live]) <= (2e-2 if dtype == torch.bfloat16 else 4e-3)
    # the row with a single kept key is that key's value row
    assert abserr(out[:, :, 7], v.to(dtype).float()[:, :, 300]) <= 1e-6


def test_tc_single_tile_and_odd_tile_count():
    for s, t in ((128, 128), (384, 128), (128, 640)):
        q, k, v, kw = _cases.kernel_case("bias_mask", s=s, t=t, d=64, b=1, h=3)
        _assert_plans_tc(q, k, v, kw, torch.bfloat16)
        _assert_plans_tc(q, k, v, kw, torch.bfloat16, which=1)
        got, ref = run_both(q, k, v, kw, torch.bfloat16, "cuda-sm100", want_dbias=False)
        _device_ok()
        check(got, ref, torch.bfloat16)


def test_tc_matches_simt_on_same_inputs():
    """The two kernel families agree with each other far inside the low-precision budget."""
    _, att = _nb()
    q, k, v, kw = _cases.kernel_case("bias_causal", s=512, t=512, d=128)
    args = [x.to(torch.bfloat16).cuda() for x in (q, k, v)]
    bias = kw["bias"].to(torch.bfloat16).cuda()
    a = att.scaled_dot_product_attention(*args, bias=bias, causal=True, backend="cuda-sm100")
    b = att.scaled_dot_product_attention(*args, bias=bias, causal=True, backend="cuda-simt")
    _device_ok()
    assert abserr(a, b) < 2e-2  # one bf16 ulp at |x| < 4


def test_tc_noncontiguous_heads_layout():
    """q/k/v stored (B, S, H, D) and viewed as (B, H, S, D): strides go straight into the TMA maps."""
    _, att = _nb()
    g = torch.Generator().manual_seed(0)
    B, H, S, D = 2, 3, 256, 64
    qkv = [torch.randn(B, S, H, D, generator=g).to(torch.bfloat16) for _ in range(3)]
    views_cpu = [x.permute(0, 2, 1, 3) for x in qkv]
    ref = O.reference_sdpa_torch(*[x.float() for x in views_cpu], causal=True)
    views = [x.cuda().permute(0, 2, 1, 3) for x in qkv]
    got = att.scaled_dot_product_attention(*views, causal=True, backend="cuda-sm100")
    _device_ok()
    assert abserr(got, ref) < LOWP_ABS


# --------------------------------------------------------------------------
# corners of the tensor-core family
# --------------------------------------------------------------------------
def test_tc_reference_broadcast_bias_gradient_case():
    """The reference's own gradient test (tests/test_nn_attention_kernel.py:120-140): a learned bias (h, s, t) shared
    over the batch, gradient of bias' shape -- here in bf16 on the tensor-core backward, s = t = 256."""
    q, k, v, kw = _cases.kernel_case("bias", s=256, t=256, d=64)
    _assert_plans_tc(q, k, v, kw, torch.bfloat16, which=1, want_dbias=True)
    got, ref = run_both(q, k, v, kw, torch.bfloat16, "cuda-sm100", want_dbias=True)
    _device_ok()
    check(got, ref, torch.bfloat16)
    assert got[4].shape == kw["bias"].shape


@pytest.mark.parametrize("d", [64, 128])
def test_tc_bias_shared_over_heads_and_batch_gradient(d):
    """bias (1, 1, s, t): the fp32 accumulator is shared by every (batch, head) pair."""
    q, k, v, kw = _cases.kernel_case("dense", b=2, h=3, s=256, t=384, d=d)
    kw["bias"] = _cases._randn((1, 1, 256, 384), 3)
    kw["causal"] = True
    _assert_plans_tc(q, k, v, kw, torch.bfloat16, which=1, want_dbias=True)
    got, ref = run_both(q, k, v, kw, torch.bfloat16, "cuda-sm100", want_dbias=True)
    _device_ok()
    check(got, ref, torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [64, 128])
def test_tc_per_key_bias_gradient(dtype, d):
    """bias (1, h, 1, t) with a gradient: each key's ds is summed over queries and batch by the key-major kernel."""
    q, k, v, kw = _cases.kernel_case("key_bias", b=2, h=2, s=384, t=256, d=d)
    _assert_plans_tc(q, k, v, kw, dtype, which=1, want_dbias=True)
    got, ref = run_both(q, k, v, kw, dtype, "cuda-sm100", want_dbias=True)
    _device_ok()
    check(got, ref, dtype)


def test_tc_expanded_kv_and_expanded_cotangent():
    """k / v expanded over the batch and over the heads (stride 0), and a cotangent that arrives as an expanded
    view (loss = out.mean(0)): the tensor-core kernels address q, k, v, dout by absolute (batch, head), so the
    host layer materialises such views; results must match the oracle on the materialised operands."""
    _, att = _nb()
    g = torch.Generator().manual_seed(0)
    B, H, S, T, D = 3, 4, 256, 256, 64
    dt = torch.bfloat16
    q = torch.randn(B, H, S, D, generator=g).to(dt)
    k1 = torch.randn(1, H, T, D, generator=g).to(dt)      # shared by the batch
    v1 = torch.randn(1, 1, T, D, generator=g).to(dt)      # shared by batch and heads (multi-query style)
    k_cpu, v_cpu = k1.expand(B, H, T, D), v1.expand(B, H, T, D)
    dout = torch.ones(1, H, S, D).to(dt).expand(B, H, S, D) / B     # cotangent of out.mean(0).sum()
    ref = O.reference_grads_torch(q, k_cpu.contiguous(), v_cpu.contiguous(), dout.contiguous())
    qg = q.cuda().requires_grad_(True)
    kg = k1.cuda().requires_grad_(True)
    vg = v1.cuda().requires_grad_(True)
    out = att.scaled_dot_product_attention(qg, kg.expand(B, H, T, D), vg.expand(B, H, T, D), backend="cuda-sm100")
    loss = out.float().mean(0).sum()
    dq, dk, dv = torch.autograd.grad(loss, [qg, kg, vg])
    _device_ok()
    assert abserr(out, ref[0]) < LOWP_ABS
    assert abserr(dq, ref[1]) < LOWP_ABS * max(1.0, float(ref[1].abs().max()))
    # gradients of the expanded operands are the sums over the expanded axes
    rk = ref[2].float().sum(0, keepdim=True)
    rv = ref[3].float().sum((0, 1), keepdim=True)
    assert abserr(dk.float(), rk) < LOWP_ABS * max(1.0, float(rk.abs().max()))
    assert abserr(dv.float(), rv) < LOWP_ABS * max(1.0, float(rv.abs().max()))


def test_tc_plan_declines_stride0_qkv_through_the_c_abi():
    """Called with a stride-0 head axis on k, the library itself declines the tensor-core family (the CUDA-core
    family indexes by stride and takes it)."""
    from nitrix_b200 import _cabi
    _, att = _nb()
    q = torch.randn(2, 4, 128, 64, device="cuda").bfloat16()
    k = torch.randn(2, 1, 128, 64, device="cuda").bfloat16().expand(2, 4, 128, 64)
    assert att.planned_kernel(q, k, q, None, None, causal=False) == _cabi.KERNEL_SIMT
    assert att.planned_kernel(q, q, q, None, None, causal=False) == _cabi.KERNEL_TCGEN05


@pytest.mark.parametrize("dtype,backend", [(torch.float32, "auto"), (torch.bfloat16, "cuda-sm100")])
def test_qk_norm_gradients(dtype, backend):
    """qk_norm = True through the CUDA path, forward and gradients (reference tests/test_nn_attention_kernel.py:146-191)."""
    _, att = _nb()
    q, k, v, kw = _cases.kernel_case("bias_causal", s=256, t=256, d=64)
    qd, kd, vd, bd = (x.to(dtype) for x in (q, k, v, kw["bias"]))
    dout = torch.from_numpy(np.random.RandomState(5).standard_normal(q.shape).astype(np.float32)).to(dtype)
    acc = torch.float64 if dtype == torch.float32 else torch.float32
    ref = O.reference_grads_torch(qd, kd, vd, dout, bias=bd, causal=True, qk_norm=True, acc_dtype=acc)
    leaves = [x.cuda().requires_grad_(True) for x in (qd, kd, vd, bd)]
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        out = att.scaled_dot_product_attention(*leaves[:3], bias=leaves[3], causal=True, qk_norm=True, backend=backend)
    grads = torch.autograd.grad(out, leaves, grad_outputs=dout.cuda())
    _device_ok()
    check([out.detach(), *grads], list(ref), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [32, 64, 128, 256])
def test_fused_qk_norm_pre_op_matches_the_reference_op(dtype, d):
    """The one-launch pre-op (nb200_qk_rms_norm / _grad) against the reference's formula in fp64 (reference
    nn/attention/_reference.py:52-77), forward and gradient, on a dense layout, a (batch, seq, head) memory order and a
    3-D input; the launch counter shows that the fused kernels ran (one launch each way for q and k together)."""
    from nitrix_b200 import _cabi
    _, att = _nb()
    g = torch.Generator().manual_seed(3)
    b, h, s, t = 2, 3, 37, 21
    q = (torch.randn(b, h, s, d, generator=g) * 3).to(dtype).cuda()
    k = (torch.randn(b, t, h, d, generator=g) * 0.01).to(dtype).cuda().permute(0, 2, 1, 3)   # heads strided
    gq = torch.randn(b, h, s, d, generator=g).to(dtype).cuda()
    gk = torch.randn(b, h, t, d, generator=g).to(dtype).cuda()

    def ref(x, gx):
        x64 = x.double().requires_grad_(True)
        y = x64 * torch.rsqrt(x64.square().mean(-1, keepdim=True) + 1e-6)
        (dx,) = torch.autograd.grad(y, x64, grad_outputs=gx.double())
        return y.detach(), dx

    assert att._qk_norm_fusable(q, k)
    ql, kl = q.clone().requires_grad_(True), k.clone().requires_grad_(True)
    before = _cabi.lib().nb200_launch_count()
    qn, kn = att.qk_rms_norm_pair(ql, kl)
    dq, dk = torch.autograd.grad([qn, kn], [ql, kl], grad_outputs=[gq, gk])
    torch.cuda.synchronize()
    assert _cabi.lib().nb200_launch_count() - before == 2
    tol = 2e-6 if dtype == torch.float32 else (1e-2 if dtype == torch.bfloat16 else 1.5e-3)
    for got, (want_y, want_dx), gy in ((qn, ref(q, gq), dq), (kn, ref(k, gk), dk)):
        assert relerr(got.detach(), want_y) <= tol
        assert relerr(gy, want_dx) <= tol
    # a 3-D (h, s, d) operand pair
    q3, k3 = q[0].contiguous(), k[0].contiguous()
    a3, b3 = att.qk_rms_norm_pair(q3, k3)
    assert relerr(a3, ref(q3, gq[0])[0]) <= tol and relerr(b3, ref(k3, gk[0])[0]) <= tol
    # layouts the kernel cannot read with 16-byte loads fall back to the element-wise form
    odd = q[..., : d - 1]
    assert not att._qk_norm_fusable(odd, odd)
    assert relerr(att.qk_rms_norm_pair(odd, odd)[0], ref(odd, gq[..., : d - 1])[0]) <= tol


def _small_fp32_backward(att):
    g = torch.Generator().manual_seed(21)
    b, h, s, t, d = 2, 2, 96, 80, 32
    q, k, v, dout = (torch.randn(b, h, n, d, generator=g).cuda() for n in (s, t, t, s))
    bias = torch.randn(b, h, s, t, generator=g).cuda()
    out, lse = att.sdpa_forward(q, k, v, bias, None, scale=d ** -0.5)
    return (q, k, v, bias, None, out, lse, dout), dict(scale=d ** -0.5, want_dbias=True)


def test_small_backward_side_stream_equals_one_stream():
    """A small problem's dq and dk / dv kernels run side by side on a second stream (fork / join events).  With
    per-kernel timing on the library keeps to one stream: both ways must give the same bits."""
    from nitrix_b200 import _cabi
    _, att = _nb()
    args, kw = _small_fp32_backward(att)
    forked = att.sdpa_backward(*args, **kw)
    torch.cuda.synchronize()
    _cabi.lib().nb200_profile(1)
    try:
        serial = att.sdpa_backward(*args, **kw)
        torch.cuda.synchronize()
    finally:
        _cabi.lib().nb200_profile(0)
    _device_ok()
    for a, b in zip(forked, serial):
        assert torch.equal(a, b)


def test_small_backward_first_called_inside_a_graph_capture():
    """A host thread whose first backward call happens while its stream is being captured: the library must not
    create its side stream then (nothing is created during a capture); the captured graph replays correctly."""
    import threading
    _, att = _nb()
    args, kw = _small_fp32_backward(att)
    want = att.sdpa_backward(*args, **kw)
    torch.cuda.synchronize()
    box = {}

    def work():
        try:
            torch.cuda.set_device(0)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    got = att.sdpa_backward(*args, **kw)
            graph.replay()
            torch.cuda.synchronize()
            box["got"] = [x.clone() for x in got]
        except Exception as e:   # surfaced in the main thread below
            box["err"] = e

    th = threading.Thread(target=work)
    th.start()
    th.join()
    assert "err" not in box, box.get("err")
    _device_ok()
    for a, b in zip(box["got"], want):
        assert torch.equal(a, b)


def test_fp32_on_the_fused_tf32_path_does_not_warn_or_raise(monkeypatch):
    """fp32 is what the reference's fused path accepts silently (attention.py:736-744): with backend='auto' an fp32
    call that lands on the 3 x TF32 tensor kernels must neither warn nor, under NITRIX_STRICT_BACKEND=1, raise."""
    nb, att = _nb()
    from nitrix_b200 import _cabi
    q, k, v, _ = _cases.kernel_case("dense", s=344, t=344, d=64)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    assert att.planned_kernel(q, k, v, None, None, causal=False) == _cabi.KERNEL_MMA_TF32X3
    monkeypatch.setenv("NITRIX_STRICT_BACKEND", "1")
    nb.reset_fallback_state()
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        att.scaled_dot_product_attention(q, k, v)
    # a head dim the tensor paths do not take still raises under strict mode
    q2 = torch.randn(1, 2, 64, 40, device="cuda")
    with pytest.raises(nb.NitrixBackendError):
        att.scaled_dot_product_attention(q2, q2, q2)


def test_packed_mask_is_packed_once_and_reused():
    """nb200_mask_pack + mask_is_bitpacked: forward and backward on the packed bits equal the byte-mask calls."""
    from nitrix_b200 import _cabi
    _, att = _nb()
    for name, shape in (("full_bias_mask", dict(s=256, t=384, d=128)), ("key_padding", dict(s=256, t=256, d=64)),
                        ("mask_b1st", dict(s=384, t=256, d=64))):
        q, k, v, kw = _cases.kernel_case(name, **shape)
        b, h, s, d = q.shape
        t = k.shape[2]
        dt = torch.bfloat16
        q, k, v = (x.to(dt).cuda() for x in (q, k, v))
        bias = kw.get("bias")
        bias4 = None if bias is None else att._to_own_extent(bias.to(dt).cuda(), (b,), h, s, t)
        mask4 = att._to_own_extent(kw["mask"].cuda(), (b,), h, s, t)
        scale = d ** -0.5
        out, lse = att.sdpa_forward(q, k, v, bias4, mask4, scale=scale)
        dout = torch.randn(out.shape, generator=torch.Generator().manual_seed(5)).to(dt).cuda()
        want = att.sdpa_backward(q, k, v, bias4, mask4, out, lse, dout, scale=scale, want_dbias=bias4 is not None)
        packed = att.pack_mask(q, k, v, mask4, with_transpose=True)
        launches = _cabi.lib().nb200_launch_count()
        out2, lse2 = att.sdpa_forward(q, k, v, bias4, packed, scale=scale)
        got = att.sdpa_backward(q, k, v, bias4, packed, out2, lse2, dout, scale=scale, want_dbias=bias4 is not None)
        _device_ok()
        assert torch.equal(out, out2) and torch.equal(lse, lse2), name
        for a, b_ in zip(got, want):
            if b_ is None:
                assert a is None
            elif a is got[0]:
                assert abserr(a, b_) <= LOWP_ABS        # dq of the one-kernel backwards: fp32 reduction order
            else:
                assert torch.equal(a, b_), name
        # no packing kernel ran in the packed calls: forward 1 launch; backward delta + kernels only
        names_after = _cabi.lib().nb200_launch_count() - launches
        assert names_after <= 5, names_after


def test_bounded_wait_times_out_and_reports():
    """The give-up branch of the kernels' mbarrier wait: a wait nothing completes expires within milliseconds, the
    kernel returns, the status word reports a time-out once and the library keeps working."""
    import ctypes as C
    from nitrix_b200 import _cabi
    _, att = _nb()
    lib = _cabi.lib()
    dev = torch.cuda.current_device()
    torch.cuda.synchronize()
    assert lib.nb200_device_status(dev) == _cabi.OK
    result = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    rc = lib.nb200_selftest_bounded_wait(C.c_void_p(result.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == _cabi.OK, _cabi.last_error()
    torch.cuda.synchronize()                      # returns: the wait was bounded
    assert result.tolist() == [0, 1]              # reported "not completed" and raised the CTA abort flag
    assert lib.nb200_device_status(dev) == _cabi.ERR_TIMEOUT
    assert "901" in _cabi.last_error()
    assert lib.nb200_device_status(dev) == _cabi.OK      # read-and-clear
    # and the next real call is healthy
    q, k, v, kw = _cases.kernel_case("causal", s=256, t=256, d=64)
    got, ref = run_both(q, k, v, kw, torch.bfloat16, "cuda-sm100")
    _device_ok()
    check(got, ref, torch.bfloat16)
