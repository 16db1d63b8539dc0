"""The LayerNorm oracle against the reference's stored vector and against its own invariants (CPU only).

Mirrors the reference's ``tests/test_nn_norm.py``: the golden case (:51-62), agreement with a plain numpy statement
(:128-136), linearity in ``out_scale`` (:151-158), normalised statistics (:169-178), gradients against finite
differences (:183-210) and the affine-shape error of the public function (:257-260).
"""
import pathlib

import numpy as np
import pytest

from oracle import norm_oracle as N

GOLD = pathlib.Path(__file__).resolve().parent / "golden"


def test_oracle_reproduces_the_reference_golden():
    z = np.load(GOLD / "layer_norm_float32.npz")
    got = N.layer_norm(z["x"], z["weight"], z["bias"], out_scale=0.5)
    assert got.dtype == np.float32 and got.shape == z["out"].shape
    np.testing.assert_allclose(got, z["out"], atol=1e-6, rtol=1e-6)


def test_out_scale_is_linear_and_statistics_are_normalised():
    rng = np.random.RandomState(2)
    x, w, b = rng.standard_normal((2, 3, 16)), rng.standard_normal(16), rng.standard_normal(16)
    base = N.layer_norm(x, w, b, out_scale=1.0)
    np.testing.assert_allclose(N.layer_norm(x, w, b, out_scale=2.5), 2.5 * base, atol=1e-12)
    xh = N.layer_norm(x, eps=1e-6)
    np.testing.assert_allclose(xh.mean(-1), 0.0, atol=1e-6)
    np.testing.assert_allclose(xh.var(-1), 1.0, atol=1e-4)


def test_sixteen_bit_input_is_reduced_in_fp32_and_cast_back():
    import torch

    rng = np.random.RandomState(3)
    x = torch.from_numpy(rng.standard_normal((4, 64)).astype(np.float32)).to(torch.bfloat16)
    got = N.layer_norm(x.float().numpy(), out_scale=0.7)          # the fp32 recipe on the quantised values
    want = torch.nn.functional.layer_norm(x.float(), (64,)) * 0.7
    np.testing.assert_allclose(got, want.numpy(), atol=2e-6)


def test_closed_form_gradients_match_finite_differences():
    rng = np.random.RandomState(5)
    x, w, b = rng.standard_normal((2, 8)), rng.standard_normal(8), rng.standard_normal(8)
    dy = rng.standard_normal((2, 8))

    def loss(x_, w_, b_):
        return float((N.layer_norm(x_, w_, b_, out_scale=0.5) * dy).sum())

    dx, dw, db = N.layer_norm_grads(x, w, dy, out_scale=0.5)
    h = 1e-6
    for arr, grad in ((x, dx), (w, dw), (b, db)):
        for idx in np.ndindex(arr.shape):
            keep = arr[idx]
            arr[idx] = keep + h
            up = loss(x, w, b)
            arr[idx] = keep - h
            dn = loss(x, w, b)
            arr[idx] = keep
            assert abs((up - dn) / (2 * h) - grad[idx]) < 1e-6, (idx, grad[idx])


def test_public_function_rejects_a_misshaped_affine_parameter():
    import torch

    from nitrix_b200.nn import norm

    with pytest.raises(ValueError, match=r"layer_norm: weight must have shape \(8,\)"):
        norm.layer_norm(torch.zeros(2, 8), torch.zeros(4))
    with pytest.raises(ValueError, match=r"layer_norm: bias must have shape \(8,\)"):
        norm.layer_norm(torch.zeros(2, 8), None, torch.zeros(8, 1))
