"""The selective-scan oracle against the reference's stored vector and its own invariants (CPU only).

Mirrors the reference's ``tests/test_nn_ssm.py``: the golden case (:69-83), the cumulative-sum limit A -> 0 named in
the reference's notes, agreement of the numpy and torch statements, and the shape errors of the public function
(:290-296).
"""
import pathlib

import numpy as np
import pytest
import torch

from oracle import scan_oracle as S

GOLD = pathlib.Path(__file__).resolve().parent / "golden"


def test_oracle_reproduces_the_reference_golden():
    z = np.load(GOLD / "selective_scan_float32.npz")
    got = S.selective_scan(z["x"], z["delta"], z["A"], z["B"], z["C"], z["D"])
    assert got.dtype == np.float32 and got.shape == z["out"].shape
    np.testing.assert_allclose(got, z["out"], atol=2e-6, rtol=2e-6)


def test_zero_state_matrix_is_a_cumulative_sum():
    rng = np.random.RandomState(0)
    x, delta = rng.standard_normal((2, 9, 4)), rng.uniform(0.1, 1.0, (2, 9, 4))
    B, C = rng.standard_normal((2, 9, 3)), rng.standard_normal((2, 9, 3))
    got = S.selective_scan(x, delta, np.zeros((4, 3)), B, C)
    h = np.cumsum(delta[..., None] * B[..., None, :] * x[..., None], axis=-3)
    np.testing.assert_allclose(got, (h * C[..., None, :]).sum(-1), atol=1e-12)


def test_numpy_and_torch_statements_agree():
    rng = np.random.RandomState(1)
    x, delta = rng.standard_normal((3, 12, 5)), rng.uniform(0.05, 0.5, (3, 12, 5))
    A, D = -rng.uniform(0.5, 2.0, (5, 4)), rng.standard_normal(5)
    B, C = rng.standard_normal((3, 12, 4)), rng.standard_normal((3, 12, 4))
    want = S.selective_scan(x, delta, A, B, C, D)
    got = S.selective_scan_torch(*(torch.from_numpy(a) for a in (x, delta, A, B, C, D))).numpy()
    np.testing.assert_allclose(got, want, atol=1e-12)


def test_public_function_rejects_misshaped_operands():
    from nitrix_b200.nn import ssm

    x, delta, A = torch.zeros(2, 6, 4), torch.zeros(2, 6, 4), torch.zeros(4, 3)
    B, C, D = torch.zeros(2, 6, 3), torch.zeros(2, 6, 3), torch.zeros(4)
    with pytest.raises(ValueError, match="B/C last dim must be n=3"):
        ssm.selective_scan(x, delta, A, B[..., :-1], C, D)
    with pytest.raises(ValueError, match=r"D must be \(d,\) with d=4"):
        ssm.selective_scan(x, delta, A, B, C, D[:-1])
    with pytest.raises(ValueError, match="x and delta must match"):
        ssm.selective_scan(x, delta[:, :-1], A, B, C, D)
