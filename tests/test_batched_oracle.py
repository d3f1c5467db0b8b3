"""Pins the batched-product oracle against the definitions the reference's own tests use
(test/batchedmul.jl:6-28: slice-by-slice products with optional permutedims) and re-states its cases."""
import numpy as np
import pytest

from oracle import batched_oracle as BO


def bmm_test(a, b, transA=False, transB=False):
    # test/batchedmul.jl:6-16
    if transA:
        a = np.transpose(a, (1, 0, 2))
    if transB:
        b = np.transpose(b, (1, 0, 2))
    return np.stack([a[:, :, i] @ b[:, :, i] for i in range(a.shape[2])], axis=2)


@pytest.mark.parametrize("TB", [np.float64, np.float32])
def test_batched_mul_like_the_reference(TB):
    # test/batchedmul.jl:40-49
    rng = np.random.default_rng(0)
    A = rng.standard_normal((7, 5, 3))
    B = rng.standard_normal((5, 7, 3)).astype(TB)
    C = rng.standard_normal((7, 6, 3))
    bt = BO.batched_transpose
    np.testing.assert_allclose(BO.batched_mul(A, B), bmm_test(A, B), rtol=1e-6)
    np.testing.assert_allclose(BO.batched_mul(bt(A), bt(B)), bmm_test(A, B, transA=True, transB=True), rtol=1e-6)
    np.testing.assert_allclose(BO.batched_mul(bt(A), C), bmm_test(A, C, transA=True), rtol=1e-6)
    np.testing.assert_allclose(BO.batched_mul(A, bt(A)), bmm_test(A, A, transB=True), rtol=1e-6)
    assert bt(bt(A)) is not None and np.shares_memory(bt(bt(A)), A)
    # errors, test/batchedmul.jl:78-80
    with pytest.raises(BO.DimensionMismatch):
        BO.batched_mul(rng.random((2, 2, 2)), rng.random((2, 2, 10)))
    with pytest.raises(BO.DimensionMismatch):
        BO.batched_mul(rng.random((2, 2, 2)), rng.random((10, 2, 2)))
    with pytest.raises(BO.DimensionMismatch):
        BO.batched_mul_into(np.zeros((2, 2, 10)), rng.random((2, 2, 2)), rng.random((2, 2, 2)))


def test_gemm_flags_alpha_beta_and_batch_of_one():
    rng = np.random.default_rng(1)
    M, N, K, nb = 6, 5, 4, 3
    for ta in "NT":
        for tb in "NT":
            A = rng.standard_normal((M, K, nb) if ta == "N" else (K, M, nb))
            B = rng.standard_normal((K, N, nb) if tb == "N" else (N, K, nb))
            C = rng.standard_normal((M, N, nb))
            got = BO.batched_gemm(ta, tb, 0.5, A, B, 2.0, C)
            want = 0.5 * bmm_test(A, B, transA=ta == "T", transB=tb == "T") + 2.0 * C
            np.testing.assert_allclose(got, want, rtol=1e-12)
    # a batch dimension of size 1 is reused for every k (src/gemm.jl:116-117); beta = 0 ignores what C held
    A = rng.standard_normal((M, K, 1)); B = rng.standard_normal((K, N, nb))
    C = np.full((M, N, nb), np.nan)
    got = BO.batched_gemm("N", "N", 1.0, A, B, 0.0, C)
    np.testing.assert_allclose(got, np.stack([A[:, :, 0] @ B[:, :, i] for i in range(nb)], axis=2))
    # matrices and N-d arrays (src/batched/batchedmul.jl:47-54, 112-125)
    A4 = rng.standard_normal((M, K, 2, 3)); B4 = rng.standard_normal((K, N, 2, 3))
    C4 = BO.batched_mul(A4, B4)
    assert C4.shape == (M, N, 2, 3)
    np.testing.assert_allclose(C4[:, :, 1, 2], A4[:, :, 1, 2] @ B4[:, :, 1, 2])
    Bm = rng.standard_normal((K, N))
    np.testing.assert_allclose(BO.batched_mul(A4[:, :, :, 0], Bm)[:, :, 1], A4[:, :, 1, 0] @ Bm)
