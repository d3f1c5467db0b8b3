"""CPU oracle of NNlib.jl's batched matrix product.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE: only the test-suite may import it.

``batched_gemm`` restates ``batched_gemm!`` (``src/gemm.jl:89-188``: one BLAS ``gemm`` per batch index,
``C_k = alpha * op(A_k) * op(B_k) + beta * C_k``, a batch dimension of size 1 in A or B being reused for
every k, ``:116-117,127-129``); ``batched_mul`` / ``batched_mul_into`` restate the front end
(``src/batched/batchedmul.jl:47-60, 225-303``: sizes, batch-size checks, the N-d reshape, and how the transpose
flags follow from the strides).  Arrays carry the reference's shapes ``(rows, cols, batch...)``; the only
arithmetic outside the reference's tree is the BLAS ``gemm`` itself, a plain matrix product (``numpy.matmul``).

Pinning: ``tests/test_batched_oracle.py`` checks it against the definitions the reference's own tests use
(``test/batchedmul.jl:6-16``: a slice-by-slice ``a[:,:,i] * b[:,:,i]`` with optional ``permutedims``) and the
cases of ``test/batchedmul.jl:40-49, 108-125``.
"""
from __future__ import annotations

import numpy as np


class DimensionMismatch(ValueError):
    """Julia's ``DimensionMismatch`` (``src/batched/batchedmul.jl:56-57``, ``src/gemm.jl:104-106``)."""


def batched_transpose(a: np.ndarray) -> np.ndarray:
    """``batched_transpose(A)``: ``PermutedDimsArray(A, (2, 1, 3))`` without copying
    (``src/batched/batchedadjtrans.jl``)."""
    if a.ndim != 3:
        raise ValueError("batched_transpose expects a 3-d array")
    return np.transpose(a, (1, 0, 2))


def batched_gemm(transA: str, transB: str, alpha, A: np.ndarray, B: np.ndarray, beta, C: np.ndarray) -> np.ndarray:
    """``batched_gemm!(transA, transB, alpha, A, B, beta, C)`` (``src/gemm.jl:89-188``), returning the new C."""
    if not (A.shape[2] == 1 or A.shape[2] == C.shape[2]):
        raise DimensionMismatch("batch size mismatch: A != C")
    if not (B.shape[2] == 1 or B.shape[2] == C.shape[2]):
        raise DimensionMismatch("batch size mismatch: B != C")
    m = A.shape[0 if transA == "N" else 1]
    ka = A.shape[1 if transA == "N" else 0]
    kb = B.shape[0 if transB == "N" else 1]
    n = B.shape[1 if transB == "N" else 0]
    if ka != kb or m != C.shape[0] or n != C.shape[1]:
        raise DimensionMismatch(f"A1 has size ({m},{ka}), B1 has size ({kb},{n}), C1 has size {C.shape[:2]}")
    out = np.empty_like(C)
    for k in range(C.shape[2]):
        a = A[:, :, k if A.shape[2] > 1 else 0]
        b = B[:, :, k if B.shape[2] > 1 else 0]
        a = a if transA == "N" else a.T
        b = b if transB == "N" else b.T
        prod = alpha * np.matmul(a, b)
        out[:, :, k] = prod if beta == 0 else prod + beta * C[:, :, k]     # beta = 0 never reads C (BLAS)
    return out


def batched_mul(A: np.ndarray, B: np.ndarray) -> np.ndarray:
    """``batched_mul(A, B)`` (``src/batched/batchedmul.jl:47-74``): ``C[:,:,k...] = A[:,:,k...] * B[:,:,k...]``;
    N-d arrays flatten their trailing dimensions (which must agree), 3-d arrays may have a batch dimension of
    size 1 on either side, a matrix counts as a batch of one (``:112-125``)."""
    A, B = np.asarray(A), np.asarray(B)
    if A.ndim == 2:
        A = A[:, :, None]
    if B.ndim == 2:
        B = B[:, :, None]
    if A.ndim > 3 or B.ndim > 3:
        if A.shape[2:] != B.shape[2:]:
            raise AssertionError("batch size has to be the same for the two arrays.")
        batch = A.shape[2:]
        A3 = np.reshape(A, A.shape[:2] + (-1,), order="F")
        B3 = np.reshape(B, B.shape[:2] + (-1,), order="F")
        C3 = batched_mul(A3, B3)
        return np.reshape(C3, C3.shape[:2] + batch, order="F")
    if not (A.shape[2] == B.shape[2] or A.shape[2] == 1 or B.shape[2] == 1):
        raise DimensionMismatch("batch size mismatch: A != B")
    if A.shape[1] != B.shape[0]:
        raise DimensionMismatch(f"A has size {A.shape[:2]}, B has size {B.shape[:2]}")
    T = np.result_type(A.dtype, B.dtype)
    C = np.zeros((A.shape[0], B.shape[1], max(A.shape[2], B.shape[2])), dtype=T)
    return batched_gemm("N", "N", T.type(1), A.astype(T, copy=False), B.astype(T, copy=False), T.type(0), C)


def batched_mul_into(C: np.ndarray, A: np.ndarray, B: np.ndarray, alpha=1.0, beta=0.0) -> np.ndarray:
    """``batched_mul!(C, A, B, alpha, beta)`` (``src/batched/batchedmul.jl:225-240``): equivalent to
    ``mul!(C[:,:,k], A[:,:,k], B[:,:,k], alpha, beta)`` for all k; returns the new C."""
    if not (A.shape[2] == C.shape[2] or A.shape[2] == 1):
        raise DimensionMismatch("batch size mismatch: A != C")
    if not (B.shape[2] == C.shape[2] or B.shape[2] == 1):
        raise DimensionMismatch("batch size mismatch: B != C")
    return batched_gemm("N", "N", alpha, A, B, beta, C)
