"""``batched_mul`` / ``batched_mul!`` of NNlib.jl for column-major CUDA tensors
(``src/batched/batchedmul.jl:47-74, 225-303``), on the library's own strided-batched product
(``nnlib_b200_batched_gemm``: tcgen05 kernel for Float16 / BFloat16, CUDA-core kernel for the rest).

Arrays are ``(rows, cols, batch...)`` with column-major strides.  ``batched_transpose(A)`` is the lazy
``PermutedDimsArray(A, (2, 1, 3))`` of the reference: a view with its first two strides swapped.  As in
``_batched_try_gemm!`` (``:258-303``) the BLAS transpose flags are read off the strides: a factor whose
first stride is 1 goes in as ``'N'``, one whose second stride is 1 as ``'T'`` of its parent; anything else
is first copied to a dense array (what the reference's ``_copy_if_faster`` does for the common case).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from .attention import _DTYPES, ArgumentError, _check, _status_word, _stream
from .layout import jl_empty, jl_reshape

__all__ = ["DimensionMismatch", "batched_mul", "batched_mul_", "batched_transpose", "batched_adjoint", "batched_mul_path"]


class DimensionMismatch(ValueError):
    """Julia's ``DimensionMismatch`` (``src/batched/batchedmul.jl:56-57``)."""


def batched_transpose(A: torch.Tensor) -> torch.Tensor:
    """Lazy transpose of every ``A[:, :, k]`` (``src/batched/batchedadjtrans.jl``): no data moves."""
    if A.ndim != 3:
        raise ArgumentError("batched_transpose expects a 3-d array")
    return A.transpose(0, 1)


batched_adjoint = batched_transpose          # real element types: adjoint == transpose


def _factor(X: torch.Tensor):
    """(parent data pointer holder, trans flag, ld, batch stride) of a 3-d factor, following
    ``_batched_try_gemm!`` (``src/batched/batchedmul.jl:270-300``)."""
    r, c, nb = X.shape
    s0, s1, s2 = X.stride()
    if s1 == 1 and r > 1 and (c == 1 or s0 >= c):
        trans, ld = 1, s0                       # stored as (c, r): the transpose of the factor
    elif s0 == 1 and (c == 1 or s1 >= r):
        trans, ld = 0, s1
    elif s1 == 1 and (c == 1 or s0 >= c):
        trans, ld = 1, s0
    else:
        Xc = jl_empty(tuple(X.shape), X.dtype, X.device)
        Xc.copy_(X)
        return _factor(Xc)
    rows_stored = c if trans else r
    ld = max(int(ld), rows_stored, 1)
    stride_b = 0 if nb == 1 else int(s2)
    if nb > 1 and stride_b == 0:
        Xc = jl_empty(tuple(X.shape), X.dtype, X.device)
        Xc.copy_(X)
        return _factor(Xc)
    return X, trans, ld, stride_b


def _params(Cm, A, B, alpha, beta):
    M, N, nb = Cm.shape
    Ak, ta, lda, sa = _factor(A)
    Bk, tb, ldb, sb = _factor(B)
    p = _lib.GemmParams()
    p.dtype = _DTYPES[Cm.dtype]
    p.transA, p.transB = ta, tb
    p.M, p.N, p.K, p.batch = M, N, A.shape[1], nb
    p.A, p.lda, p.strideA = Ak.data_ptr(), lda, sa
    p.B, p.ldb, p.strideB = Bk.data_ptr(), ldb, sb
    p.C, p.ldc = Cm.data_ptr(), max(int(Cm.stride(1)), M, 1)
    p.strideC = int(Cm.stride(2)) if nb > 1 else max(int(Cm.stride(1)), M, 1) * max(N, 1)
    p.alpha, p.beta = float(alpha), float(beta)
    p.status = _status_word(Cm.device).data_ptr()
    return p, (Ak, Bk)


def batched_mul_(Cm: torch.Tensor, A: torch.Tensor, B: torch.Tensor, alpha=1.0, beta=0.0) -> torch.Tensor:
    """``batched_mul!(C, A, B, α, β)``: ``C[:,:,k] = α A[:,:,k] B[:,:,k] + β C[:,:,k]``; a batch dimension of
    size 1 in ``A`` or ``B`` is used for every ``k``.  Never copies ``C``; returns it."""
    for name, t in (("C", Cm), ("A", A), ("B", B)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda or t.ndim != 3:
            raise TypeError(f"{name} must be a 3-d CUDA tensor")
    if not (A.dtype == B.dtype == Cm.dtype) or Cm.dtype not in _DTYPES:
        raise TypeError("batched_mul!: A, B and C must share one element type out of Float16, BFloat16, Float32")
    if not (A.shape[2] == Cm.shape[2] or A.shape[2] == 1):
        raise DimensionMismatch("batch size mismatch: A != C")
    if not (B.shape[2] == Cm.shape[2] or B.shape[2] == 1):
        raise DimensionMismatch("batch size mismatch: B != C")
    if A.shape[1] != B.shape[0] or A.shape[0] != Cm.shape[0] or B.shape[1] != Cm.shape[1]:
        raise DimensionMismatch(f"A has size {tuple(A.shape[:2])}, B has size {tuple(B.shape[:2])}, "
                                f"C has size {tuple(Cm.shape[:2])}")
    if Cm.numel() and Cm.stride(0) != 1 and Cm.shape[0] > 1:
        raise ArgumentError("batched_mul!: C must have unit stride along its first dimension")
    p, keep = _params(Cm, A, B, alpha, beta)
    with torch.cuda.device(Cm.device):
        _check(_lib.load().nnlib_b200_batched_gemm(C.byref(p), _stream()), "batched_gemm")
    del keep
    return Cm


def batched_mul_path(Cm, A, B) -> int:
    """``_lib.PATH_UMMA`` / ``PATH_SIMT``: the kernel family :func:`batched_mul_` would use (for tests)."""
    p, _ = _params(Cm, A, B, 1.0, 0.0)
    return _lib.load().nnlib_b200_batched_gemm_path(C.byref(p))


def batched_mul(A: torch.Tensor, B: torch.Tensor) -> torch.Tensor:
    """``batched_mul(A, B)`` / ``A ⊠ B``: ``C[:,:,k...] = A[:,:,k...] * B[:,:,k...]``.  N-d arrays flatten their
    (equal) trailing dimensions; for 3-d arrays either side may have a batch of one; a matrix counts as a
    batch of one (``src/batched/batchedmul.jl:47-60, 112-125``)."""
    if A.ndim == 2:
        A = A.unsqueeze(2)
    if B.ndim == 2:
        B = B.unsqueeze(2)
    if A.ndim > 3 or B.ndim > 3:
        if tuple(A.shape[2:]) != tuple(B.shape[2:]):
            raise AssertionError("batch size has to be the same for the two arrays.")
        batch = tuple(A.shape[2:])
        C3 = batched_mul(jl_reshape(A, (A.shape[0], A.shape[1], -1)), jl_reshape(B, (B.shape[0], B.shape[1], -1)))
        return jl_reshape(C3, tuple(C3.shape[:2]) + batch)
    if not (A.shape[2] == B.shape[2] or A.shape[2] == 1 or B.shape[2] == 1):
        raise DimensionMismatch("batch size mismatch: A != B")
    Cm = jl_empty((A.shape[0], B.shape[1], max(A.shape[2], B.shape[2])), A.dtype, A.device)
    return batched_mul_(Cm, A, B)
