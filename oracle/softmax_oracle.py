"""CPU oracle of softmax / logsoftmax and their pullbacks.

TEST INFRASTRUCTURE ONLY: imported by ``tests/`` (and by nothing the library
ships).  A numpy restatement of NNlib.jl ``src/softmax.jl``: ``_softmax!``
(:69-79), ``_∇softmax!`` (:98-101), ``_logsoftmax!`` (:147-157) and
``∇logsoftmax`` (:170-190), including the branch for non-finite column maxima
(:71-76, :149-154).  Pinned by the reference's own known-answer tests
(``test/softmax.jl:16-75``) in ``tests/test_softmax_oracle.py``.  ``dims`` is
1-based; ``None`` stands for Julia's ``:`` (all dimensions).
"""
from __future__ import annotations

import numpy as np


def _axis(x, dims):
    if dims is None:
        return None
    if isinstance(dims, (tuple, list)):
        return tuple(d - 1 for d in dims)
    return dims - 1


def _pad(x, dims):
    """Julia lets ``dims`` name trailing singleton dimensions the array does not have: add them."""
    x = np.asarray(x)
    top = max(dims) if isinstance(dims, (tuple, list)) else (dims or 0)
    return x.reshape(x.shape + (1,) * max(0, top - x.ndim)), x.shape


def softmax(x, dims=1):
    x, shape = _pad(x, dims)
    return _softmax(x, dims).reshape(shape)


def _softmax(x, dims):
    x = x.astype(np.float64 if x.dtype == np.float64 else np.float32)
    ax = _axis(x, dims)
    with np.errstate(invalid="ignore", over="ignore"):
        m = np.max(x, axis=ax, keepdims=True)                       # fast_maximum (:118): NaN propagates
        finite = np.exp(x - m)
        out = np.where(np.isposinf(m), np.where(np.isposinf(x), 1.0, 0.0), finite).astype(x.dtype)
        # (the sum is accumulated in Float64: numpy adds one by one over several axes at once, which costs a
        # Float32 sum of 10^4 terms five digits; the reference's sum! is pairwise)
        return out / np.sum(out, axis=ax, keepdims=True, dtype=np.float64).astype(x.dtype)


def logsoftmax(x, dims=1):
    x, shape = _pad(x, dims)
    return _logsoftmax(x, dims).reshape(shape)


def _logsoftmax(x, dims):
    x = x.astype(np.float64 if x.dtype == np.float64 else np.float32)
    ax = _axis(x, dims)
    with np.errstate(invalid="ignore", over="ignore", divide="ignore"):
        m = np.max(x, axis=ax, keepdims=True)
        out = np.where(np.isposinf(m), np.where(np.isposinf(x), 0.0, -np.inf), x - m).astype(x.dtype)
        return out - np.log(np.sum(np.exp(out), axis=ax, keepdims=True, dtype=np.float64)).astype(x.dtype)


def softmax_pullback(dy, y, dims=1):
    (y, shape), (dy, _) = _pad(y, dims), _pad(dy, dims)
    ax = _axis(y, dims)
    dx = dy * y
    return (dx - y * np.sum(dx, axis=ax, keepdims=True, dtype=np.float64).astype(dx.dtype)).reshape(shape)


def logsoftmax_pullback(dy, y, dims=1):
    (y, shape), (dy, _) = _pad(y, dims), _pad(dy, dims)
    ax = _axis(y, dims)
    return (dy - np.sum(dy, axis=ax, keepdims=True, dtype=np.float64).astype(dy.dtype) * np.exp(y)).reshape(shape)
