"""``softmax`` / ``logsoftmax`` over one dimension of a column-major CUDA array
and their pullbacks (NNlib.jl ``src/softmax.jl:56-79, 118-157``; the CUDA
methods live in ``ext/NNlibCUDACUDNNExt/softmax.jl``), on the library's own
kernels.  ``dims`` is 1-based like the reference's; a ``Colon`` (all
dimensions) is spelled ``dims=None``; a tuple of consecutive dimensions is reduced as one.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib
from .attention import _DTYPES, ArgumentError, _check, _require_dense_cuda, _stream
from .layout import is_column_major, jl_empty

__all__ = ["softmax", "logsoftmax", "softmax_pullback", "logsoftmax_pullback"]


def _split(shape, dims):
    """(inner, n, outer) of a reduction over Julia dimension(s) ``dims``: an int, a tuple of consecutive
    dimensions (they merge into one extent of the column-major array) or None for all of them."""
    shape = tuple(int(s) for s in shape)
    if dims is None:
        return 1, math.prod(shape), 1
    ds = sorted(set(int(d) for d in dims)) if isinstance(dims, (tuple, list)) else [int(dims)]
    if not ds or ds[0] < 1:
        raise ArgumentError(f"dims = {dims} is not a dimension of an array of size {shape}")
    if ds != list(range(ds[0], ds[-1] + 1)):
        raise ArgumentError(f"dims = {dims}: only consecutive dimensions can be reduced in one pass")
    full = shape + (1,) * max(0, ds[-1] - len(shape))      # trailing singleton dimensions, as Julia allows
    lo, hi = ds[0] - 1, ds[-1]
    return math.prod(full[:lo]), math.prod(full[lo:hi]), math.prod(full[hi:])


def _run(x: torch.Tensor, dy: Optional[torch.Tensor], dims, log: bool, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if isinstance(x, torch.Tensor) and x.is_cuda and x.numel() == 0:
        _split(x.shape, dims)                       # still validates dims
        return out if out is not None else jl_empty(tuple(x.shape), x.dtype, x.device)
    _require_dense_cuda("x", x)
    if not is_column_major(x):
        raise ArgumentError("softmax: the array must be dense column-major")
    if dy is not None:
        _require_dense_cuda("dy", dy)
        if tuple(dy.shape) != tuple(x.shape) or dy.dtype != x.dtype or not is_column_major(dy):
            raise ArgumentError("softmax pullback: dy must match y in size, eltype and layout")
    if out is None:
        out = jl_empty(tuple(x.shape), x.dtype, x.device)
    else:
        # softmax!(out, x): the result array is the caller's; it may be x (or dy) itself
        _require_dense_cuda("out", out)
        if tuple(out.shape) != tuple(x.shape) or out.dtype != x.dtype or not is_column_major(out) \
                or out.device != x.device:
            raise ArgumentError("softmax!: out must match the input in size, eltype, layout and device")
    inner, n, outer = _split(x.shape, dims)
    p = _lib.SoftmaxParams()
    p.dtype = _DTYPES[x.dtype]
    p.log = 1 if log else 0
    p.inner, p.n, p.outer = inner, n, outer
    p.x = x.data_ptr()
    p.dy = dy.data_ptr() if dy is not None else None
    p.out = out.data_ptr()
    lib = _lib.load()
    with torch.cuda.device(x.device):
        if dy is None:
            _check(lib.nnlib_b200_softmax_fwd(C.byref(p), _stream()), "softmax_fwd")
        else:
            _check(lib.nnlib_b200_softmax_bwd(C.byref(p), _stream()), "softmax_bwd")
    return out


def softmax(x: torch.Tensor, *, dims: Optional[int] = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``softmax(x; dims)`` (``src/softmax.jl:56``); with ``out`` it is ``softmax!(out, x; dims)``
    (``:66-67``) and ``out`` may be ``x`` itself."""
    return _run(x, None, dims, log=False, out=out)


def logsoftmax(x: torch.Tensor, *, dims: Optional[int] = 1, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``logsoftmax(x; dims)`` (``src/softmax.jl:133``); ``out`` as in :func:`softmax`."""
    return _run(x, None, dims, log=True, out=out)


def softmax_pullback(dy: torch.Tensor, y: torch.Tensor, *, dims: Optional[int] = 1,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``∇softmax(dy, y; dims) = y .* (dy .- sum(dy .* y; dims))`` (``src/softmax.jl:84-101``); with ``out``
    it is ``∇softmax!(out, dy, y)``, and ``out`` may be ``dy`` or ``y``."""
    return _run(y, dy, dims, log=False, out=out)


def logsoftmax_pullback(dy: torch.Tensor, y: torch.Tensor, *, dims: Optional[int] = 1,
                        out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``∇logsoftmax(dy, y; dims) = dy .- sum(dy; dims) .* exp.(y)`` (``src/softmax.jl:164-190``); ``out`` as
    in :func:`softmax_pullback`."""
    return _run(y, dy, dims, log=True, out=out)
