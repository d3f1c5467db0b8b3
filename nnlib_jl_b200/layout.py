"""Column-major ("Julia layout") torch tensors.

NNlib's arrays are column-major: element ``(e, l, b)`` of an ``(E, L, B)``
array sits at linear offset ``e + E*l + E*L*b``.  A torch tensor with the SAME
shape ``(E, L, B)`` and strides ``(1, E, E*L)`` is exactly that memory, so the
host API keeps the reference's shapes and index meaning.  Such a tensor is a
permuted view of a contiguous tensor of the reversed shape; the helpers here
create, test, reshape and convert them without copies.
"""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch


def _rev(n: int):
    return tuple(range(n - 1, -1, -1))


def jl_empty(shape: Sequence[int], dtype=torch.float32, device="cpu") -> torch.Tensor:
    """Uninitialised column-major tensor of the given (Julia) shape."""
    shape = tuple(int(s) for s in shape)
    strides, acc = [], 1
    for n in shape:                      # first dimension fastest (an empty dimension counts as 1, as torch does)
        strides.append(acc)
        acc *= max(n, 1)
    return torch.empty_strided(shape, strides, dtype=dtype, device=device)


def jl_zeros(shape, dtype=torch.float32, device="cpu") -> torch.Tensor:
    t = jl_empty(shape, dtype, device)
    t.zero_()
    return t


def is_column_major(t: torch.Tensor) -> bool:
    """Dense column-major?  Size-1 dimensions may carry any stride."""
    expected = 1
    for size, stride in zip(t.shape, t.stride()):
        if size != 1 and stride != expected:
            return False
        expected *= size
    return True


def jl_reshape(t: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
    """Column-major reshape (Julia's ``reshape``) of a dense column-major
    tensor; never copies.  One entry of ``shape`` may be -1."""
    if not is_column_major(t):
        raise ValueError("jl_reshape needs a dense column-major tensor")
    shape = tuple(int(s) for s in shape)
    flat = t.permute(_rev(t.ndim)) if t.ndim else t   # row-major view of the same memory
    out = flat.reshape(shape[::-1])
    return out.permute(_rev(len(shape))) if shape else out


def jl_from_numpy(a: np.ndarray, dtype=None, device="cpu") -> torch.Tensor:
    """numpy array (any memory order) with a Julia shape → column-major tensor."""
    a = np.asarray(a)
    t = torch.from_numpy(np.ascontiguousarray(a.transpose(_rev(a.ndim))))
    if dtype is not None:
        t = t.to(dtype)
    t = t.to(device)
    return t.permute(_rev(a.ndim)) if a.ndim else t


def jl_to_numpy(t: torch.Tensor) -> np.ndarray:
    """Tensor → numpy array of the same shape; bf16 / f16 are widened to float32."""
    t = t.detach()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    return t.cpu().numpy()


def as_column_major(t: torch.Tensor) -> torch.Tensor:
    """Column-major copy of ``t`` unless it already is column-major."""
    if is_column_major(t):
        return t
    out = jl_empty(t.shape, t.dtype, t.device)
    out.copy_(t)
    return out
