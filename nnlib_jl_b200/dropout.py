"""Counter-based dropout for attention scores.

:class:`PhiloxDropout` is the ``fdrop`` the fused kernels understand: instead
of drawing ``rand!`` into a scores-sized array (NNlib.jl src/dropout.jl:77-87)
the keep/drop decision of score ``(j, i, h, b)`` is a pure function of the seed
and the position, computed in the kernel with Philox4x32-10.  The rule is the
reference's: keep iff ``u > p``, kept entries scaled by ``1/(1-p)``.  The same
object applied to a materialised score array (CPU or CUDA tensor) reproduces
that mask on the host, so it is a drop-in ``fdrop`` for the reference's generic
path as well.
"""
from __future__ import annotations

import itertools

import numpy as np
import torch

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Vectorised Philox4x32-10.  ``c*``: uint32 arrays (broadcastable), ``k*``:
    python ints.  Returns four uint32 arrays."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) & _MASK32 for c in (c0, c1, c2, c3))
    c0, c1, c2, c3 = np.broadcast_arrays(c0, c1, c2, c3)
    for r in range(10):
        kk0 = np.uint64((k0 + r * _W0) & 0xFFFFFFFF)
        kk1 = np.uint64((k1 + r * _W1) & 0xFFFFFFFF)
        p0 = _M0 * c0
        p1 = _M1 * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ kk0) & _MASK32
        n1 = p1 & _MASK32
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ kk1) & _MASK32
        n3 = p0 & _MASK32
        c0, c1, c2, c3 = n0, n1, n2, n3
    return tuple(c.astype(np.uint32) for c in (c0, c1, c2, c3))


def drop_threshold(p: float) -> int:
    """A score is dropped iff its 16-bit random lane is ``< floor(p * 2**16)`` — the
    integer form of the reference's keep rule ``rand > p``."""
    return min(int(np.floor(float(np.float32(p)) * 65536.0)), 0xFFFF)


def keep_mask(shape4, p: float, seed: int, offset: int = 0, h0: int = 0, b0: int = 0, H_total=None) -> np.ndarray:
    """Boolean keep-mask of a ``(Lkv, Lq, H, B)`` score array, identical to the
    one the kernels draw (see the dropout comment in ``include/nnlib_b200.h``)."""
    Lkv, Lq, H, B = (int(s) for s in shape4)
    H_total = H if H_total is None else int(H_total)
    j = np.arange(Lkv, dtype=np.uint64).reshape(Lkv, 1, 1, 1)
    i = np.arange(Lq, dtype=np.uint64).reshape(1, Lq, 1, 1)
    h = np.arange(H, dtype=np.uint64).reshape(1, 1, H, 1) + np.uint64(h0)
    b = np.arange(B, dtype=np.uint64).reshape(1, 1, 1, B) + np.uint64(b0)
    r = i + np.uint64(Lq) * (h + np.uint64(H_total) * b)
    off_lo, off_hi = offset & 0xFFFFFFFF, (offset >> 32) & 0xFFFFFFFF
    c0 = j >> np.uint64(3)
    c1 = r & _MASK32
    c2 = ((r >> np.uint64(32)) + np.uint64(off_hi)) & _MASK32
    c3 = np.uint64(off_lo)
    w = philox4x32_10(c0, c1, c2, c3, seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    w = np.stack(np.broadcast_arrays(*w), axis=0)            # (4, Lkv, Lq, H, B)
    lane = j & np.uint64(7)                                   # eight 16-bit lanes per Philox call
    sel = np.broadcast_to((lane >> np.uint64(1)).astype(np.int64), w.shape[1:])
    word = np.take_along_axis(w, sel[None], axis=0)[0].astype(np.uint32)
    half = (word >> (np.uint32(16) * (lane & np.uint64(1)).astype(np.uint32))) & np.uint32(0xFFFF)
    return half >= np.uint32(drop_threshold(p))


class PhiloxDropout:
    """``fdrop`` for :func:`dot_product_attention` that the fused kernels run
    in place.  Every call consumes one Philox offset, so successive calls draw
    independent masks; two objects built with the same ``(p, seed, offset)``
    draw the same sequence."""

    _seed_counter = itertools.count(0x5EED)

    def __init__(self, p: float, seed: int | None = None, offset: int = 0):
        if not (0.0 <= p < 1.0):
            raise ValueError("PhiloxDropout expects a probability 0 <= p < 1")
        self.p = float(p)
        self.seed = int(seed) if seed is not None else next(PhiloxDropout._seed_counter)
        self.offset = int(offset)

    def take_offset(self) -> int:
        off = self.offset
        self.offset += 1
        return off

    def __call__(self, alpha):
        """Apply to a materialised ``(Lkv, Lq, H, B...)`` score array."""
        if self.p == 0.0:
            return alpha
        off = self.take_offset()
        shape = tuple(alpha.shape)
        if len(shape) < 3:
            raise ValueError("PhiloxDropout expects a (Lkv, Lq, H, B...) score array")
        B = int(np.prod(shape[3:])) if len(shape) > 3 else 1
        keep = keep_mask(shape[:3] + (B,), self.p, self.seed, off).reshape(shape, order="F")
        scale = 1.0 / (1.0 - self.p)
        if isinstance(alpha, torch.Tensor):
            k = torch.from_numpy(np.ascontiguousarray(keep)).to(alpha.device)
            return alpha * (k.to(alpha.dtype) * scale)
        return alpha * (keep.astype(alpha.dtype) * alpha.dtype.type(scale))

    def __repr__(self):
        return f"PhiloxDropout(p={self.p}, seed={self.seed}, offset={self.offset})"
