"""CPU oracle for the dropout keep-mask: Philox4x32-10, restated scalar-first.

TEST INFRASTRUCTURE ONLY (see attention_oracle.py).  The reference draws its
dropout mask with ``rand!`` (NNlib.jl src/dropout.jl:77-87), which no other
implementation can reproduce bit for bit; the library replaces the draw with
the counter-based generator Philox4x32-10 (Salmon, Moraes, Dror, Shaw:
"Parallel random numbers: as easy as 1, 2, 3", SC'11).  This file restates
that published algorithm independently of the package's own host copy, is
pinned by the Random123 known-answer vectors in the tests, and defines which
score positions survive: position (j, i, h, b) is dropped iff 16-bit lane
``j % 8`` (low half of an output word for even j, high half for odd j, word
``(j % 8) // 2``) of ``philox(counter = (j // 8, r_lo, r_hi + off_hi, off_lo),
key = seed)`` is ``< floor(p * 2**16)``, with ``r = i + Lq*((h+h0) + H_total*(b+b0))``.
"""
from __future__ import annotations

import numpy as np

M0, M1 = 0xD2511F53, 0xCD9E8D57
W0, W1 = 0x9E3779B9, 0xBB67AE85
U32 = 0xFFFFFFFF


def philox4x32_10_scalar(ctr, key):
    """Pure-python reference: ctr = 4 ints, key = 2 ints → 4 ints."""
    c0, c1, c2, c3 = (int(c) & U32 for c in ctr)
    k0, k1 = (int(k) & U32 for k in key)
    for _ in range(10):
        p0 = M0 * c0
        p1 = M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & U32, p1 & U32, ((p0 >> 32) ^ c3 ^ k1) & U32, p0 & U32
        k0 = (k0 + W0) & U32
        k1 = (k1 + W1) & U32
    return c0, c1, c2, c3


def philox4x32_10_np(c0, c1, c2, c3, k0, k1):
    """numpy-vectorised form of the same rounds (uint64 arithmetic)."""
    c0, c1, c2, c3 = np.broadcast_arrays(*(np.asarray(c, dtype=np.uint64) for c in (c0, c1, c2, c3)))
    k0, k1 = int(k0) & U32, int(k1) & U32
    m32 = np.uint64(U32)
    s32 = np.uint64(32)
    for _ in range(10):
        p0 = np.uint64(M0) * c0
        p1 = np.uint64(M1) * c2
        c0, c1, c2, c3 = ((p1 >> s32) ^ c1 ^ np.uint64(k0)) & m32, p1 & m32, \
                         ((p0 >> s32) ^ c3 ^ np.uint64(k1)) & m32, p0 & m32
        k0 = (k0 + W0) & U32
        k1 = (k1 + W1) & U32
    return c0, c1, c2, c3


def keep_mask(shape4, p, seed, offset=0, h0=0, b0=0, H_total=None):
    """Bool array (Lkv, Lq, H, B): True where the score survives dropout."""
    Lkv, Lq, H, B = (int(s) for s in shape4)
    H_total = H if H_total is None else int(H_total)
    thresh = min(int(np.floor(float(np.float32(p)) * 2.0 ** 16)), 0xFFFF)
    out = np.empty((Lkv, Lq, H, B), dtype=bool)
    j = np.arange(Lkv, dtype=np.uint64)
    for b in range(B):
        for h in range(H):
            i = np.arange(Lq, dtype=np.uint64)
            r = i + np.uint64(Lq) * np.uint64((h + h0) + H_total * (b + b0))
            words = philox4x32_10_np((j >> np.uint64(3))[:, None], (r & np.uint64(U32))[None, :],
                                     (((r >> np.uint64(32)) + np.uint64((offset >> 32) & U32)) & np.uint64(U32))[None, :],
                                     np.uint64(offset & U32), seed & U32, (seed >> 32) & U32)
            w = np.stack(words, axis=0)                       # (4, Lkv, Lq)
            lane = (j & np.uint64(7)).astype(np.int64)
            sel = (lane >> 1)[None, :, None]
            word = np.take_along_axis(w, np.broadcast_to(sel, (1, Lkv, Lq)), axis=0)[0]
            half = (word >> (np.uint64(16) * (lane & 1).astype(np.uint64))[:, None]) & np.uint64(0xFFFF)
            out[:, :, h, b] = half >= np.uint64(thresh)
    return out
