"""CPU oracle: a numpy restatement of NNlib.jl's multi-head attention path.

THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke
check and the CPU-baseline leg of the benchmark may import it; the shipped
library never routes through it.

Every function follows the reference step by step and cites the lines it
restates (paths are relative to the NNlib.jl project root).  Arrays use the
reference's own (Julia) shapes: ``q`` is ``(E, Lq, B...)``, the scores ``α`` are
``(Lkv, Lq, H, B...)``.  numpy holds them in whatever memory order it likes; the
*index meaning* is the reference's.  The only arithmetic that lives outside the
reference's tree is the BLAS ``sgemm`` behind ``batched_mul`` (OpenBLAS through
libblastrampoline, ``src/gemm.jl:141-149``): a plain matrix product, restated
here with ``numpy.matmul``.

Pinning: `tests/test_oracle_golden.py` checks this file against every
known-answer vector the reference's own tests hold for the path
(``test/attention.jl:25-34`` and the softmax tables of ``test/softmax.jl``),
transcribed under ``tests/golden/``.
"""
from __future__ import annotations

import math
from typing import Callable, Optional

import numpy as np

__all__ = [
    "ArgumentError",
    "dot_product_attention",
    "dot_product_attention_scores",
    "make_causal_mask",
    "softmax",
    "batched_mul",
    "dropout_apply",
    "split_heads",
    "join_heads",
    "attention_rows",
]


class ArgumentError(ValueError):
    """Stands for Julia's ``ArgumentError`` (``src/attention.jl:42,55-78``)."""


# --------------------------------------------------------------------------
# building blocks
# --------------------------------------------------------------------------

def split_heads(x: np.ndarray, nheads: int) -> np.ndarray:
    """``reshape(x, size(x,1) ÷ nheads, nheads, size(x)[2:end]...)``
    (``src/attention.jl:158``).  Julia reshapes are column-major, hence
    ``order='F'``: head ``h`` owns features ``h*d .. h*d+d-1``."""
    e = x.shape[0]
    return np.reshape(x, (e // nheads, nheads) + x.shape[1:], order="F")


def join_heads(x: np.ndarray) -> np.ndarray:
    """``reshape(x, :, size(x)[3:end]...)`` (``src/attention.jl:159``)."""
    return np.reshape(x, (x.shape[0] * x.shape[1],) + x.shape[2:], order="F")


def batched_mul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """``C[:,:,k...] = A[:,:,k...] * B[:,:,k...]`` for every trailing batch
    index (``src/batched/batchedmul.jl:47-60``; the CPU kernel is one ``gemm``
    per slice, ``src/gemm.jl:121-161``)."""
    # numpy.matmul batches over LEADING axes; move the reference's trailing
    # batch axes to the front and back again.
    nb = a.ndim - 2
    perm_in = tuple(range(2, 2 + nb)) + (0, 1)
    perm_out = (nb, nb + 1) + tuple(range(nb))
    c = np.matmul(np.transpose(a, perm_in), np.transpose(b, perm_in))
    return np.transpose(c, perm_out)


def softmax(x: np.ndarray, dims: int = 0) -> np.ndarray:
    """``softmax(x; dims)`` → ``_softmax!`` (``src/softmax.jl:56,69-79``).

    ``dims`` is 0-based here (the reference's ``dims=1`` is ``dims=0``).
    Follows the reference's two branches: when every maximum is finite,
    ``exp(x - max)``; otherwise a maximum of ``+Inf`` turns the slice into an
    indicator of its ``+Inf`` entries and a maximum of ``-Inf`` (a slice with
    nothing to attend to) yields ``exp(-Inf - -Inf) = NaN`` throughout.
    """
    x = np.asarray(x)
    ft = x.dtype if np.issubdtype(x.dtype, np.floating) else np.dtype(np.float64)
    x = x.astype(ft, copy=False)
    one, zero, inf = ft.type(1), ft.type(0), ft.type(np.inf)
    # fast_maximum: reduce(max, x; dims, init=-Inf)  (src/softmax.jl:118)
    max_ = np.max(x, axis=dims, keepdims=True, initial=-np.inf)
    with np.errstate(invalid="ignore", over="ignore"):
        if np.all(np.isfinite(max_)):
            out = np.exp(x - max_)
        else:
            out = np.where(max_ == inf, np.where(x == inf, one, zero),
                           np.exp(x - max_)).astype(ft, copy=False)
        tmp = np.sum(out, axis=dims, keepdims=True)
        out = out / tmp
    return out


def dropout_apply(alpha: np.ndarray, u: np.ndarray, p: float) -> np.ndarray:
    """``_dropout!`` with the uniform draws ``u`` made explicit: keep iff
    ``u > p``, kept entries scaled by ``1/(1-p)`` (``src/dropout.jl:77-87``)."""
    val = alpha.dtype.type(1.0 / (1.0 - p))
    return ((u > p) * val) * alpha


def make_causal_mask(x: np.ndarray, dims: int = 2) -> np.ndarray:
    """``triu(trues_like(x, (len, len)))`` ⇒ ``m[i, j] = (i <= j)`` with
    ``i`` the kv index and ``j`` the query index (``src/attention.jl:149-153``).
    ``dims`` is 1-based like the reference's keyword."""
    n = x.shape[dims - 1]
    return np.triu(np.ones((n, n), dtype=bool))


# --------------------------------------------------------------------------
# the path itself
# --------------------------------------------------------------------------

def _bcast_to_scores(a: np.ndarray, ndim: int = 4) -> np.ndarray:
    """Julia broadcasting aligns LEADING dimensions (missing trailing dims
    count as 1); numpy aligns trailing ones.  Pad with trailing singleton axes
    so that ``a`` broadcasts against a ``(Lkv, Lq, H, B)`` array the way the
    reference's ``logits .+ bias`` does (``src/attention.jl:131,137``)."""
    a = np.asarray(a)
    if a.ndim > ndim:
        raise ArgumentError("bias/mask has more dimensions than the scores")
    return a.reshape(a.shape + (1,) * (ndim - a.ndim))


def dot_product_attention_scores(
    q: np.ndarray,
    k: np.ndarray,
    bias: Optional[np.ndarray] = None,
    *,
    fdrop: Callable[[np.ndarray], np.ndarray] = lambda a: a,
    mask: Optional[np.ndarray] = None,
) -> np.ndarray:
    """``dot_product_attention_scores`` (``src/attention.jl:112-127``).

    ``q``: ``(d, H, Lq, B)``, ``k``: ``(d, H, Lkv, B)`` → ``α``:
    ``(Lkv, Lq, H, B)``.  Steps, in the reference's order: permute k and q,
    scale **q** by ``1/sqrt(d)`` in the element type (``:118``), batched
    product (``:119``), ``+ bias`` (``:122``), masked entries to ``typemin``
    (``:123,133-138``), ``softmax(dims=1)`` (``:125``), ``fdrop`` (``:126``).
    """
    if q.ndim != 4 or k.ndim != 4:
        raise ArgumentError("scores expect 4-d (d, H, L, B) inputs")
    T = np.result_type(q.dtype, k.dtype)
    if not np.issubdtype(T, np.floating):
        T = np.dtype(np.float64)
    q = q.astype(T, copy=False)
    k = k.astype(T, copy=False)
    kt = np.transpose(k, (2, 0, 1, 3))                      # (Lkv, d, H, B)
    qt = np.transpose(q, (0, 2, 1, 3)) / T.type(math.sqrt(q.shape[0]))  # (d, Lq, H, B)
    logits = batched_mul(kt, qt)                            # (Lkv, Lq, H, B)
    if bias is not None:
        logits = logits + _bcast_to_scores(bias)
    if mask is not None:
        neginf = logits.dtype.type(-np.inf)
        logits = np.where(_bcast_to_scores(mask).astype(bool), logits, neginf)
    alpha = softmax(logits, dims=0)
    return fdrop(alpha)


def _dot_product_attention(q4, k4, v4, bias, fdrop, mask):
    """``_dot_product_attention`` (``src/attention.jl:86-101``):
    ``x[d,h,i,b] = Σ_j α[j,i,h,b] · v[d,h,j,b]``."""
    alpha = dot_product_attention_scores(q4, k4, bias, fdrop=fdrop, mask=mask)
    vt = np.transpose(v4, (0, 2, 1, 3))                     # (dv, Lkv, H, B)
    x = batched_mul(vt.astype(alpha.dtype, copy=False), alpha)  # (dv, Lq, H, B)
    x = np.transpose(x, (0, 2, 1, 3))                       # (dv, H, Lq, B)
    return x, alpha


def dot_product_attention(
    q: np.ndarray,
    k: np.ndarray,
    v: np.ndarray,
    bias: Optional[np.ndarray] = None,
    *,
    fdrop: Callable[[np.ndarray], np.ndarray] = lambda a: a,
    mask: Optional[np.ndarray] = None,
    nheads: int = 1,
):
    """``dot_product_attention`` — the N-d wrapper (``src/attention.jl:40-50``)
    and the validated 3-d method (``:52-84``) in one function.

    Returns ``(x, α)`` with ``x``: ``(Ev, Lq, B...)`` and ``α``:
    ``(Lkv, Lq, H, B...)``; ``α`` is the array *after* ``fdrop`` and ``x`` is
    computed from that same array (``:91,97,126``).
    """
    q, k, v = (np.asarray(a) for a in (q, k, v))
    if not (q.ndim == k.ndim == v.ndim) or q.ndim < 2:
        raise ArgumentError("q, k, v must have the same number of dimensions (>= 2)")
    batch_size = q.shape[2:]
    if q.ndim != 3:
        if not (batch_size == k.shape[2:] == v.shape[2:]):
            raise ArgumentError("Batch dimensions have to be the same.")
        q, k, v = (np.reshape(a, a.shape[:2] + (-1,), order="F") for a in (q, k, v))
    if any(a.shape[0] % nheads != 0 for a in (q, k, v)):
        raise ArgumentError(
            "First dimension in query, key and value must be divisible by `nheads`.")
    if not (q.shape[2] == k.shape[2] == v.shape[2]):
        raise ArgumentError("Batch dimensions have to be the same.")
    if q.shape[0] != k.shape[0]:
        raise ArgumentError("First dimension in query and key has to be the same.")
    if k.shape[1] != v.shape[1]:
        raise ArgumentError("Second dimension in key and value has to be the same.")

    q4, k4, v4 = (split_heads(a, nheads) for a in (q, k, v))
    x4, alpha = _dot_product_attention(q4, k4, v4, bias, fdrop, mask)
    x = join_heads(x4)
    if len(batch_size) != 1:
        x = np.reshape(x, x.shape[:2] + batch_size, order="F")
        alpha = np.reshape(alpha, alpha.shape[:3] + batch_size, order="F")
    return x, alpha


# --------------------------------------------------------------------------
# row-sampled oracle for sizes whose full score array does not fit anywhere
# --------------------------------------------------------------------------

def attention_rows(q, k, v, nheads, rows, b, h, *, causal=False, mask=None,
                   bias=None, dtype=np.float64):
    """Exact attention for the chosen query ``rows`` of one ``(b, h)`` unit.

    Same arithmetic as :func:`dot_product_attention` restricted to a set of
    query positions, in ``dtype`` (Float64 by default), so that the size of
    the score array is ``len(rows) × Lkv`` instead of ``Lq × Lkv × H × B``.
    ``q``, ``k``, ``v`` are 3-d ``(E, L, B)`` arrays.  Returns
    ``(x_rows (dv, n), alpha_rows (Lkv, n), lse (n,))`` where ``lse`` is the
    natural-log sum of exponentials of the masked, biased logits.
    """
    rows = np.asarray(rows)
    d = q.shape[0] // nheads
    dv = v.shape[0] // nheads
    qh = q[h * d:(h + 1) * d, :, b][:, rows].astype(dtype)          # (d, n)
    kh = k[h * d:(h + 1) * d, :, b].astype(dtype)                   # (d, Lkv)
    vh = v[h * dv:(h + 1) * dv, :, b].astype(dtype)                 # (dv, Lkv)
    logits = kh.T @ (qh / dtype(math.sqrt(d)))                      # (Lkv, n)
    lkv = kh.shape[1]
    if bias is not None:
        bb = np.broadcast_to(_bcast_to_scores(bias), (lkv, q.shape[1], nheads, q.shape[2]))
        logits = logits + bb[:, rows, h, b].astype(dtype)
    keep = np.ones_like(logits, dtype=bool)
    if causal:
        keep &= np.arange(lkv)[:, None] <= rows[None, :]
    if mask is not None:
        mm = np.broadcast_to(_bcast_to_scores(mask), (lkv, q.shape[1], nheads, q.shape[2]))
        keep &= mm[:, rows, h, b].astype(bool)
    logits = np.where(keep, logits, -np.inf)
    alpha = softmax(logits, dims=0)
    with np.errstate(divide="ignore", invalid="ignore"):
        m = np.max(logits, axis=0)
        lse = m + np.log(np.sum(np.exp(logits - m), axis=0))
    x = vh @ alpha
    return x, alpha, lse


# --------------------------------------------------------------------------
# gradient of the path (what Zygote composes from the reference's rrules)
# --------------------------------------------------------------------------

def dot_product_attention_grad(q, k, v, dy, bias=None, *, mask=None, nheads=1, keep=None, p=0.0):
    """Pullback of ``y = dot_product_attention(q, k, v, bias; mask, nheads, fdrop)[1]`` for 3-d inputs,
    assembled from the reference's own rules: ``rrule(batched_mul)`` (``dA = dC·Bᵀ``, ``dB = Aᵀ·dC``,
    ``src/batched/batchedmul.jl:96-110``), ``∇softmax`` (``dx = y .* (dy .- sum(dy .* y; dims))``,
    ``src/softmax.jl:84-110``), the dropout pullback (``dy .* keep ./ (1-p)``, ``src/dropout.jl:106-122``),
    ``ifelse`` masking (no gradient through masked entries) and the ``1/sqrt(d)`` scaling of q
    (``src/attention.jl:118``).  ``keep`` is the Bool ``(Lkv, Lq, H, B)`` dropout mask (None: no dropout).
    Returns ``(dq, dk, dv, dbias)``; ``dbias`` has the shape of ``bias`` (None without bias)."""
    q, k, v, dy = (np.asarray(a, dtype=np.float64) for a in (q, k, v, dy))
    d = q.shape[0] // nheads
    q4, k4, v4, dy4 = (split_heads(a, nheads) for a in (q, k, v, dy))          # (d, H, L, B)
    scale = 1.0 / math.sqrt(d)
    fdrop = (lambda a: a) if keep is None else (lambda a: a * keep / (1.0 - p))
    alpha = dot_product_attention_scores(q4, k4, None if bias is None else np.asarray(bias, dtype=np.float64),
                                         mask=mask)                            # pre-dropout (Lkv, Lq, H, B)
    alpha_d = fdrop(alpha)
    # x[e,h,i,b] = Σ_j v[e,h,j,b] α'[j,i,h,b]
    dv4 = np.einsum("ehib,jihb->ehjb", dy4, alpha_d)
    dalpha_d = np.einsum("ehib,ehjb->jihb", dy4, v4)
    dalpha = dalpha_d if keep is None else dalpha_d * keep / (1.0 - p)
    dlogits = alpha * (dalpha - np.sum(dalpha * alpha, axis=0, keepdims=True))  # ∇softmax over kv
    if mask is not None:
        dlogits = np.where(np.broadcast_to(_bcast_to_scores(mask).astype(bool), dlogits.shape), dlogits, 0.0)
    dq4 = scale * np.einsum("jihb,ehjb->ehib", dlogits, k4)
    dk4 = scale * np.einsum("jihb,ehib->ehjb", dlogits, q4)
    dbias = None
    if bias is not None:
        b4 = _bcast_to_scores(bias)
        axes = tuple(ax for ax in range(4) if b4.shape[ax] == 1 and dlogits.shape[ax] != 1)
        dbias = np.sum(dlogits, axis=axes, keepdims=True).reshape(np.asarray(bias).shape)
    return join_heads(dq4), join_heads(dk4), join_heads(dv4), dbias


def attention_grad_unit(q, k, v, dy, nheads, b, h, *, causal=False, dtype=np.float64):
    """Pullback of :func:`dot_product_attention` restricted to ONE ``(b, h)`` unit, in ``dtype`` (Float64):
    the same rules as :func:`dot_product_attention_grad` (``src/batched/batchedmul.jl:96-110``,
    ``src/softmax.jl:84-110``, ``src/attention.jl:118``) on the unit's ``(Lkv, Lq)`` score matrix only, so
    that a single unit of a problem whose whole score array fits nowhere can be checked exactly.  ``q``,
    ``k``, ``v``, ``dy`` are 3-d ``(E, L, B)`` arrays; returns ``(dq (d, Lq), dk (d, Lkv), dv (dv, Lkv))``
    of that unit.  Units are independent (``batched_mul`` never mixes batch indices), so these are the
    unit's slices of the full gradient."""
    d = q.shape[0] // nheads
    dv_ = v.shape[0] // nheads
    qh = np.asarray(q[h * d:(h + 1) * d, :, b], dtype=dtype)            # (d, Lq)
    kh = np.asarray(k[h * d:(h + 1) * d, :, b], dtype=dtype)            # (d, Lkv)
    vh = np.asarray(v[h * dv_:(h + 1) * dv_, :, b], dtype=dtype)        # (dv, Lkv)
    dyh = np.asarray(dy[h * dv_:(h + 1) * dv_, :, b], dtype=dtype)      # (dv, Lq)
    scale = dtype(1.0 / math.sqrt(d))
    logits = kh.T @ (qh * scale)                                        # (Lkv, Lq)
    if causal:
        keep = np.arange(kh.shape[1])[:, None] <= np.arange(qh.shape[1])[None, :]
        logits = np.where(keep, logits, -np.inf)
    alpha = softmax(logits, dims=0)
    del logits
    dvh = dyh @ alpha.T                                                 # dv[e,j] = Σ_i dy[e,i] α[j,i]
    dalpha = vh.T @ dyh                                                 # (Lkv, Lq)
    dlogits = alpha * (dalpha - np.sum(dalpha * alpha, axis=0, keepdims=True))
    del alpha, dalpha
    dqh = scale * (kh @ dlogits)                                        # (d, Lq)
    dkh = scale * (qh @ dlogits.T)                                      # (d, Lkv)
    return dqh, dkh, dvh
