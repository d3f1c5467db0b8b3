"""Host-side mirror of NNlib.jl's attention API for column-major CUDA tensors.

Same names, argument meaning and error behaviour as the reference
(``src/attention.jl``): ``dot_product_attention(q, k, v, [bias]; fdrop, mask,
nheads)`` returns ``(x, α)``, ``dot_product_attention_scores(q, k, [bias];
fdrop, mask)`` returns ``α``, ``make_causal_mask(x; dims)`` returns a Bool
matrix.  This module is what the Julia ``CuArray`` methods in
``julia/ext/NNlibCUDAExt/attention.jl`` do, statement for statement, with
``ctypes`` in place of ``ccall``: validate, fill one params struct, call
``libnnlib_b200.so`` on the current stream.  All arithmetic happens in that
library; nothing here falls back to PyTorch ops or to the CPU.

Tensors use the reference's shapes with column-major strides (see
``layout.py``): ``q`` is ``(E, Lq, B...)``, ``α`` is ``(Lkv, Lq, H, B...)``.
"""
from __future__ import annotations

import ctypes as C
import math
import threading
import weakref
from typing import Callable, Optional

import torch

from . import _lib
from .dropout import PhiloxDropout
from .layout import is_column_major, jl_empty, jl_reshape

__all__ = [
    "ArgumentError",
    "CausalMask",
    "LazyAttnScores",
    "PhiloxDropout",
    "dot_product_attention",
    "dot_product_attention_scores",
    "dot_product_attention_pullback",
    "make_causal_mask",
    "identity",
    "device_health",
    "check_status",
    "set_math_mode",
    "math_mode",
    "set_scores_mode",
    "scores_mode",
]


# Float32 arrays: exact fp32 arithmetic by default (the reference's GPU tests hold Float32 to 1e-5); in fast
# math mode the two products run on the tensor cores with TF32 operands.  The Julia methods read
# CUDA.math_mode() == CUDA.FAST_MATH, the switch CUDA.jl gives cuBLAS for the reference's own batched_mul.
_fast_math = False


def set_math_mode(mode: str) -> None:
    """``"default"``: Float32 attention in exact fp32 on the CUDA cores.  ``"fast"``: Float32 attention on
    the tensor cores with TF32 operands (max-abs error about 3e-3 on unit-variance inputs).  16-bit element
    types are not affected."""
    global _fast_math
    if mode not in ("default", "fast"):
        raise ValueError("math mode must be 'default' or 'fast'")
    _fast_math = (mode == "fast")


def math_mode() -> str:
    return "fast" if _fast_math else "default"


# The reference returns the scores eagerly; here they are rebuilt on first use by default, so that
# ``x, _ = dot_product_attention(...)`` never pays for them.  A caller that always reads α can ask for the eager
# form: one library call produces x and α together, and for short key sequences (every query's score row in
# tensor memory: kv_len <= 512 at d = 64, <= 256 at d = 128) that is one kernel instead of two.
_eager_scores = False


def set_scores_mode(mode: str) -> None:
    """``"lazy"`` (default): α is a :class:`LazyAttnScores`.  ``"eager"``: α is computed with x and returned
    as an ordinary array, like the reference does."""
    global _eager_scores
    if mode not in ("lazy", "eager"):
        raise ValueError("scores mode must be 'lazy' or 'eager'")
    _eager_scores = (mode == "eager")


def scores_mode() -> str:
    return "eager" if _eager_scores else "lazy"


class ArgumentError(ValueError):
    """Julia's ``ArgumentError`` (thrown by ``src/attention.jl:42,55-78``)."""


class CausalMask:
    """Sentinel accepted as ``mask=``: the causal pattern ``kv <= query + offset``
    without materialising the Bool matrix.  ``offset = 0`` is what
    ``make_causal_mask`` returns (1 GiB at L = 32768); ``offset = kv_len - q_len``
    aligns the last query with the last key — new queries against a longer
    key / value history, which the reference can only express with a
    hand-built Bool mask (``make_causal_mask`` is square)."""

    def __init__(self, offset: int = 0):
        self.offset = int(offset)

    def __repr__(self):
        return "CausalMask()" if self.offset == 0 else f"CausalMask(offset={self.offset})"


def identity(x):
    return x


_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}

# id(tensor) -> (weak reference to that tensor, its version counter, L) for the Bool matrices that
# make_causal_mask built and that no PyTorch operation has written to since.  Nothing else is trusted: a
# freed matrix's address (and id) can be handed to the next one, so an entry counts only while its weak
# reference still yields the very object being asked about.
_made_causal: dict = {}
_made_causal_lock = threading.Lock()


# One int32 per device that every kernel launched through this module reports to: a launch that gave up on
# a bounded wait, and every launch skipped afterwards, writes NNLIB_B200_TIMEOUT there (see the header of
# include/nnlib_b200.h, "fail-stop behaviour").  Looked at wherever this module synchronises anyway.
_status_words: dict = {}
_status_lock = threading.Lock()


def _status_word(dev: torch.device) -> torch.Tensor:
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    with _status_lock:
        w = _status_words.get(idx)
        if w is None:
            w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
            _status_words[idx] = w
    return w


def check_status(device=None) -> None:
    """Raise :class:`NNlibB200Error` if a kernel launched through this module on ``device`` gave up on a
    bounded wait (its results, and those of every later launch on that device, are invalid).  Reads one
    int32 from the device, which waits for the work enqueued so far; the word is cleared."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    with _status_lock:
        w = _status_words.get(idx)
    if w is None:
        return
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise _lib.NNlibB200Error(v, "a kernel of an earlier call")


def _check(rc: int, where: str):
    if rc == _lib.OK:
        return
    if rc == _lib.INVALID_ARG:
        raise ArgumentError(f"{where}: {_lib.strerror(rc)}")
    raise _lib.NNlibB200Error(rc, where)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream of the current device as a raw handle (the short way when torch offers it: building
    a Stream object costs several microseconds per call, which a small problem notices)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _require_dense_cuda(name: str, t: torch.Tensor):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise TypeError(f"{name} lives on {t.device}: this method is defined for CUDA arrays only")
    if t.dtype not in _DTYPES:
        raise TypeError(f"{name} has eltype {t.dtype}; supported: Float16, BFloat16, Float32")
    if not is_column_major(t):
        raise TypeError(f"{name} is not a dense column-major array (strides {t.stride()} for size {tuple(t.shape)})")


def _bcast_strides(name: str, t: torch.Tensor, full: tuple) -> list:
    """Element strides of ``t`` against the ``(Lkv, Lq, H, B)`` scores, 0 where
    ``t`` broadcasts.  Julia broadcasting: missing trailing dims count as 1."""
    if t.ndim > 4:
        raise ArgumentError(f"{name} has {t.ndim} dimensions; scores have 4")
    out = []
    for dim in range(4):
        size = t.shape[dim] if dim < t.ndim else 1
        if size == 1:
            out.append(0)
        elif size == full[dim]:
            out.append(int(t.stride(dim)))
        else:
            raise ArgumentError(
                f"{name} of size {tuple(t.shape)} does not broadcast to scores of size {full}")
    return out


class _Problem:
    """Everything one call of the library needs, kept alive together."""

    def __init__(self, q, k, v, bias, mask, nheads, dropout: Optional[PhiloxDropout], need_v: bool,
                 rng_origin=None):
        self.dev = q.device
        self.dtype = q.dtype
        E, Lq, B = q.shape
        Lkv = k.shape[1]
        H = nheads
        self.E, self.Lq, self.B, self.Lkv, self.H = E, Lq, B, Lkv, H
        self.d = E // H
        self.q, self.k, self.v = q, k, v
        self.Ev = v.shape[0] if need_v else E
        self.dv = self.Ev // H
        p = _lib.AttnParams()
        p.dtype = _DTYPES[q.dtype]
        p.d, p.dv, p.H, p.Lq, p.Lkv, p.B = self.d, self.dv, H, Lq, Lkv, B
        p.q, p.k = q.data_ptr(), k.data_ptr()
        if need_v:
            p.v = v.data_ptr()
        full = (Lkv, Lq, H, B)
        self.keep = [q, k, v]
        if bias is not None:
            if not isinstance(bias, torch.Tensor) or not bias.is_cuda:
                raise TypeError("bias must be a CUDA tensor")
            if bias.dtype not in _DTYPES:
                bias = bias.to(torch.float32)
            st = _bcast_strides("bias", bias, full)
            p.bias = bias.data_ptr()
            p.bias_dtype = _DTYPES[bias.dtype]
            p.bias_stride = (C.c_int64 * 4)(*st)
            self.keep.append(bias)
        causal = False
        if isinstance(mask, CausalMask):
            causal = True
            p.causal_offset = mask.offset
        elif mask is not None:
            if not isinstance(mask, torch.Tensor) or not mask.is_cuda or mask.dtype != torch.bool:
                raise TypeError("mask must be a Bool CUDA tensor, a CausalMask() or None")
            if _is_causal_matrix(mask, Lq, Lkv):
                causal = True
            else:
                st = _bcast_strides("mask", mask, full)
                m8 = mask.view(torch.uint8)
                p.mask = m8.data_ptr()
                p.mask_stride = (C.c_int64 * 4)(*st)
                self.keep.append(m8)
        p.causal = 1 if causal else 0
        p.nan_on_fully_masked = 1
        p.allow_tf32 = 1 if (_fast_math and q.dtype == torch.float32) else 0
        p.scale = 0.0
        if dropout is not None and dropout.p > 0.0:
            p.dropout_p = dropout.p
            p.philox_seed = dropout.seed & 0xFFFFFFFFFFFFFFFF
            p.philox_offset = dropout.take_offset() & 0xFFFFFFFFFFFFFFFF
            if rng_origin is not None:
                # this call is a shard: (first head, first batch, heads of the whole problem)
                p.rng_h0, p.rng_b0, p.rng_H = (int(v_) for v_ in rng_origin)
        self.status_word = _status_word(self.dev)
        p.status = self.status_word.data_ptr()
        self.p = p

    def alloc_lse(self):
        self.lse = jl_empty((self.Lq, self.H, self.B), torch.float32, self.dev)
        self.p.lse = self.lse.data_ptr()
        return self.lse

    def alloc_x(self):
        self.x = jl_empty((self.Ev, self.Lq, self.B), self.dtype, self.dev)
        self.p.x = self.x.data_ptr()
        return self.x

    def alloc_alpha(self):
        a = jl_empty((self.Lkv, self.Lq, self.H, self.B), self.dtype, self.dev)
        self.p.alpha = a.data_ptr()
        return a


def _is_causal_matrix(mask: torch.Tensor, Lq: int, Lkv: int) -> bool:
    """Is ``mask`` an ``(L, L)`` Bool matrix holding exactly ``kv <= query``?  A matrix that
    :func:`make_causal_mask` returned and that has not been written to since (same object, same version
    counter) is known to; every other square Bool matrix is read on the device each time it is passed
    (one pass over it and a 4-byte copy back), so a matrix that was modified, or a new one that landed
    on a freed one's address, is never mistaken for the causal pattern."""
    if mask.ndim != 2 or Lq != Lkv or tuple(mask.shape) != (Lkv, Lq) or not is_column_major(mask):
        return False
    with _made_causal_lock:
        hit = _made_causal.get(id(mask))
    if hit is not None and hit[0]() is mask and hit[1] == mask._version and hit[2] == Lq:
        return True
    lib = _lib.load()
    flag = torch.empty(1, dtype=torch.int32, device=mask.device)
    with torch.cuda.device(mask.device):
        _check(lib.nnlib_b200_causal_check(mask.view(torch.uint8).data_ptr(), Lq, flag.data_ptr(), _stream()),
               "causal_check")
    return bool(flag.item())


def _known_causal_matrix(mask, Lq: int, Lkv: int) -> bool:
    """The part of :func:`_is_causal_matrix` that needs no device work: ``mask`` is a matrix that
    :func:`make_causal_mask` returned for this length and that has not been written to since."""
    if not isinstance(mask, torch.Tensor) or mask.ndim != 2 or Lq != Lkv or tuple(mask.shape) != (Lkv, Lq):
        return False
    with _made_causal_lock:
        hit = _made_causal.get(id(mask))
    return hit is not None and hit[0]() is mask and hit[1] == mask._version and hit[2] == Lq


class LazyAttnScores:
    """The ``α`` of ``(x, α) = dot_product_attention(...)``, materialised on
    first use.  The fused kernel keeps one log-sum-exp per query; the
    ``(Lkv, Lq, H, B...)`` array is rebuilt from it (same dropout mask) by the
    scores kernel only if somebody looks at it.  ``x, _ = ...`` never pays for
    it."""

    def __init__(self, problem: _Problem, shape: tuple):
        self._problem = problem
        self._shape = tuple(shape)
        self._value: Optional[torch.Tensor] = None

    # -- array-like surface ------------------------------------------------
    @property
    def shape(self):
        return torch.Size(self._shape)

    def size(self, dim=None):
        return self.shape if dim is None else self._shape[dim]

    @property
    def ndim(self):
        return len(self._shape)

    @property
    def dtype(self):
        return self._problem.dtype

    @property
    def device(self):
        return self._problem.dev

    @property
    def is_materialized(self) -> bool:
        return self._value is not None

    def reshape(self, *shape):
        """Column-major reshape that stays lazy (the N-d wrapper of the
        reference reshapes α, ``src/attention.jl:48``)."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list, torch.Size)):
            shape = tuple(shape[0])
        n = math.prod(self._shape)
        if math.prod(shape) != n:
            raise ValueError(f"cannot reshape scores of size {self._shape} to {shape}")
        out = LazyAttnScores(self._problem, shape)
        out._base = self
        return out

    def materialize(self) -> torch.Tensor:
        base = getattr(self, "_base", None)
        if base is not None:
            return jl_reshape(base.materialize(), self._shape)
        if self._value is None:
            pr = self._problem
            alpha = pr.alloc_alpha()
            if pr.Lkv > 0 and pr.Lq > 0 and pr.B > 0:
                with torch.cuda.device(pr.dev):
                    _check(_lib.load().nnlib_b200_attn_scores(C.byref(pr.p), _stream()), "attn_scores")
            self._value = jl_reshape(alpha, self._shape)
        return self._value

    def __array__(self, dtype=None):
        t = self.materialize()
        if t.dtype in (torch.bfloat16, torch.float16):
            t = t.float()
        a = t.cpu().numpy()
        check_status(self._problem.dev)      # the copy synchronised anyway
        return a if dtype is None else a.astype(dtype)

    def __getitem__(self, idx):
        return self.materialize()[idx]

    def __getattr__(self, name):
        # anything else (sum, float, cpu, ...) acts on the materialised tensor
        if name.startswith("_"):
            raise AttributeError(name)
        return getattr(self.materialize(), name)

    def __repr__(self):
        state = "materialized" if self.is_materialized else "lazy"
        return f"LazyAttnScores(size={self._shape}, dtype={self.dtype}, {state})"


def _validate_3d(q, k, v, nheads):
    """The four checks of ``src/attention.jl:55-78``, same order and wording."""
    if any(t.shape[0] % nheads != 0 for t in (q, k, v)):
        raise ArgumentError(
            "First dimension in query, key and value must be divisible by `nheads`.\n"
            f"Instead:\n- size(q): {tuple(q.shape)}\n- size(k): {tuple(k.shape)}\n"
            f"- size(v): {tuple(v.shape)}\n- nheads: {nheads}")
    if not (q.shape[2] == k.shape[2] == v.shape[2]):
        raise ArgumentError(
            "Batch dimensions have to be the same. Instead:\n"
            f"- size(q): {tuple(q.shape)}\n- size(k): {tuple(k.shape)}\n- size(v): {tuple(v.shape)}")
    if q.shape[0] != k.shape[0]:
        raise ArgumentError(
            "First dimension in query and key has to be the same. Instead:\n"
            f"- size(q): {tuple(q.shape)}\n- size(k): {tuple(k.shape)}")
    if k.shape[1] != v.shape[1]:
        raise ArgumentError(
            "Second dimension in key and value has to be the same. Instead:\n"
            f"- size(k): {tuple(k.shape)}\n- size(v): {tuple(v.shape)}")


def dot_product_attention(q, k, v, bias=None, *, fdrop: Callable = identity, mask=None, nheads: int = 1):
    """Multi-head dot-product attention (``src/attention.jl:40-84``).

    ``q``: ``(qk_dim, q_len, batch...)``, ``k``: ``(qk_dim, kv_len, batch...)``,
    ``v``: ``(v_dim, kv_len, batch...)``, column-major CUDA tensors of one
    element type.  Returns ``(x, α)`` with ``x``: ``(v_dim, q_len, batch...)``
    and ``α``: ``(kv_len, q_len, nheads, batch...)`` — the scores *after*
    ``fdrop``, from which ``x`` was computed.

    ``fdrop``: ``identity`` or a :class:`PhiloxDropout` run fused (α is then a
    :class:`LazyAttnScores`); any other callable gets the materialised scores,
    and ``x`` is computed from what it returns.  ``mask``: Bool tensor
    broadcastable to the scores (true = attend), the result of
    :func:`make_causal_mask`, or ``CausalMask()``.
    """
    for name, t in (("query", q), ("key", k), ("value", v)):
        _require_dense_cuda(name, t)
    if not (q.ndim == k.ndim == v.ndim):
        raise TypeError("query, key and value must have the same number of dimensions")
    if q.ndim < 2:
        raise TypeError("query, key and value need at least (features, length) dimensions")
    if not (q.dtype == k.dtype == v.dtype):
        raise TypeError("query, key and value must share one element type")
    batch_size = tuple(q.shape[2:])
    if q.ndim != 3:
        # N-d wrapper, src/attention.jl:40-50: flatten the batch dims, restore them on both outputs.
        if not (batch_size == tuple(k.shape[2:]) == tuple(v.shape[2:])):
            raise ArgumentError("Batch dimensions have to be the same.")
        q, k, v = (jl_reshape(t, (t.shape[0], t.shape[1], -1)) for t in (q, k, v))
    nheads = int(nheads)
    _validate_3d(q, k, v, nheads)

    if fdrop is None or fdrop is identity:
        x, alpha = _fused(q, k, v, bias, mask, nheads, None)
    elif isinstance(fdrop, PhiloxDropout):
        x, alpha = _fused(q, k, v, bias, mask, nheads, fdrop)
    else:
        x, alpha = _unfused(q, k, v, bias, mask, nheads, fdrop)

    if len(batch_size) != 1:
        x = jl_reshape(x, tuple(x.shape[:2]) + batch_size)
        alpha = alpha.reshape(tuple(alpha.shape[:3]) + batch_size) if isinstance(alpha, LazyAttnScores) \
            else jl_reshape(alpha, tuple(alpha.shape[:3]) + batch_size)
    return x, alpha


def _fused(q, k, v, bias, mask, nheads, dropout):
    pr = _Problem(q, k, v, bias, mask, nheads, dropout, need_v=True)
    x = pr.alloc_x()
    pr.alloc_lse()
    if _eager_scores:
        alpha = pr.alloc_alpha()
        if pr.Lq > 0 and pr.B > 0 and pr.Lkv > 0:
            with torch.cuda.device(pr.dev):
                _check(_lib.load().nnlib_b200_attention(C.byref(pr.p), None, 0, _stream()), "attention")
        return x, alpha
    if pr.Lq > 0 and pr.B > 0:
        lib = _lib.load()
        with torch.cuda.device(pr.dev):
            # few queries against many keys: the library splits the keys of a unit over several CTAs when that
            # pays and tells how much scratch memory the partial results need (0: the ordinary forward)
            need = lib.nnlib_b200_attn_decode_workspace_bytes(C.byref(pr.p)) if pr.Lq <= 128 else 0
            if need:
                ws = torch.empty(need, dtype=torch.uint8, device=pr.dev)
                _check(lib.nnlib_b200_attn_decode(C.byref(pr.p), ws.data_ptr(), need, _stream()), "attn_decode")
            else:
                _check(lib.nnlib_b200_attn_fwd(C.byref(pr.p), _stream()), "attn_fwd")
    return x, LazyAttnScores(pr, (pr.Lkv, pr.Lq, pr.H, pr.B))


def _fused_into(q, k, v, mask, nheads, x_out, lse_out):
    """The fused call writing into caller-owned buffers (no allocation): ``x_out`` is a column-major
    ``(Ev, Lq, B)`` array of the inputs' element type, ``lse_out`` a Float32 array of ``Lq*H*B`` elements."""
    pr = _Problem(q, k, v, None, mask, nheads, None, need_v=True)
    if tuple(x_out.shape) != (pr.Ev, pr.Lq, pr.B) or x_out.dtype != pr.dtype or not is_column_major(x_out):
        raise ArgumentError("x_out must be a dense column-major (Ev, Lq, B) array of the inputs' element type")
    if lse_out.dtype != torch.float32 or lse_out.numel() < pr.Lq * pr.H * pr.B or not lse_out.is_contiguous():
        raise ArgumentError("lse_out must be a contiguous Float32 array of at least Lq*H*B elements")
    pr.x = x_out
    pr.p.x = x_out.data_ptr()
    pr.lse = lse_out
    pr.p.lse = lse_out.data_ptr()
    if pr.Lq > 0 and pr.B > 0:
        with torch.cuda.device(pr.dev):
            _check(_lib.load().nnlib_b200_attn_fwd(C.byref(pr.p), _stream()), "attn_fwd")
    return x_out


def _fused_with_origin(q, k, v, bias, mask, nheads, dropout, rng_origin):
    """The fused call for a shard of a larger problem (see ``shard.py``):
    ``rng_origin`` places the shard's heads and batches in the whole problem so
    that dropout draws the whole problem's mask.  Returns x only."""
    pr = _Problem(q, k, v, bias, mask, nheads, dropout, need_v=True, rng_origin=rng_origin)
    x = pr.alloc_x()
    pr.alloc_lse()
    if pr.Lq > 0 and pr.B > 0:
        with torch.cuda.device(pr.dev):
            _check(_lib.load().nnlib_b200_attn_fwd(C.byref(pr.p), _stream()), "attn_fwd")
    return x


def dot_product_attention_pullback(q, k, v, bias=None, *, fdrop: Callable = identity, mask=None, nheads: int = 1):
    """``rrule``-style forward: returns ``(x, α, back)`` where ``back(dx)`` gives ``(dq, dk, dv, dbias)``,
    the cotangents Zygote would compose from the reference's rules for ``batched_mul``, ``softmax`` and
    ``dropout`` on this path (``src/batched/batchedmul.jl:96-110``, ``src/softmax.jl:84-116``,
    ``src/dropout.jl:106-122``).  3-d inputs; ``fdrop`` must be ``identity`` or a :class:`PhiloxDropout`
    (the pullback replays its mask).  ``dbias`` has the shape and element type of ``bias`` (None without)."""
    for name, t in (("query", q), ("key", k), ("value", v)):
        _require_dense_cuda(name, t)
    if not (q.ndim == k.ndim == v.ndim == 3):
        raise TypeError("the pullback is defined for 3-d (features, length, batch) arrays")
    nheads = int(nheads)
    _validate_3d(q, k, v, nheads)
    if not (fdrop is None or fdrop is identity or isinstance(fdrop, PhiloxDropout)):
        raise ArgumentError("pullback: fdrop must be identity or a PhiloxDropout")
    dropout = fdrop if isinstance(fdrop, PhiloxDropout) else None
    pr = _Problem(q, k, v, bias, mask, nheads, dropout, need_v=True)
    x = pr.alloc_x()
    pr.alloc_lse()
    lib = _lib.load()
    if pr.Lq > 0 and pr.B > 0:
        with torch.cuda.device(pr.dev):
            _check(lib.nnlib_b200_attn_fwd(C.byref(pr.p), _stream()), "attn_fwd")
    alpha = LazyAttnScores(pr, (pr.Lkv, pr.Lq, pr.H, pr.B))

    def back(dx: torch.Tensor):
        _require_dense_cuda("dx", dx)
        if tuple(dx.shape) != tuple(x.shape) or dx.dtype != x.dtype:
            raise ArgumentError(f"dx must have size {tuple(x.shape)} and eltype {x.dtype}")
        dq = jl_empty(q.shape, q.dtype, pr.dev)
        dk = jl_empty(k.shape, k.dtype, pr.dev)
        dv = jl_empty(v.shape, v.dtype, pr.dev)
        delta = torch.empty(pr.Lq * pr.H * pr.B, dtype=torch.float32, device=pr.dev)
        g = _lib.AttnGrads()
        g.dx, g.dq, g.dk, g.dv, g.delta = dx.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr()
        dbias32 = None
        if bias is not None:
            dbias32 = torch.zeros(tuple(bias.shape)[::-1], dtype=torch.float32, device=pr.dev)
            dbias32 = dbias32.permute(*range(bias.ndim - 1, -1, -1)) if bias.ndim else dbias32
            g.dbias = dbias32.data_ptr()
            g.dbias_stride = (C.c_int64 * 4)(*_bcast_strides("bias", dbias32, (pr.Lkv, pr.Lq, pr.H, pr.B)))
        back.path = lib.nnlib_b200_attn_bwd_path(C.byref(pr.p), C.byref(g))   # PATH_UMMA / PATH_SIMT, for tests
        with torch.cuda.device(pr.dev):
            _check(lib.nnlib_b200_attn_bwd(C.byref(pr.p), C.byref(g), _stream()), "attn_bwd")
        return dq, dk, dv, (None if dbias32 is None else dbias32.to(bias.dtype))

    return x, alpha, back


def _unfused(q, k, v, bias, mask, nheads, fdrop):
    """``fdrop`` is an opaque callable: materialise α, let the caller's
    function transform it, then x = V·α′ (``src/attention.jl:91-98``)."""
    pr = _Problem(q, k, v, bias, mask, nheads, None, need_v=True)
    lib = _lib.load()
    x = pr.alloc_x()
    pr.alloc_lse()
    alpha = pr.alloc_alpha()
    with torch.cuda.device(pr.dev):
        if pr.Lq > 0 and pr.B > 0:
            _check(lib.nnlib_b200_attn_stats(C.byref(pr.p), _stream()), "attn_stats")
            _check(lib.nnlib_b200_attn_scores(C.byref(pr.p), _stream()), "attn_scores")
        alpha2 = fdrop(alpha)
        if not isinstance(alpha2, torch.Tensor) or tuple(alpha2.shape) != tuple(alpha.shape):
            raise ArgumentError("fdrop must return an array of the scores' size")
        if alpha2.dtype != pr.dtype or not is_column_major(alpha2) or alpha2.device != pr.dev:
            fixed = jl_empty(alpha.shape, pr.dtype, pr.dev)
            fixed.copy_(alpha2)
            alpha2 = fixed
        pr.p.alpha = alpha2.data_ptr()
        if pr.Lq > 0 and pr.B > 0:
            _check(lib.nnlib_b200_attn_apply(C.byref(pr.p), _stream()), "attn_apply")
    return x, alpha2


def dot_product_attention_scores(q, k, bias=None, *, fdrop: Callable = identity, mask=None):
    """Attention scores only (``src/attention.jl:112-127``).  ``q``:
    ``(d, nheads, q_len, batch)``, ``k``: ``(d, nheads, kv_len, batch)`` of one
    element type → ``α``: ``(kv_len, q_len, nheads, batch)``."""
    for name, t in (("query", q), ("key", k)):
        _require_dense_cuda(name, t)
    if q.ndim != 4 or k.ndim != 4:
        raise TypeError("dot_product_attention_scores expects 4-d (d, nheads, len, batch) arrays")
    if q.dtype != k.dtype:
        raise TypeError("query and key must share one element type")
    d, H, Lq, B = q.shape
    if tuple(k.shape[:2]) != (d, H) or k.shape[3] != B:
        raise ArgumentError(f"query of size {tuple(q.shape)} and key of size {tuple(k.shape)} do not match")
    q3 = jl_reshape(q, (d * H, Lq, B))
    k3 = jl_reshape(k, (d * H, k.shape[2], B))
    dropout = fdrop if isinstance(fdrop, PhiloxDropout) else None
    pr = _Problem(q3, k3, k3, bias, mask, H, dropout, need_v=False)
    pr.alloc_lse()
    alpha = pr.alloc_alpha()
    if pr.Lq > 0 and pr.B > 0 and pr.Lkv > 0:
        lib = _lib.load()
        with torch.cuda.device(pr.dev):
            _check(lib.nnlib_b200_attn_stats(C.byref(pr.p), _stream()), "attn_stats")
            _check(lib.nnlib_b200_attn_scores(C.byref(pr.p), _stream()), "attn_scores")
    if dropout is None and fdrop is not None and fdrop is not identity:
        alpha = fdrop(alpha)
    return alpha


def make_causal_mask(x: torch.Tensor, dims: int = 2) -> torch.Tensor:
    """Bool square matrix ``m`` of side ``size(x, dims)`` with ``m[i, j] = i <= j``
    (``src/attention.jl:149-153``; ``dims`` is 1-based like the reference's),
    on the device of ``x``.  Passing it (unmodified) as ``mask=`` selects the
    kernels' causal mode without reading the matrix; once it has been written
    to it is treated like any other Bool mask."""
    if not isinstance(x, torch.Tensor) or not x.is_cuda:
        raise TypeError("make_causal_mask: this method is defined for CUDA arrays only")
    n = int(x.shape[dims - 1])
    m = jl_empty((n, n), torch.bool, x.device)
    with torch.cuda.device(x.device):
        _check(_lib.load().nnlib_b200_causal_fill(m.view(torch.uint8).data_ptr(), n, _stream()), "causal_fill")
    key = id(m)
    with _made_causal_lock:
        _made_causal[key] = (weakref.ref(m), m._version, n)
    weakref.finalize(m, _forget_causal, key)
    return m


def _forget_causal(key):
    with _made_causal_lock:
        hit = _made_causal.get(key)
        if hit is not None and hit[0]() is None:
            del _made_causal[key]


def device_health(device=None) -> None:
    """Synchronise and raise if a kernel of the library gave up on a bounded
    wait since the last call (``nnlib_b200_device_health``)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        rc = _lib.load().nnlib_b200_device_health(_stream())
    try:
        check_status(dev)
    finally:
        if rc != _lib.OK:
            raise _lib.NNlibB200Error(rc, "device_health")
