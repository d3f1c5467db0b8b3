"""Attention on arrays that live in host memory.

The reference's method takes arrays wherever they are; a caller whose q, k, v
sit in (pinned) host memory pays two PCIe crossings around the kernels.  The
(batch, head) units are independent (NNlib.jl ``src/attention.jl:87-99``), so
the batch can be cut into chunks and the three engines of the GPU kept busy at
once: while chunk ``i`` is in the kernels, chunk ``i+1`` crosses the bus on the
host-to-device copy engine and the result of chunk ``i-1`` returns on the
device-to-host engine.  The bus is full duplex, so the step costs about
``max(bytes_in, bytes_out) / bandwidth`` instead of their sum plus the kernels.
"""
from __future__ import annotations

import torch

from .attention import ArgumentError, CausalMask, _fused_into, _known_causal_matrix, check_status
from .layout import jl_empty

__all__ = ["HostPipelinedAttention"]


class HostPipelinedAttention:
    """Reusable pipeline for ``x = dot_product_attention(q, k, v; mask, nheads)[1]`` with q, k, v and x in
    pinned host memory.

    Host arrays are torch tensors of shape ``(B, L, E)`` (row-major: the memory
    of Julia's column-major ``(E, L, B)``).  ``mask`` is ``None``,
    ``CausalMask()`` or a Bool device array shared by all batch elements (such
    as the result of ``make_causal_mask``).  Device staging buffers for two chunks (inputs, output, log-sum-exp) are allocated once
    in the constructor; :meth:`__call__` enqueues the whole pipeline and returns
    after the last result byte has been ordered on ``out_stream`` (call
    ``synchronize()`` or wait on :attr:`done` to read ``hx``).

    What is left exposed at the end of the step is the last kernel and the last copy back, so the queries of
    the last batch element are taken in ``tail_split`` ranges (a range of queries is a contiguous block of q
    and of x, and needs nothing but its own rows of q beside the element's k and v): its kernels and copies
    back run while the rest of its q is still arriving, and only a ``tail_split``-th of a result follows the
    last input byte.
    """

    def __init__(self, E: int, Ev: int, Lq: int, Lkv: int, B: int, dtype: torch.dtype, *, nheads: int,
                 mask=None, chunk: int = 1, device=None, tail_split: int = 4):
        if mask is not None and not isinstance(mask, CausalMask):
            # a Bool array on the device that does not depend on the batch (what make_causal_mask returns, or
            # any (Lkv, Lq[, H]) mask): every chunk uses it as it is
            if not (isinstance(mask, torch.Tensor) and mask.dtype == torch.bool and mask.is_cuda
                    and (mask.ndim <= 3 or mask.shape[3] == 1)):
                raise ArgumentError("HostPipelinedAttention: mask must be None, CausalMask() or a Bool CUDA array "
                                    "that is the same for every batch element")
        if chunk < 1 or B < 1:
            raise ArgumentError("HostPipelinedAttention: batch and chunk must be positive")
        self.dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.E, self.Ev, self.Lq, self.Lkv, self.B = int(E), int(Ev), int(Lq), int(Lkv), int(B)
        self.dtype, self.nheads, self.mask = dtype, int(nheads), mask
        self.chunk = min(int(chunk), self.B)
        self.tail_split = max(1, min(int(tail_split), self.Lq // 256)) if self.Lq >= 512 else 1
        c = self.chunk
        # two staging sets: one is being filled while the other is in the kernels
        self.dq = [jl_empty((E, Lq, c), dtype, self.dev) for _ in range(2)]
        self.dk = [jl_empty((E, Lkv, c), dtype, self.dev) for _ in range(2)]
        self.dv = [jl_empty((Ev, Lkv, c), dtype, self.dev) for _ in range(2)]
        self.dx = [jl_empty((Ev, Lq, c), dtype, self.dev) for _ in range(2)]
        self.lse = [torch.empty(Lq * self.nheads * c, dtype=torch.float32, device=self.dev) for _ in range(2)]
        with torch.cuda.device(self.dev):
            self.in_stream = torch.cuda.Stream()
            self.out_stream = torch.cuda.Stream()
            self.loaded = [torch.cuda.Event() for _ in range(2)]      # staging set s holds its chunk
            self.computed = [torch.cuda.Event() for _ in range(2)]    # x of staging set s is ready
            self.drained = [torch.cuda.Event() for _ in range(2)]     # x of staging set s has left the device
            self.consumed = [torch.cuda.Event() for _ in range(2)]    # the kernels no longer read staging set s
            self.done = torch.cuda.Event()
            self.piece_loaded = [torch.cuda.Event() for _ in range(self.tail_split)]
            self.piece_computed = [torch.cuda.Event() for _ in range(self.tail_split)]

    @staticmethod
    def _check_host(name, t, shape, dtype):
        if not isinstance(t, torch.Tensor) or t.is_cuda or tuple(t.shape) != tuple(shape) or t.dtype != dtype \
                or not t.is_contiguous():
            raise ArgumentError(f"{name} must be a contiguous host tensor of shape {tuple(shape)} and dtype {dtype}")
        if not t.is_pinned():
            raise ArgumentError(f"{name} must live in pinned host memory (the copies are asynchronous)")

    def __call__(self, hq: torch.Tensor, hk: torch.Tensor, hv: torch.Tensor, hx: torch.Tensor) -> torch.Tensor:
        B, c = self.B, self.chunk
        self._check_host("q", hq, (B, self.Lq, self.E), self.dtype)
        self._check_host("k", hk, (B, self.Lkv, self.E), self.dtype)
        self._check_host("v", hv, (B, self.Lkv, self.Ev), self.dtype)
        self._check_host("x", hx, (B, self.Lq, self.Ev), self.dtype)
        with torch.cuda.device(self.dev):
            comp = torch.cuda.current_stream()
            start = torch.cuda.Event()
            start.record(comp)
            self.in_stream.wait_event(start)       # the pipeline starts after earlier work of the caller's stream
            self.out_stream.wait_event(start)
            n = (B + c - 1) // c
            for i in range(n):
                s = i & 1
                b0, b1 = i * c, min(B, (i + 1) * c)
                w = b1 - b0
                tail = (i == n - 1) and self.tail_split > 1
                # ---- host -> device (copy engine 1)
                if i >= 2:
                    self.in_stream.wait_event(self.consumed[s])       # chunk i-2 no longer needs this set
                with torch.cuda.stream(self.in_stream):
                    self.dk[s].permute(2, 1, 0)[:w].copy_(hk[b0:b1], non_blocking=True)
                    self.dv[s].permute(2, 1, 0)[:w].copy_(hv[b0:b1], non_blocking=True)
                    if not tail:
                        self.dq[s].permute(2, 1, 0)[:w].copy_(hq[b0:b1], non_blocking=True)
                    elif w > 1:
                        self.dq[s].permute(2, 1, 0)[:w - 1].copy_(hq[b0:b1 - 1], non_blocking=True)
                    self.loaded[s].record(self.in_stream)
                # ---- kernels (caller's stream)
                comp.wait_event(self.loaded[s])
                if i >= 2:
                    comp.wait_event(self.drained[s])                  # x of chunk i-2 has been copied out
                q, k, v, x = self.dq[s], self.dk[s], self.dv[s], self.dx[s]
                wf = w - 1 if tail else w                              # batch elements handled whole
                if wf > 0:
                    qf, kf, vf, xf = (q, k, v, x) if wf == c else (q[:, :, :wf], k[:, :, :wf], v[:, :, :wf], x[:, :, :wf])
                    _fused_into(qf, kf, vf, self.mask, self.nheads, xf, self.lse[s])
                    self.computed[s].record(comp)
                    self.out_stream.wait_event(self.computed[s])
                    with torch.cuda.stream(self.out_stream):
                        hx[b0:b0 + wf].copy_(xf.permute(2, 1, 0), non_blocking=True)
                if tail:
                    # the last batch element, one range of queries after the other
                    e = w - 1
                    causal_matrix = _known_causal_matrix(self.mask, self.Lq, self.Lkv)
                    step = -(-self.Lq // self.tail_split)
                    lse_off = wf * self.Lq * self.nheads
                    for pz in range(self.tail_split):
                        l0, l1 = pz * step, min(self.Lq, (pz + 1) * step)
                        if l0 >= l1:
                            break
                        with torch.cuda.stream(self.in_stream):
                            q.permute(2, 1, 0)[e, l0:l1].copy_(hq[b1 - 1, l0:l1], non_blocking=True)
                            self.piece_loaded[pz].record(self.in_stream)
                        comp.wait_event(self.piece_loaded[pz])
                        if self.mask is None:
                            m = None
                        elif isinstance(self.mask, CausalMask):
                            m = CausalMask(self.mask.offset + l0)
                        elif causal_matrix:
                            m = CausalMask(l0)             # the same pattern for queries l0 .. l1 - 1, nothing to read
                        else:
                            m = self.mask[:, l0:l1]
                        _fused_into(q[:, l0:l1, e:e + 1], k[:, :, e:e + 1], v[:, :, e:e + 1], m, self.nheads,
                                    x[:, l0:l1, e:e + 1], self.lse[s][lse_off + l0 * self.nheads:])
                        self.piece_computed[pz].record(comp)
                        self.out_stream.wait_event(self.piece_computed[pz])
                        with torch.cuda.stream(self.out_stream):
                            hx[b1 - 1, l0:l1].copy_(x.permute(2, 1, 0)[e, l0:l1], non_blocking=True)
                self.consumed[s].record(comp)
                with torch.cuda.stream(self.out_stream):
                    self.drained[s].record(self.out_stream)
            self.done.record(self.out_stream)
            comp.wait_event(self.done)             # later work on the caller's stream sees hx complete
        return hx

    def synchronize(self) -> None:
        """Wait for the last call's results; raises if one of its kernels gave up on a bounded wait."""
        self.done.synchronize()
        check_status(self.dev)
