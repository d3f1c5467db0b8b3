"""Multi-GPU driver: the (batch, head) units of one attention call spread over
the GPUs of a box.

Every (batch, head) pair of ``dot_product_attention`` is an independent
problem (NNlib.jl src/attention.jl:87-99: the batched products never mix the
trailing dimensions), so the path shards with NO collective: the units are
split into contiguous, balanced ranges, one per device; each device gets its
slices of q/k/v (and of bias/mask where those are not broadcast), runs the
ordinary single-GPU call on its own stream in its own host thread, and writes
its slice of x.  Dropout masks depend only on the global (head, batch)
position, so a sharded call draws the same mask as an unsharded one.

``partition_units`` / ``rank_rects`` are pure host logic and are also what a
one-process-per-GPU launch (torchrun) uses to pick each rank's share.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from .layout import jl_empty

__all__ = ["Rect", "partition_units", "rank_rects", "ShardResult", "ShardError", "ShardedAttention"]


@dataclass(frozen=True)
class Rect:
    """Batches [b0, b0+nb) x heads [h0, h0+nh)."""
    b0: int
    nb: int
    h0: int
    nh: int

    @property
    def units(self) -> int:
        return self.nb * self.nh


def _range_to_rects(u0: int, u1: int, H: int) -> List[Rect]:
    """Unit range [u0, u1) (unit u = b*H + h, batch-major) as rectangles: a
    leading partial batch, whole batches, a trailing partial batch."""
    rects = []
    u = u0
    while u < u1:
        b, h = divmod(u, H)
        if h == 0 and u1 - u >= H:
            nb = (u1 - u) // H
            rects.append(Rect(b, nb, 0, H))
            u += nb * H
        else:
            nh = min(H - h, u1 - u)
            rects.append(Rect(b, 1, h, nh))
            u += nh
    return rects


def partition_units(B: int, H: int, n: int) -> List[List[Rect]]:
    """Split the B*H units into ``n`` contiguous ranges whose sizes differ by at
    most one unit.  When ``n`` divides ``B`` every share is a batch slice."""
    if n < 1:
        raise ValueError("need at least one shard")
    total = B * H
    base, extra = divmod(total, n)
    out, u = [], 0
    for r in range(n):
        cnt = base + (1 if r < extra else 0)
        out.append(_range_to_rects(u, u + cnt, H))
        u += cnt
    return out


def rank_rects(B: int, H: int, rank: int, world: int) -> List[Rect]:
    """The share of ``rank`` in a ``world``-process launch."""
    return partition_units(B, H, world)[rank]


@dataclass
class ShardResult:
    device: str
    rects: List[Rect] = field(default_factory=list)
    ok: bool = False
    error: Optional[BaseException] = None


class ShardError(RuntimeError):
    """Some shards failed.  ``results`` has one entry per device; the slices of
    ``x`` owned by shards with ``ok=True`` hold valid output."""

    def __init__(self, results: Sequence[ShardResult], x):
        self.results = list(results)
        self.x = x
        bad = [f"{r.device}: {type(r.error).__name__}: {r.error}" for r in results if not r.ok]
        super().__init__("attention shards failed: " + "; ".join(bad))


def _slice_bcast(t: Optional[torch.Tensor], rect: Rect, H: int, B: int):
    """bias / mask restricted to a rectangle: dims of size H / B are sliced,
    broadcast (size-1 or absent) dims are passed through."""
    if t is None or not isinstance(t, torch.Tensor):
        return t
    idx = [slice(None)] * t.ndim
    if t.ndim > 2 and t.shape[2] == H and H != 1:
        idx[2] = slice(rect.h0, rect.h0 + rect.nh)
    if t.ndim > 3 and t.shape[3] == B and B != 1:
        idx[3] = slice(rect.b0, rect.b0 + rect.nb)
    return t[tuple(idx)]


def _cuda_compute(dev, q, k, v, bias, mask, nheads, dropout, rng_origin):
    """Default per-rectangle computation: the single-GPU library call."""
    from . import attention as A
    with torch.cuda.device(dev):
        return A._fused_with_origin(q, k, v, bias, mask, nheads, dropout, rng_origin)


class ShardedAttention:
    """``dot_product_attention`` over several devices of one box.

    ``devices``: torch device strings (default: every visible GPU).  Inputs may
    live on the host (pinned memory makes the copies asynchronous) or on any
    device; ``x`` is returned on ``out_device`` (default: host).  One host thread
    per device; a failing shard does not disturb the others — after all threads
    have joined, :class:`ShardError` reports per-device status.

    ``compute`` replaces the per-rectangle GPU call (tests inject host-side
    failures and CPU stand-ins through it).  ``out=`` in the call gives the
    ``(Ev, Lq, B)`` array the shards write into (a caller that calls repeatedly
    keeps one pinned array instead of paying for a new one each time).
    """

    def __init__(self, devices: Optional[Sequence[str]] = None, compute: Optional[Callable] = None,
                 out_device: str = "cpu"):
        if devices is None:
            devices = [f"cuda:{i}" for i in range(torch.cuda.device_count())]
        if not devices:
            raise ValueError("ShardedAttention needs at least one device")
        self.devices = [str(d) for d in devices]
        self.compute = compute or _cuda_compute
        self.out_device = out_device
        self._pipes = {}      # per-device pipelines for shards whose arrays cross the bus (see _pipelined)

    def _pipelined(self, slot, dev, rect, q, k, v, x, bias, mask, dropout, H) -> bool:
        """A rectangle of whole batch elements whose inputs and output sit in pinned host memory goes through
        a per-device :class:`HostPipelinedAttention` (one batch element at a time, so that the copy of the
        next element, the kernels of this one and the copy back of the previous one overlap).  Returns False
        when the rectangle does not qualify (a head range, bias, dropout, a mask array, device-resident or pageable arrays, an injected ``compute``) — the caller then takes the plain route."""
        from .attention import CausalMask
        from .hostio import HostPipelinedAttention
        if self.compute is not _cuda_compute or not str(dev).startswith("cuda"):
            return False
        if rect.h0 != 0 or rect.nh != H or bias is not None or dropout is not None or rect.nb < 2:
            return False
        if not (mask is None or isinstance(mask, CausalMask)):
            return False                                       # mask arrays take the plain route
        hosts = [t.permute(2, 1, 0) for t in (q, k, v, x)]      # (B, L, E) views of the column-major arrays
        if any(t.is_cuda or not t.is_contiguous() or not t.is_pinned() for t in hosts):
            return False
        E, Lq, _ = q.shape
        Ev, Lkv = v.shape[0], k.shape[1]
        # one pipeline per worker thread (`slot`): two shards may share a device, never staging buffers
        key = (slot, str(dev), E, Ev, Lq, Lkv, rect.nb, q.dtype, H, repr(mask))
        pipe = self._pipes.get(key)
        if pipe is None:
            pipe = HostPipelinedAttention(E, Ev, Lq, Lkv, rect.nb, q.dtype, nheads=H, mask=mask, chunk=1, device=dev)
            self._pipes[key] = pipe
        bs = slice(rect.b0, rect.b0 + rect.nb)
        with torch.cuda.device(dev):
            pipe(hosts[0][bs], hosts[1][bs], hosts[2][bs], hosts[3][bs])
        return True

    def __call__(self, q, k, v, bias=None, *, fdrop=None, mask=None, nheads: int = 1, out=None):
        from .attention import ArgumentError, PhiloxDropout, _validate_3d, identity
        if q.ndim != 3:
            raise ArgumentError("ShardedAttention takes 3-d (features, length, batch) arrays")
        _validate_3d(q, k, v, nheads)
        if fdrop is not None and fdrop is not identity and not isinstance(fdrop, PhiloxDropout):
            raise ArgumentError("sharded attention runs fused: fdrop must be identity or a PhiloxDropout")
        dropout = None
        if isinstance(fdrop, PhiloxDropout) and fdrop.p > 0:
            # one offset for the whole call so that every shard draws from the same mask
            dropout = PhiloxDropout(fdrop.p, fdrop.seed, fdrop.take_offset())
        E, Lq, B = q.shape
        Ev = v.shape[0]
        H = nheads
        d, dv = E // H, Ev // H
        if out is not None:
            if tuple(out.shape) != (Ev, Lq, B) or out.dtype != q.dtype:
                raise ArgumentError(f"out must have size {(Ev, Lq, B)} and eltype {q.dtype}")
            x = out
        elif self.out_device == "cpu" and torch.cuda.is_available():
            # pinned from the start (no pageable detour): the shards' device-to-host copies are asynchronous
            x = torch.empty((B, Lq, Ev), dtype=q.dtype, pin_memory=True).permute(2, 1, 0)
        else:
            x = jl_empty((Ev, Lq, B), q.dtype, self.out_device)
        plan = partition_units(B, H, len(self.devices))
        results = [ShardResult(dev, rects) for dev, rects in zip(self.devices, plan)]

        def work(res: ShardResult):
            try:
                for rect in res.rects:
                    bs = slice(rect.b0, rect.b0 + rect.nb)
                    if self._pipelined(results.index(res), res.device, rect, q, k, v, x, bias, mask, dropout, H):
                        continue
                    qs = q[rect.h0 * d:(rect.h0 + rect.nh) * d, :, bs]
                    ks = k[rect.h0 * d:(rect.h0 + rect.nh) * d, :, bs]
                    vs = v[rect.h0 * dv:(rect.h0 + rect.nh) * dv, :, bs]
                    dev = res.device
                    on_dev = []
                    for t in (qs, ks, vs):
                        dt = jl_empty(t.shape, t.dtype, dev)
                        dt.copy_(t, non_blocking=True)
                        on_dev.append(dt)
                    bias_d = _slice_bcast(bias, rect, H, B)
                    mask_d = _slice_bcast(mask, rect, H, B)
                    if isinstance(bias_d, torch.Tensor):
                        bias_d = bias_d.to(dev, non_blocking=True)
                    if isinstance(mask_d, torch.Tensor):
                        mask_d = mask_d.to(dev, non_blocking=True)
                    drop = None if dropout is None else PhiloxDropout(dropout.p, dropout.seed, dropout.offset)
                    y = self.compute(dev, *on_dev, bias_d, mask_d, rect.nh, drop, (rect.h0, rect.b0, H))
                    x[rect.h0 * dv:(rect.h0 + rect.nh) * dv, :, bs].copy_(y, non_blocking=True)
                if str(res.device).startswith("cuda"):
                    torch.cuda.synchronize(res.device)
                    from .attention import check_status
                    check_status(res.device)      # a kernel that gave up fails this shard, not the others
                res.ok = True
            except BaseException as e:  # reported per shard, never swallowed
                res.error = e

        threads = [threading.Thread(target=work, args=(r,), name=f"attn-shard-{r.device}") for r in results]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if not all(r.ok for r in results):
            raise ShardError(results, x)
        self.last_results = results
        return x
