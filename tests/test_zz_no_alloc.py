"""``nnlib_b200_attention_static`` — the entry point for callers that cannot
allocate device memory at the call site (the device is owned by a memory pool,
the host language's allocator must not run there, or the caller only holds
input/output pointers).  It keeps the per-query log-sum-exp in a fixed array
inside the library instead of a caller-supplied workspace.

Checked here, through the C ABI: on two calls in a row (different problems, the
second smaller, so stale contents of the shared array would show) its x and
alpha equal those of ``nnlib_b200_attention`` with a caller workspace; and a
problem with more than ``NNLIB_B200_STATIC_MAX_QUERIES`` queries is refused.
This file sorts last on purpose: a run that stops at the first failure has
then already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import nnlib_jl_b200 as nb
from nnlib_jl_b200 import _lib

DEV = "cuda:0"


class _DeviceFloats:
    """n float32 values at a raw device address, for torch.as_tensor."""

    def __init__(self, ptr, n):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}


def _params(q, k, v, x, alpha, H, causal):
    E, Lq, B = q.shape
    p = _lib.AttnParams()
    p.dtype = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}[q.dtype]
    p.d, p.dv, p.H, p.Lq, p.Lkv, p.B = E // H, v.shape[0] // H, H, Lq, k.shape[1], B
    p.q, p.k, p.v, p.x, p.alpha = q.data_ptr(), k.data_ptr(), v.data_ptr(), x.data_ptr(), alpha.data_ptr()
    p.causal = int(causal)
    return p


def _both_ways(lib, dtype, E, H, Lq, Lkv, B, causal, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    q = nb.jl_empty((E, Lq, B), dtype, DEV); q.normal_(generator=g)
    k = nb.jl_empty((E, Lkv, B), dtype, DEV); k.normal_(generator=g)
    v = nb.jl_empty((E, Lkv, B), dtype, DEV); v.normal_(generator=g)
    st = torch.cuda.current_stream().cuda_stream
    # existing entry point, workspace owned by the caller
    x_ref = nb.jl_zeros((E, Lq, B), dtype, DEV)
    a_ref = nb.jl_zeros((Lkv, Lq, H, B), dtype, DEV)
    p = _params(q, k, v, x_ref, a_ref, H, causal)
    need = lib.nnlib_b200_workspace_bytes(C.byref(p))
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    assert lib.nnlib_b200_attention(C.byref(p), ws.data_ptr(), need, st) == _lib.OK
    # new entry point: no workspace argument at all
    x_new = nb.jl_zeros((E, Lq, B), dtype, DEV)
    a_new = nb.jl_zeros((Lkv, Lq, H, B), dtype, DEV)
    p2 = _params(q, k, v, x_new, a_new, H, causal)
    assert lib.nnlib_b200_attention_static(C.byref(p2), st) == _lib.OK
    torch.cuda.synchronize()
    nb.device_health(DEV)
    # same kernels, same inputs: the tolerance the parity tests use for this dtype is generous here
    tol = {torch.bfloat16: 2e-2, torch.float16: 3e-3, torch.float32: 1e-5}[dtype]
    assert torch.isfinite(x_new.float()).all() and torch.isfinite(a_new.float()).all()
    assert (x_new.float() - x_ref.float()).abs().max().item() <= tol
    assert (a_new.float() - a_ref.float()).abs().max().item() <= tol
    assert a_new.float().sum(0).sub(1).abs().max().item() <= 1e-2
    # the log-sum-exp really went through the library's own array: its first Lq*H*B entries hold what the
    # workspace of the other entry point holds (same kernels, same inputs)
    ptr, nbytes = C.c_void_p(), C.c_size_t()
    assert lib.nnlib_b200_static_scratch(C.byref(ptr), C.byref(nbytes)) == _lib.OK
    assert nbytes.value == 4 * _lib.STATIC_MAX_QUERIES and ptr.value % 256 == 0
    n = Lq * H * B
    scratch = torch.as_tensor(_DeviceFloats(ptr.value, n), device=DEV)
    assert torch.equal(scratch, ws.view(torch.float32)[:n])


@pytest.mark.gpu
def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    lib = _lib.load()
    # call 1: tensor-core kernels, 2*3*700 = 4200 queries
    _both_ways(lib, torch.bfloat16, 256, 2, 700, 900, 3, causal=False, seed=1)
    # call 2 right after, smaller and causal: entries of the array beyond its 600 queries still hold call 1's values
    _both_ways(lib, torch.bfloat16, 128, 1, 600, 600, 1, causal=True, seed=2)
    # and once through the CUDA-core kernels (Float32 inputs)
    _both_ways(lib, torch.float32, 48, 3, 70, 50, 2, causal=False, seed=3)


def test_static_scratch_entry_refuses_oversized_problems():
    # answered on the host before any CUDA call, so this part needs no GPU
    lib = _lib.load()
    p = _lib.AttnParams()
    p.dtype = _lib.BF16
    p.d = p.dv = 128
    p.q = p.k = p.v = p.x = p.alpha = 0x1000
    p.H, p.Lq, p.Lkv, p.B = 32, 4096, 4096, 8                 # exactly 2^20 queries: within the limit
    assert 32 * 4096 * 8 == _lib.STATIC_MAX_QUERIES
    p.B = 9
    assert lib.nnlib_b200_attention_static(C.byref(p), None) == _lib.WORKSPACE_TOO_SMALL
    p.B, p.Lq = 1, (1 << 20) + 1
    p.H = 1
    assert lib.nnlib_b200_attention_static(C.byref(p), None) == _lib.WORKSPACE_TOO_SMALL
    assert lib.nnlib_b200_attention_static(None, None) == _lib.INVALID_ARG
