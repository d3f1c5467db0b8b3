"""The C-ABI shared library without a GPU: it loads, exports every symbol the
header declares, its params struct matches the ctypes mirror, and argument
checking answers before any CUDA call is made."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

from nnlib_jl_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "nnlib_b200.h"


def test_every_declared_symbol_is_exported(lib):
    declared = re.findall(r"NNLIB_B200_API\s+[\w\s\*]+?\b(nnlib_b200_\w+)\s*\(", HEADER.read_text())
    assert len(declared) >= 14
    assert set(declared) == set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name


def test_nothing_else_is_exported(lib):
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True).stdout
    names = [ln.split()[-1] for ln in out.splitlines() if ln.strip()]
    assert names and all(n.startswith("nnlib_b200_") for n in names), names


def test_struct_layout_matches_header(tmp_path):
    src = tmp_path / "sz.c"
    src.write_text(
        '#include "nnlib_b200.h"\n#include <stdio.h>\n#include <stddef.h>\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu\\n\", sizeof(nnlib_b200_attn_params),"
        "offsetof(nnlib_b200_attn_params, q), offsetof(nnlib_b200_attn_params, bias_stride),"
        "offsetof(nnlib_b200_attn_params, scale), offsetof(nnlib_b200_attn_params, status));return 0;}\n")
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-std=c99", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    A = _lib.AttnParams
    assert got == [C.sizeof(A), A.q.offset, A.bias_stride.offset, A.scale.offset, A.status.offset]


def test_version_and_strerror(lib):
    assert lib.nnlib_b200_version() == 200
    assert _lib.strerror(0) == "ok"
    for code in (-1, -2, -3, -4, -5, -99):
        assert _lib.strerror(code)
    assert lib.nnlib_b200_launch_count() >= 0


def _params(**kw):
    p = _lib.AttnParams()
    p.dtype = _lib.BF16
    p.d = p.dv = 64
    p.H, p.Lq, p.Lkv, p.B = 2, 16, 16, 1
    # fake non-null pointers: validation must reject the call before touching them
    p.q = p.k = p.v = p.x = 0x1000
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("bad", [
    dict(dtype=7), dict(d=0), dict(H=0), dict(Lq=-1), dict(dropout_p=1.0), dict(dropout_p=-0.1),
    dict(scale=-1.0), dict(q=None), dict(x=None), dict(q_stride_l=64), dict(struct_size=8),
    dict(bias=0x1000, bias_dtype=9), dict(rng_h0=-1), dict(lse_stride_b=1),
])
def test_invalid_arguments_are_rejected_without_a_gpu(lib, bad):
    p = _params(**bad)
    assert lib.nnlib_b200_attn_fwd(C.byref(p), None) == _lib.INVALID_ARG


def test_null_params_and_missing_outputs(lib):
    assert lib.nnlib_b200_attn_fwd(None, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_scores(C.byref(_params()), None) == _lib.INVALID_ARG      # lse / alpha missing
    assert lib.nnlib_b200_attn_apply(C.byref(_params()), None) == _lib.INVALID_ARG       # alpha missing
    assert lib.nnlib_b200_attn_stats(C.byref(_params()), None) == _lib.INVALID_ARG       # lse missing
    assert lib.nnlib_b200_causal_fill(None, 4, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_causal_check(None, 4, None, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attention(None, None, 0, None) == _lib.INVALID_ARG


def _grads(**kw):
    g = _lib.AttnGrads()
    g.dx = g.dq = g.dk = g.dv = g.delta = 0x3000   # fake non-null pointers, never dereferenced here
    for k, v in kw.items():
        setattr(g, k, v)
    return g


def test_backward_argument_checks_and_path_without_a_gpu(lib):
    p = _params(lse=0x2000)
    # the forward's lse is required, so are dx / dq / dk / dv / delta, and the struct size is checked
    assert lib.nnlib_b200_attn_bwd(C.byref(_params()), C.byref(_grads()), None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_bwd(C.byref(p), None, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(_grads(dx=None)), None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(_grads(delta=None)), None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(_grads(struct_size=8)), None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(_grads(dx_stride_l=8)), None) == _lib.INVALID_ARG
    g = _grads()
    g.dbias_stride[1] = -1
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(g), None) == _lib.INVALID_ARG
    # the same validation in front of the path query; without a driver only the CUDA-core path is on offer
    assert lib.nnlib_b200_attn_bwd_path(C.byref(_params()), C.byref(_grads())) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_bwd_path(C.byref(p), C.byref(_grads())) in (_lib.PATH_SIMT, _lib.PATH_UMMA)
    assert lib.nnlib_b200_attn_bwd_path(C.byref(_params(lse=0x2000, dtype=_lib.F32)), C.byref(_grads())) == _lib.PATH_SIMT
    assert lib.nnlib_b200_attn_bwd_path(C.byref(_params(lse=0x2000, d=2048, dv=2048)), C.byref(_grads())) \
        == _lib.UNSUPPORTED_SHAPE
    # empty problems are fine and launch nothing
    before = lib.nnlib_b200_launch_count()
    assert lib.nnlib_b200_attn_bwd(C.byref(_params(lse=0x2000, B=0)), C.byref(_grads()), None) == _lib.OK
    assert lib.nnlib_b200_launch_count() == before


def test_softmax_argument_checks_without_a_gpu(lib):
    def sp(**kw):
        p = _lib.SoftmaxParams()
        p.dtype = _lib.F32
        p.inner, p.n, p.outer = 1, 8, 4
        p.x = p.out = p.dy = 0x4000
        for k, v in kw.items():
            setattr(p, k, v)
        return p
    for fn in (lib.nnlib_b200_softmax_fwd, lib.nnlib_b200_softmax_bwd):
        assert fn(None, None) == _lib.INVALID_ARG
        assert fn(C.byref(sp(struct_size=4)), None) == _lib.INVALID_ARG
        assert fn(C.byref(sp(dtype=5)), None) == _lib.INVALID_ARG
        assert fn(C.byref(sp(n=-1)), None) == _lib.INVALID_ARG
        assert fn(C.byref(sp(x=None)), None) == _lib.INVALID_ARG
        assert fn(C.byref(sp(out=None)), None) == _lib.INVALID_ARG
        assert fn(C.byref(sp(inner=2 ** 40, n=2 ** 40)), None) == _lib.INVALID_ARG      # size overflow
    assert lib.nnlib_b200_softmax_bwd(C.byref(sp(dy=None)), None) == _lib.INVALID_ARG
    before = lib.nnlib_b200_launch_count()
    assert lib.nnlib_b200_softmax_fwd(C.byref(sp(n=0, x=None, out=None)), None) == _lib.OK    # empty: nothing to do
    assert lib.nnlib_b200_launch_count() == before


def test_empty_problems_enqueue_nothing(lib):
    before = lib.nnlib_b200_launch_count()
    assert lib.nnlib_b200_attn_fwd(C.byref(_params(Lq=0)), None) == _lib.OK
    assert lib.nnlib_b200_attn_fwd(C.byref(_params(B=0)), None) == _lib.OK
    assert lib.nnlib_b200_causal_fill(None, 0, None) == _lib.OK
    assert lib.nnlib_b200_launch_count() == before


def test_workspace_bytes(lib):
    p = _params(Lq=100, H=3, B=5)
    assert lib.nnlib_b200_workspace_bytes(C.byref(p)) == 100 * 3 * 5 * 4
    p.lse = 0x2000
    assert lib.nnlib_b200_workspace_bytes(C.byref(p)) == 0
    assert lib.nnlib_b200_attention(C.byref(_params()), None, 0, None) == _lib.WORKSPACE_TOO_SMALL


def test_path_selection_is_pure_host_logic(lib):
    # f32 and odd head sizes go to the CUDA-core kernels; the selection needs no device
    assert lib.nnlib_b200_attn_path(C.byref(_params(dtype=_lib.F32))) == _lib.PATH_SIMT
    assert lib.nnlib_b200_attn_path(C.byref(_params(d=48, dv=48))) == _lib.PATH_SIMT
    assert lib.nnlib_b200_attn_path(C.byref(_params(d=2048, dv=2048))) == _lib.UNSUPPORTED_SHAPE
    assert lib.nnlib_b200_attn_path(C.byref(_params(q=0x1004))) == _lib.PATH_SIMT          # unaligned rows


def test_composites_check_both_halves_before_anything_is_enqueued(lib):
    # x + alpha in one call: a missing alpha (checked by the second half only) must be reported before the first
    # half runs, i.e. without a CUDA call — this box has no GPU, so anything else would answer CUDA_ERROR
    before = lib.nnlib_b200_launch_count()
    p = _params(lse=0x2000)                       # alpha missing
    assert lib.nnlib_b200_attention(C.byref(p), None, 0, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attention_static(C.byref(_params()), None) == _lib.INVALID_ARG
    p = _params(lse=0x2000, alpha=0x3000, alpha_stride_b=1)      # batches of alpha would overlap
    assert lib.nnlib_b200_attention(C.byref(p), None, 0, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_launch_count() == before


def test_backward_wants_dk_dv_whenever_there_are_keys(lib):
    # no queries but keys: dk and dv are still written (zeros), so they must be given
    p = _params(lse=0x2000, Lq=0)
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(_grads(dk=None)), None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(_grads(dv=None)), None) == _lib.INVALID_ARG
    # no keys at all: nothing to write
    assert lib.nnlib_b200_attn_bwd(C.byref(_params(lse=0x2000, Lq=0, Lkv=0)), C.byref(_grads(dk=None, dv=None)), None) == _lib.OK


def _gemm(**kw):
    g = _lib.GemmParams()
    g.dtype = _lib.BF16
    g.M, g.N, g.K, g.batch = 64, 32, 16, 2
    g.A = g.B = g.C = 0x5000
    g.lda, g.ldb, g.ldc = 64, 16, 64
    g.strideA, g.strideB, g.strideC = 64 * 16, 16 * 32, 64 * 32
    for k, v in kw.items():
        setattr(g, k, v)
    return g


def test_batched_gemm_argument_checks_and_path_without_a_gpu(lib):
    assert lib.nnlib_b200_batched_gemm(None, None) == _lib.INVALID_ARG
    for bad in (dict(struct_size=8), dict(dtype=9), dict(transA=2), dict(M=-1), dict(lda=63), dict(ldb=15), dict(ldc=63),
                dict(A=None), dict(C=None), dict(strideC=100), dict(alpha=float("nan")), dict(strideA=-1),
                dict(transA=1, lda=15)):
        assert lib.nnlib_b200_batched_gemm(C.byref(_gemm(**bad)), None) == _lib.INVALID_ARG, bad
    # the path is pure host logic: aligned 16-bit operands take the tensor cores (when the driver is there),
    # Float32 and unaligned leading dimensions the CUDA-core kernel
    assert lib.nnlib_b200_batched_gemm_path(C.byref(_gemm())) in (_lib.PATH_UMMA, _lib.PATH_SIMT)
    assert lib.nnlib_b200_batched_gemm_path(C.byref(_gemm(dtype=_lib.F32))) == _lib.PATH_SIMT
    assert lib.nnlib_b200_batched_gemm_path(C.byref(_gemm(lda=65))) == _lib.PATH_SIMT
    assert lib.nnlib_b200_batched_gemm_path(C.byref(_gemm(A=0x5004))) == _lib.PATH_SIMT
    # empty products enqueue nothing
    before = lib.nnlib_b200_launch_count()
    assert lib.nnlib_b200_batched_gemm(C.byref(_gemm(batch=0)), None) == _lib.OK
    assert lib.nnlib_b200_batched_gemm(C.byref(_gemm(M=0, lda=1, ldc=1)), None) == _lib.OK
    assert lib.nnlib_b200_launch_count() == before


def test_decode_entry_and_new_fields_without_a_gpu(lib):
    assert lib.nnlib_b200_attn_decode(None, None, 0, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_attn_decode_workspace_bytes(None) == 0
    assert lib.nnlib_b200_attn_decode(C.byref(_params(Lq=0)), None, 0, None) == _lib.OK        # empty: nothing to do
    assert lib.nnlib_b200_attn_fwd(C.byref(_params(causal=1, causal_offset=2 ** 40)), None) == _lib.INVALID_ARG
    # more than one query tile never splits; neither does a short key sequence
    assert lib.nnlib_b200_attn_decode_workspace_bytes(C.byref(_params(Lq=129, Lkv=100000))) == 0
    assert lib.nnlib_b200_attn_decode_workspace_bytes(C.byref(_params(Lq=1, Lkv=128))) == 0
    # Float32 takes the tensor cores only when the caller allows TF32
    assert lib.nnlib_b200_attn_path(C.byref(_params(dtype=_lib.F32))) == _lib.PATH_SIMT
    assert lib.nnlib_b200_attn_path(C.byref(_params(dtype=_lib.F32, allow_tf32=1))) in (_lib.PATH_TILE, _lib.PATH_SIMT)
    assert lib.nnlib_b200_selftest_wait_runout(0, None, None) == _lib.INVALID_ARG
    assert lib.nnlib_b200_static_scratch(None, None) == _lib.INVALID_ARG
