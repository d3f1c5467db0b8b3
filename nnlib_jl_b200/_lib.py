"""ctypes binding of ``libnnlib_b200.so`` (declared in ``include/nnlib_b200.h``).

This is what the Julia extension does with ``ccall``: fill one
``nnlib_b200_attn_params`` struct with device pointers, sizes and strides and
hand it to an entry point together with the current stream.  There is no
fallback: if the shared library is missing or an entry point is absent, loading
raises.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

F16, BF16, F32 = 0, 1, 2

OK = 0
INVALID_ARG = -1
UNSUPPORTED_SHAPE = -2
CUDA_ERROR = -3
TIMEOUT = -4
WORKSPACE_TOO_SMALL = -5

STATIC_MAX_QUERIES = 1 << 20

PATH_SIMT = 1
PATH_UMMA = 2
PATH_TILE = 3

LIB_NAME = "libnnlib_b200.so"
LIB_PATH = Path(__file__).resolve().parent / LIB_NAME

# every symbol include/nnlib_b200.h declares
EXPORTS = (
    "nnlib_b200_attn_fwd",
    "nnlib_b200_attn_decode",
    "nnlib_b200_attn_decode_workspace_bytes",
    "nnlib_b200_attn_stats",
    "nnlib_b200_attn_scores",
    "nnlib_b200_attn_apply",
    "nnlib_b200_attention",
    "nnlib_b200_workspace_bytes",
    "nnlib_b200_attention_static",
    "nnlib_b200_static_scratch",
    "nnlib_b200_attn_bwd",
    "nnlib_b200_attn_bwd_path",
    "nnlib_b200_batched_gemm",
    "nnlib_b200_batched_gemm_path",
    "nnlib_b200_causal_fill",
    "nnlib_b200_causal_check",
    "nnlib_b200_attn_path",
    "nnlib_b200_softmax_fwd",
    "nnlib_b200_softmax_bwd",
    "nnlib_b200_device_health",
    "nnlib_b200_selftest_wait_runout",
    "nnlib_b200_strerror",
    "nnlib_b200_version",
    "nnlib_b200_last_cuda_error",
    "nnlib_b200_launch_count",
)


class AttnParams(C.Structure):
    """Mirror of ``nnlib_b200_attn_params`` (field order and types must match
    the header exactly)."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("dtype", C.c_int32),
        ("bias_dtype", C.c_int32),
        ("d", C.c_int64), ("dv", C.c_int64), ("H", C.c_int64),
        ("Lq", C.c_int64), ("Lkv", C.c_int64), ("B", C.c_int64),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("x", C.c_void_p),
        ("q_stride_l", C.c_int64), ("q_stride_b", C.c_int64),
        ("k_stride_l", C.c_int64), ("k_stride_b", C.c_int64),
        ("v_stride_l", C.c_int64), ("v_stride_b", C.c_int64),
        ("x_stride_l", C.c_int64), ("x_stride_b", C.c_int64),
        ("bias", C.c_void_p), ("bias_stride", C.c_int64 * 4),
        ("mask", C.c_void_p), ("mask_stride", C.c_int64 * 4),
        ("causal", C.c_int32), ("nan_on_fully_masked", C.c_int32),
        ("scale", C.c_float),
        ("dropout_p", C.c_float),
        ("philox_seed", C.c_uint64), ("philox_offset", C.c_uint64),
        ("rng_h0", C.c_int64), ("rng_b0", C.c_int64), ("rng_H", C.c_int64),
        ("lse", C.c_void_p), ("lse_stride_b", C.c_int64),
        ("alpha", C.c_void_p), ("alpha_stride_b", C.c_int64),
        ("status", C.c_void_p),
        ("allow_tf32", C.c_int32), ("reserved0", C.c_int32),
        ("causal_offset", C.c_int64),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(AttnParams)
        if "nan_on_fully_masked" not in kw:
            self.nan_on_fully_masked = 1


class AttnGrads(C.Structure):
    """Mirror of ``nnlib_b200_attn_grads``."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("dx", C.c_void_p), ("dx_stride_l", C.c_int64), ("dx_stride_b", C.c_int64),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dbias", C.c_void_p), ("dbias_stride", C.c_int64 * 4),
        ("delta", C.c_void_p),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(AttnGrads)


class GemmParams(C.Structure):
    """Mirror of ``nnlib_b200_gemm_params``."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("dtype", C.c_int32), ("transA", C.c_int32), ("transB", C.c_int32), ("reserved", C.c_int32),
        ("M", C.c_int64), ("N", C.c_int64), ("K", C.c_int64), ("batch", C.c_int64),
        ("A", C.c_void_p), ("lda", C.c_int64), ("strideA", C.c_int64),
        ("B", C.c_void_p), ("ldb", C.c_int64), ("strideB", C.c_int64),
        ("C", C.c_void_p), ("ldc", C.c_int64), ("strideC", C.c_int64),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("status", C.c_void_p),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(GemmParams)
        if "alpha" not in kw:
            self.alpha = 1.0


class SoftmaxParams(C.Structure):
    """Mirror of ``nnlib_b200_softmax_params``."""

    _fields_ = [
        ("struct_size", C.c_size_t),
        ("dtype", C.c_int32), ("log", C.c_int32),
        ("inner", C.c_int64), ("n", C.c_int64), ("outer", C.c_int64),
        ("x", C.c_void_p), ("dy", C.c_void_p), ("out", C.c_void_p),
    ]

    def __init__(self, **kw):
        super().__init__(**kw)
        self.struct_size = C.sizeof(SoftmaxParams)


_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it (or any export) is missing."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("NNLIB_B200_LIB", str(LIB_PATH)))
    if not path.exists():
        raise ImportError(
            f"{path} not found: build it with `python -m nnlib_jl_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for this path)")
    lib = C.CDLL(str(path))
    missing = [s for s in EXPORTS if not hasattr(lib, s)]
    if missing:
        raise ImportError(f"{path} lacks symbols {missing}")
    P = C.POINTER(AttnParams)
    for name in ("nnlib_b200_attn_fwd", "nnlib_b200_attn_stats", "nnlib_b200_attn_scores", "nnlib_b200_attn_apply"):
        fn = getattr(lib, name)
        fn.argtypes = [P, C.c_void_p]
        fn.restype = C.c_int
    lib.nnlib_b200_attn_decode.argtypes = [P, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.nnlib_b200_attn_decode.restype = C.c_int
    lib.nnlib_b200_attn_decode_workspace_bytes.argtypes = [P]
    lib.nnlib_b200_attn_decode_workspace_bytes.restype = C.c_size_t
    lib.nnlib_b200_attention.argtypes = [P, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.nnlib_b200_attention.restype = C.c_int
    lib.nnlib_b200_attention_static.argtypes = [P, C.c_void_p]
    lib.nnlib_b200_attention_static.restype = C.c_int
    lib.nnlib_b200_static_scratch.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]
    lib.nnlib_b200_static_scratch.restype = C.c_int
    lib.nnlib_b200_selftest_wait_runout.argtypes = [C.c_uint64, C.c_void_p, C.c_void_p]
    lib.nnlib_b200_selftest_wait_runout.restype = C.c_int
    lib.nnlib_b200_attn_bwd.argtypes = [P, C.POINTER(AttnGrads), C.c_void_p]
    lib.nnlib_b200_attn_bwd.restype = C.c_int
    lib.nnlib_b200_attn_bwd_path.argtypes = [P, C.POINTER(AttnGrads)]
    lib.nnlib_b200_attn_bwd_path.restype = C.c_int
    lib.nnlib_b200_workspace_bytes.argtypes = [P]
    lib.nnlib_b200_workspace_bytes.restype = C.c_size_t
    lib.nnlib_b200_batched_gemm.argtypes = [C.POINTER(GemmParams), C.c_void_p]
    lib.nnlib_b200_batched_gemm.restype = C.c_int
    lib.nnlib_b200_batched_gemm_path.argtypes = [C.POINTER(GemmParams)]
    lib.nnlib_b200_batched_gemm_path.restype = C.c_int
    lib.nnlib_b200_causal_fill.argtypes = [C.c_void_p, C.c_int64, C.c_void_p]
    lib.nnlib_b200_causal_fill.restype = C.c_int
    lib.nnlib_b200_causal_check.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]
    lib.nnlib_b200_causal_check.restype = C.c_int
    lib.nnlib_b200_softmax_fwd.argtypes = [C.POINTER(SoftmaxParams), C.c_void_p]
    lib.nnlib_b200_softmax_fwd.restype = C.c_int
    lib.nnlib_b200_softmax_bwd.argtypes = [C.POINTER(SoftmaxParams), C.c_void_p]
    lib.nnlib_b200_softmax_bwd.restype = C.c_int
    lib.nnlib_b200_attn_path.argtypes = [P]
    lib.nnlib_b200_attn_path.restype = C.c_int
    lib.nnlib_b200_device_health.argtypes = [C.c_void_p]
    lib.nnlib_b200_device_health.restype = C.c_int
    lib.nnlib_b200_strerror.argtypes = [C.c_int]
    lib.nnlib_b200_strerror.restype = C.c_char_p
    lib.nnlib_b200_version.argtypes = []
    lib.nnlib_b200_version.restype = C.c_int
    lib.nnlib_b200_last_cuda_error.argtypes = []
    lib.nnlib_b200_last_cuda_error.restype = C.c_int
    lib.nnlib_b200_launch_count.argtypes = []
    lib.nnlib_b200_launch_count.restype = C.c_uint64
    _lib = lib
    return lib


def strerror(code: int) -> str:
    return load().nnlib_b200_strerror(code).decode()


class NNlibB200Error(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        extra = ""
        if code == CUDA_ERROR:
            extra = f" (cudaError {load().nnlib_b200_last_cuda_error()})"
        super().__init__(f"{where}: {strerror(code)}{extra} [{code}]")
