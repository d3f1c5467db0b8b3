"""batched_mul / batched_mul! on the device (through the C ABI) against the CPU oracle: the reference's own
cases (test/batchedmul.jl), all four transpose combinations, ragged sizes, batch broadcast, alpha / beta,
both kernel families.  Tolerances: the Float32 oracle on the upcast inputs, relative to the largest entry of
the result; bf16 8e-3, f16 1e-3 (one rounding of the fp32 accumulator), f32 1e-5."""
import ctypes as C

import numpy as np
import pytest
import torch

import nnlib_jl_b200 as nb
from nnlib_jl_b200 import _lib, batched as BM
from oracle import batched_oracle as BO

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
REL = {torch.bfloat16: 8e-3, torch.float16: 1e-3, torch.float32: 1e-5}


def _round_to(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dtype).float().numpy()


def _dev(a, dtype):
    return nb.jl_from_numpy(np.asarray(a, dtype=np.float32), dtype=dtype, device=DEV)


def _close(got, want, dtype, what=""):
    got, want = got.astype(np.float64), want.astype(np.float64)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    assert np.isfinite(got).all(), what
    scale = np.abs(want).max() + 1e-30
    err = np.abs(got - want).max()
    assert err <= REL[dtype] * scale, f"{what}: {err / scale:.3e} of max |C|"


@pytest.fixture(autouse=True)
def _health():
    yield
    nb.device_health(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_reference_cases_small(dtype):
    # test/batchedmul.jl:40-49 — sizes (7,5,3) x (5,7,3): leading dimensions that no 16-byte rule fits, so
    # these run on the CUDA-core kernel
    rng = np.random.default_rng(0)
    An = _round_to(rng.standard_normal((7, 5, 3)), dtype)
    Bn = _round_to(rng.standard_normal((5, 7, 3)), dtype)
    Cn = _round_to(rng.standard_normal((7, 6, 3)), dtype)
    A, B, Cc = (_dev(a, dtype) for a in (An, Bn, Cn))
    bt, obt = nb.batched_transpose, BO.batched_transpose
    _close(nb.jl_to_numpy(nb.batched_mul(A, B)), BO.batched_mul(An, Bn), dtype, "A*B")
    _close(nb.jl_to_numpy(nb.batched_mul(bt(A), bt(B))), BO.batched_mul(obt(An), obt(Bn)), dtype, "A'*B'")
    _close(nb.jl_to_numpy(nb.batched_mul(bt(A), Cc)), BO.batched_mul(obt(An), Cn), dtype, "A'*C")
    _close(nb.jl_to_numpy(nb.batched_mul(A, bt(A))), BO.batched_mul(An, obt(An)), dtype, "A*A'")
    with pytest.raises(BM.DimensionMismatch):
        nb.batched_mul(_dev(rng.random((2, 2, 2)), dtype), _dev(rng.random((2, 2, 10)), dtype))
    with pytest.raises(BM.DimensionMismatch):
        nb.batched_mul(_dev(rng.random((2, 2, 2)), dtype), _dev(rng.random((10, 2, 2)), dtype))
    with pytest.raises(BM.DimensionMismatch):
        nb.batched_mul_(nb.jl_zeros((2, 2, 10), dtype, DEV), _dev(rng.random((2, 2, 2)), dtype),
                        _dev(rng.random((2, 2, 2)), dtype))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("ta,tb", [("N", "N"), ("T", "N"), ("N", "T"), ("T", "T")])
@pytest.mark.parametrize("M,N,K,nbatch", [
    (128, 128, 64, 1),        # one tile, one K block
    (256, 256, 128, 2),       # the 256 x 256 tile
    (200, 136, 72, 3),        # ragged in every dimension (multiples of 8: the tensor-core path)
    (520, 264, 200, 2),       # several tiles, partial last ones
    (96, 384, 320, 2),        # short M: 128-column tile
    (384, 104, 136, 1),       # narrow N: 128-row tile, two accumulators in turn
])
def test_tensor_core_product_all_transposes(dtype, ta, tb, M, N, K, nbatch):
    rng = np.random.default_rng(M * 7 + N * 3 + K + nbatch)
    An = _round_to(rng.standard_normal((M, K, nbatch) if ta == "N" else (K, M, nbatch)), dtype)
    Bn = _round_to(rng.standard_normal((K, N, nbatch) if tb == "N" else (N, K, nbatch)), dtype)
    A, B = _dev(An, dtype), _dev(Bn, dtype)
    opA = A if ta == "N" else nb.batched_transpose(A)
    opB = B if tb == "N" else nb.batched_transpose(B)
    Cd = nb.jl_empty((M, N, nbatch), dtype, DEV)
    assert BM.batched_mul_path(Cd, opA, opB) == _lib.PATH_UMMA
    got = nb.jl_to_numpy(nb.batched_mul(opA, opB))
    want = BO.batched_gemm(ta, tb, np.float32(1), An, Bn, np.float32(0), np.zeros((M, N, nbatch), np.float32))
    _close(got, want, dtype, f"{ta}{tb} {M}x{N}x{K}x{nbatch}")


def test_alpha_beta_batch_of_one_and_padded_leading_dimensions():
    """batched_mul!(C, A, B, α, β) with B shared by all batches (size(B,3) == 1), A a strided view whose
    columns are padded (lda > M), C written in place with β ≠ 0 and columns beyond the tile untouched."""
    dtype = torch.bfloat16
    rng = np.random.default_rng(5)
    M, N, K, nbatch = 136, 200, 96, 3
    Abig = _round_to(rng.standard_normal((160, K, nbatch)), dtype)          # lda = 160
    Bn = _round_to(rng.standard_normal((K, N, 1)), dtype)
    Cn = _round_to(rng.standard_normal((M, N, nbatch)), dtype)
    Ab = _dev(Abig, dtype)
    A = Ab[:M]                                                               # (M, K, nbatch) view, strides (1, 160, ...)
    B, Cd = _dev(Bn, dtype), _dev(Cn, dtype)
    assert BM.batched_mul_path(Cd, A, B) == _lib.PATH_UMMA
    out = nb.batched_mul_(Cd, A, B, 0.5, -2.0)
    assert out is Cd
    want = BO.batched_gemm("N", "N", np.float32(0.5), Abig[:M], Bn, np.float32(-2.0), Cn)
    _close(nb.jl_to_numpy(Cd), want, dtype, "alpha/beta")
    # beta = 0 must not read C: NaNs in it do not leak
    Cd.fill_(float("nan"))
    nb.batched_mul_(Cd, A, B)
    _close(nb.jl_to_numpy(Cd), BO.batched_mul(Abig[:M], Bn), dtype, "beta = 0 over NaN")
    # matrix factor and N-d batch (src/batched/batchedmul.jl:47-54, 112-125)
    A4n = _round_to(rng.standard_normal((64, 72, 2, 3)), dtype)
    B4n = _round_to(rng.standard_normal((72, 40, 2, 3)), dtype)
    C4 = nb.batched_mul(_dev(A4n, dtype), _dev(B4n, dtype))
    assert tuple(C4.shape) == (64, 40, 2, 3)
    _close(nb.jl_to_numpy(C4), BO.batched_mul(A4n, B4n), dtype, "4-d")
    Bm = _round_to(rng.standard_normal((72, 40)), dtype)
    _close(nb.jl_to_numpy(nb.batched_mul(_dev(A4n[:, :, :, 0], dtype), _dev(Bm, dtype))),
           BO.batched_mul(A4n[:, :, :, 0], Bm), dtype, "array x matrix")


def test_both_kernel_families_agree_and_attention_products():
    """The two products of the attention path written with batched_mul, as the reference does
    (src/attention.jl:119 logits = batched_mul(kt, qt); :97 x = batched_mul(vt, α)), on the tensor cores,
    against the CUDA-core kernel forced on the same call through the raw ABI."""
    dtype = torch.float16
    rng = np.random.default_rng(6)
    Lkv, Lq, d, HB = 264, 200, 64, 4
    kt = _round_to(rng.standard_normal((Lkv, d, HB)), dtype)
    qt = _round_to(rng.standard_normal((d, Lq, HB)) / 8, dtype)
    logits = nb.batched_mul(_dev(kt, dtype), _dev(qt, dtype))
    _close(nb.jl_to_numpy(logits), BO.batched_mul(kt, qt), dtype, "logits")
    lib = _lib.load()
    # same product with unaligned (odd) leading dimensions: CUDA-core kernel
    ktp = nb.jl_zeros((Lkv + 1, d, HB), dtype, DEV)
    ktp[:Lkv] = _dev(kt, dtype)
    Cs = nb.jl_empty((Lkv, Lq, HB), dtype, DEV)
    assert BM.batched_mul_path(Cs, ktp[:Lkv], _dev(qt, dtype)) == _lib.PATH_SIMT
    nb.batched_mul_(Cs, ktp[:Lkv], _dev(qt, dtype))
    _close(nb.jl_to_numpy(Cs), nb.jl_to_numpy(logits).astype(np.float32), dtype, "cuda-core vs tcgen05")
    assert lib.nnlib_b200_batched_gemm(None, None) == _lib.INVALID_ARG


def test_large_product_against_float32():
    """A size where the persistent grid runs many tiles per CTA and K spans many ring turns: 2 x (1024 x 1536 x
    1280) in bf16 against numpy's Float32 product of the same (rounded) inputs."""
    dtype = torch.bfloat16
    rng = np.random.default_rng(8)
    M, N, K, nbatch = 1024, 1536, 1280, 2
    An = _round_to(rng.standard_normal((M, K, nbatch)), dtype)
    Bn = _round_to(rng.standard_normal((K, N, nbatch)), dtype)
    got = nb.jl_to_numpy(nb.batched_mul(_dev(An, dtype), _dev(Bn, dtype)))
    _close(got, BO.batched_mul(An, Bn), dtype, "large NN")
    got = nb.jl_to_numpy(nb.batched_mul(nb.batched_transpose(_dev(np.transpose(An, (1, 0, 2)), dtype)),
                                        nb.batched_transpose(_dev(np.transpose(Bn, (1, 0, 2)), dtype))))
    _close(got, BO.batched_mul(An, Bn), dtype, "large TT")


@pytest.mark.parametrize("seed", range(40))
def test_random_products_match_the_oracle(seed):
    """Seeded random draws: element type, transposes, sizes from a few elements to several tiles (multiples of 8
    or not — the second kind takes the CUDA-core kernel), batch count, a batch of one on either side, alpha / beta,
    padded leading dimensions."""
    rng = np.random.default_rng(11000 + seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    ta, tb = str(rng.choice(["N", "T"])), str(rng.choice(["N", "T"]))
    if rng.random() < 0.6:
        M, N, K = (int(8 * rng.integers(1, 70)) for _ in range(3))
    else:
        M, N, K = (int(rng.integers(1, 300)) for _ in range(3))
    if dtype == torch.float32:
        M, N, K = min(M, 200), min(N, 200), min(K, 200)
    nbatch = int(rng.integers(1, 5))
    ba = 1 if rng.random() < 0.2 else nbatch                  # size(A, 3) == 1: the same matrix for every batch
    bb = 1 if rng.random() < 0.2 else nbatch
    pad_a = int(rng.choice([0, 0, 8, 3]))                     # rows of padding under each column of A's storage
    sa = (M, K) if ta == "N" else (K, M)
    sb = (K, N) if tb == "N" else (N, K)
    Abig = _round_to(rng.standard_normal((sa[0] + pad_a, sa[1], ba)), dtype)
    Bn = _round_to(rng.standard_normal((sb[0], sb[1], bb)), dtype)
    Cn = _round_to(rng.standard_normal((M, N, nbatch)), dtype)
    An = Abig[:sa[0]]
    A = _dev(Abig, dtype)[:sa[0]]
    B, Cd = _dev(Bn, dtype), _dev(Cn, dtype)
    opA = A if ta == "N" else nb.batched_transpose(A)
    opB = B if tb == "N" else nb.batched_transpose(B)
    alpha, beta = (1.0, 0.0) if rng.random() < 0.5 else (float(rng.choice([0.5, -1.5, 2.0])), float(rng.choice([0.0, 1.0, -0.5])))
    what = f"seed {seed}: {dtype} {ta}{tb} {M}x{N}x{K} batches {ba}/{bb}/{nbatch} pad {pad_a} alpha {alpha} beta {beta}"
    nb.batched_mul_(Cd, opA, opB, alpha, beta)
    want = BO.batched_gemm(ta, tb, np.float32(alpha), An, Bn, np.float32(beta), Cn)
    _close(nb.jl_to_numpy(Cd), want, dtype, what)
