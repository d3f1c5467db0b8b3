"""softmax / logsoftmax kernels against the CPU oracle (the comparison the reference's
test/ext_cuda/softmax.jl makes between its CPU and CUDA methods)."""
import numpy as np
import pytest
import torch

import nnlib_jl_b200 as nb
from nnlib_jl_b200 import softmax as SM
from oracle import softmax_oracle as S

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {torch.float32: 2e-6, torch.float16: 2e-3, torch.bfloat16: 1.6e-2}


def _dev(a, dtype):
    return nb.jl_from_numpy(np.asarray(a, dtype=np.float32), device=DEV).to(dtype) if dtype != torch.float32 \
        else nb.jl_from_numpy(np.asarray(a, dtype=np.float32), device=DEV)


def _round(a, dtype):
    return torch.from_numpy(np.asarray(a, dtype=np.float32)).to(dtype).float().numpy()


def _as_cm(t, dtype):
    """column-major device tensor of element type dtype"""
    out = nb.jl_empty(tuple(t.shape), dtype, DEV)
    out.copy_(t)
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape,dims", [
    ((5, 7), 1), ((5, 7), 2), ((300, 33), 1), ((2000, 9), 1), ((4100, 3), 1),      # warp- and block-per-column
    ((256, 10, 32), 2), ((16, 5, 3, 4), 3), ((16, 5, 3, 4), 4), ((7, 9), None), ((3, 4), 3), ((6, 5, 4), (1, 2)), ((6, 5, 4), (2, 3)),
])
def test_forward_and_pullbacks_match_the_oracle(dtype, shape, dims):
    rng = np.random.default_rng(5)
    xn = _round(3.0 * rng.standard_normal(shape), dtype)
    dyn = _round(rng.standard_normal(shape), dtype)
    x, dy = _as_cm(_dev(xn, dtype), dtype), _as_cm(_dev(dyn, dtype), dtype)
    tol = TOL[dtype]
    y = SM.softmax(x, dims=dims)
    ly = SM.logsoftmax(x, dims=dims)
    yo, lyo = S.softmax(xn, dims), S.logsoftmax(xn, dims)
    np.testing.assert_allclose(nb.jl_to_numpy(y), yo, atol=tol, rtol=tol)
    np.testing.assert_allclose(nb.jl_to_numpy(ly), lyo, atol=tol * max(1.0, np.abs(lyo).max()), rtol=tol)
    # pullbacks take the device's own (rounded) y, like the reference's rrule does
    yr, lyr = nb.jl_to_numpy(y), nb.jl_to_numpy(ly)
    dx = SM.softmax_pullback(dy, y, dims=dims)
    np.testing.assert_allclose(nb.jl_to_numpy(dx), S.softmax_pullback(dyn, yr, dims), atol=4 * tol, rtol=4 * tol)
    dlx = SM.logsoftmax_pullback(dy, ly, dims=dims)
    want = S.logsoftmax_pullback(dyn, lyr, dims)
    np.testing.assert_allclose(nb.jl_to_numpy(dlx), want, atol=4 * tol * max(1.0, np.abs(want).max()), rtol=4 * tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape,dims", [((300, 33), 1), ((70000, 3), 1), ((64, 50, 4), 2)])
def test_in_place_forms(dtype, shape, dims):
    """softmax!(x, x) and the pullbacks written over dy or y (src/softmax.jl:66, 98-101): the same values as
    the out-of-place calls, for a warp per column, a block per column with re-read columns, and the
    strided kernel."""
    rng = np.random.default_rng(7)
    x = _as_cm(_dev(_round(3.0 * rng.standard_normal(shape), dtype), dtype), dtype)
    dy = _as_cm(_dev(_round(rng.standard_normal(shape), dtype), dtype), dtype)
    for fwd, bwd in ((SM.softmax, SM.softmax_pullback), (SM.logsoftmax, SM.logsoftmax_pullback)):
        y = fwd(x, dims=dims)
        xc = x.clone()
        assert fwd(xc, dims=dims, out=xc) is xc
        assert torch.equal(xc, y)
        dx = bwd(dy, y, dims=dims)
        dyc, yc = dy.clone(), y.clone()
        bwd(dyc, y, dims=dims, out=dyc)
        bwd(dy, yc, dims=dims, out=yc)
        assert torch.equal(dyc, dx) and torch.equal(yc, dx)


def test_inf_nan_table_on_device():
    # test/softmax.jl:62-75 and the masked-input regression of test/ext_cuda/softmax.jl:34-78
    f, inf, nan = np.float32, np.inf, np.nan
    for xn in (f([[1, 2], [3, inf]]), f([[1, -inf], [3, inf]]), f([[1, inf], [3, inf]]), f([[1, 2], [3, nan]]),
               f([[-inf, 1], [-inf, 2]]), f([[-1000, 1], [-1000, -inf]])):
        for dims in (1, 2):
            x = _as_cm(_dev(xn, torch.float32), torch.float32)
            np.testing.assert_allclose(nb.jl_to_numpy(SM.softmax(x, dims=dims)), S.softmax(xn, dims), rtol=1e-6, atol=1e-7)
            got, want = nb.jl_to_numpy(SM.logsoftmax(x, dims=dims)), S.logsoftmax(xn, dims)
            np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-6)
    # masked entries are exactly zero, the others sum to one
    rng = np.random.default_rng(6)
    xn = rng.standard_normal((64, 50)).astype(np.float32)
    keep = rng.random((64, 50)) > 0.4
    keep[0] = True
    xm = np.where(keep, xn, -np.inf).astype(np.float32)
    y = nb.jl_to_numpy(SM.softmax(_as_cm(_dev(xm, torch.float32), torch.float32)))
    assert ((y > 0) == keep).all()
    np.testing.assert_allclose(y.sum(0), 1.0, rtol=1e-5)


def test_argument_checks():
    x = nb.jl_zeros((4, 5), torch.float32, DEV)
    with pytest.raises(nb.ArgumentError):
        SM.softmax(x, dims=0)
    with pytest.raises(nb.ArgumentError):
        SM.softmax(nb.jl_zeros((4, 5, 6), torch.float32, DEV), dims=(1, 3))
    with pytest.raises(nb.ArgumentError):
        SM.softmax_pullback(nb.jl_zeros((4, 6), torch.float32, DEV), x)
    with pytest.raises(TypeError):
        SM.softmax(torch.zeros(3, 3))
    assert tuple(SM.softmax(nb.jl_zeros((0, 5), torch.float32, DEV)).shape) == (0, 5)


@pytest.mark.parametrize("seed", range(40))
def test_random_shapes_and_dims_match_the_oracle(seed):
    """Seeded random draws: element type, rank 1 to 4, sizes that land on every kernel variant (a warp, a block
    or a large block per column, cached or re-read columns, the strided kernel), any run of consecutive dims,
    forward / log forward and both pullbacks, out of place and in place."""
    rng = np.random.default_rng(12000 + seed)
    dtype = [torch.float32, torch.float16, torch.bfloat16][seed % 3]
    rank = int(rng.integers(1, 5))
    first = int(rng.choice([1, 3, 8, 33, 64, 257, 512, 1000, 2048, 4100, 9000, 20000]))
    rest = [int(rng.integers(1, 7)) for _ in range(rank - 1)]
    shape = tuple([min(first, max(1, 600000 // int(np.prod(rest)))) if rest else first] + rest)
    lo = int(rng.integers(1, rank + 1)); hi = int(rng.integers(lo, rank + 1))
    dims = lo if lo == hi else tuple(range(lo, hi + 1))
    xn = _round(3.0 * rng.standard_normal(shape), dtype)
    dyn = _round(rng.standard_normal(shape), dtype)
    x, dy = _as_cm(_dev(xn, dtype), dtype), _as_cm(_dev(dyn, dtype), dtype)
    tol = TOL[dtype]
    what = f"seed {seed}: {dtype} shape {shape} dims {dims}"
    y, ly = SM.softmax(x, dims=dims), SM.logsoftmax(x, dims=dims)
    yo, lyo = S.softmax(xn, dims), S.logsoftmax(xn, dims)
    np.testing.assert_allclose(nb.jl_to_numpy(y), yo, atol=tol, rtol=tol, err_msg=what)
    np.testing.assert_allclose(nb.jl_to_numpy(ly), lyo, atol=tol * max(1.0, np.abs(lyo).max()), rtol=tol, err_msg=what)
    yr, lyr = nb.jl_to_numpy(y), nb.jl_to_numpy(ly)
    dx = SM.softmax_pullback(dy, y, dims=dims)
    np.testing.assert_allclose(nb.jl_to_numpy(dx), S.softmax_pullback(dyn, yr, dims), atol=4 * tol, rtol=4 * tol, err_msg=what)
    dlx = SM.logsoftmax_pullback(dy, ly, dims=dims)
    want = S.logsoftmax_pullback(dyn, lyr, dims)
    np.testing.assert_allclose(nb.jl_to_numpy(dlx), want, atol=4 * tol * max(1.0, np.abs(want).max()), rtol=4 * tol, err_msg=what)
    # in place: the same values as out of place, bit for bit
    x2 = _as_cm(_dev(xn, dtype), dtype)
    SM.softmax(x2, dims=dims, out=x2)
    assert torch.equal(x2, y), what
    dy2 = _as_cm(_dev(dyn, dtype), dtype)
    SM.softmax_pullback(dy2, y, dims=dims, out=dy2)
    assert torch.equal(dy2, dx), what
