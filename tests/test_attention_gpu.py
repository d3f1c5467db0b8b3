"""Parity of the CUDA path (through the C ABI of libnnlib_b200.so) with the CPU
oracle, on the reference's own test cases (test/attention.jl,
test/ext_amdgpu/attention.jl) and on the benchmark configurations.

Tolerances (max-abs, mean-rel = mean|y-ŷ| / mean|ŷ|) against the Float32 oracle
evaluated on the upcast inputs:
    bf16 : 2e-2 , 5e-3        f16 : 3e-3 , 1e-3        f32 : 1e-5 (atol, like the reference's GPU tests)
"""
import math
import time

import numpy as np
import pytest
import torch

import nnlib_jl_b200 as nb
from nnlib_jl_b200 import _lib
from oracle import attention_oracle as O
from oracle import philox_oracle as P

pytestmark = pytest.mark.gpu

TOL = {torch.bfloat16: (2e-2, 5e-3), torch.float16: (3e-3, 1e-3), torch.float32: (1e-5, 1e-5)}
DEV = "cuda:0"


def _round_to(a: np.ndarray, dtype) -> np.ndarray:
    """float32 values of `a` after rounding to the tensor dtype (what the device sees)."""
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dtype).float().numpy()


def _dev(a: np.ndarray, dtype):
    return nb.jl_from_numpy(a.astype(np.float32), dtype=dtype, device=DEV)


def _close(got: np.ndarray, want: np.ndarray, dtype, what=""):
    max_abs, mean_rel = TOL[dtype]
    assert got.shape == want.shape, (what, got.shape, want.shape)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.isfinite(got).all(), f"{what}: non-finite values"
    assert err.max() <= max_abs, f"{what}: max-abs {err.max():.3e} > {max_abs}"
    denom = np.abs(want).mean()
    if denom > 0:
        assert err.mean() / denom <= mean_rel, f"{what}: mean-rel {err.mean() / denom:.3e} > {mean_rel}"


@pytest.fixture(autouse=True)
def _health():
    yield
    nb.device_health(DEV)   # turns a silent bounded-wait abort into a test failure


def _path(q, k, v, nheads):
    """Which kernel family the library picks for these tensors."""
    p = _lib.AttnParams()
    p.dtype = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[q.dtype]
    p.H = nheads
    p.d, p.dv = q.shape[0] // nheads, v.shape[0] // nheads
    p.Lq, p.Lkv, p.B = q.shape[1], k.shape[1], q.shape[2]
    x = nb.jl_empty((v.shape[0], q.shape[1], q.shape[2]), q.dtype, q.device)
    p.q, p.k, p.v, p.x = q.data_ptr(), k.data_ptr(), v.data_ptr(), x.data_ptr()
    return _lib.load().nnlib_b200_attn_path(p)


# --------------------------------------------------------------------------
# the reference's own tests, run on the device
# --------------------------------------------------------------------------

def test_specific_results(golden):
    # test/attention.jl:25-34 on the device (Float32 → CUDA-core kernel)
    g = golden["attention_specific"]
    qn = np.arange(1, 13, dtype=np.float32).reshape(g["q_shape"], order="F") / 12
    q = _dev(qn, torch.float32)
    y, a = nb.dot_product_attention(q, q, q, nheads=2)
    ytrue = np.array(g["ytrue_colmajor"]).reshape(g["ytrue_shape"], order="F")
    atrue = np.array(g["alphatrue_colmajor"]).reshape(g["alphatrue_shape"], order="F")
    np.testing.assert_allclose(nb.jl_to_numpy(y), ytrue, atol=1e-5, rtol=0)
    np.testing.assert_allclose(np.asarray(a), atrue, atol=1e-5, rtol=0)


@pytest.mark.parametrize("batch_size", [(), (1,), (2,), (2, 1, 3)])
@pytest.mark.parametrize("nheads", [1, 3, 5])
def test_compare_cpu_gpu_small(batch_size, nheads):
    # test/ext_amdgpu/attention.jl:1-23 (CPU vs device, atol 1f-5) and test/attention.jl:1-15
    rng = np.random.default_rng(10)
    n, lenq, lenkv = 15, 3, 4
    qn = rng.random((n, lenq) + batch_size, dtype=np.float32)
    kn = rng.random((n, lenkv) + batch_size, dtype=np.float32)
    vn = rng.random((n, lenkv) + batch_size, dtype=np.float32)
    y, a = nb.dot_product_attention(_dev(qn, torch.float32), _dev(kn, torch.float32), _dev(vn, torch.float32),
                                    nheads=nheads)
    assert y.is_cuda and y.dtype == torch.float32
    assert tuple(y.shape) == (n, lenq) + batch_size
    assert tuple(a.shape) == (lenkv, lenq, nheads) + batch_size
    an = np.asarray(a)
    np.testing.assert_allclose(an.sum(0), np.ones((lenq, nheads) + batch_size), rtol=1e-5)
    yo, ao = O.dot_product_attention(qn, kn, vn, nheads=nheads)
    np.testing.assert_allclose(nb.jl_to_numpy(y), yo, atol=1e-5, rtol=0)
    np.testing.assert_allclose(an, ao, atol=1e-5, rtol=0)


def test_scores_4d_matches_3d_entry():
    # test/attention.jl:17-23
    qn = np.arange(1, 25, dtype=np.float32).reshape((4, 2, 3, 1), order="F") / 24
    q4 = _dev(qn, torch.float32)
    a = nb.dot_product_attention_scores(q4, q4)
    q3 = nb.jl_reshape(q4, (8, 3, 1))
    _, a2 = nb.dot_product_attention(q3, q3, q3, nheads=2)
    np.testing.assert_allclose(nb.jl_to_numpy(a), np.asarray(a2), atol=1e-6)
    np.testing.assert_allclose(nb.jl_to_numpy(a), O.dot_product_attention_scores(qn, qn), atol=1e-5)


def test_mask_and_causal_support():
    # test/attention.jl:36-52 and test/ext_amdgpu/attention.jl:25-34
    rng = np.random.default_rng(11)
    qn = rng.random((4, 2, 3, 1), dtype=np.float32)
    kn = rng.random((4, 2, 5, 1), dtype=np.float32)
    mask = rng.random((5, 3)) > 0.5
    mask[0] = True
    a = nb.jl_to_numpy(nb.dot_product_attention_scores(
        _dev(qn, torch.float32), _dev(kn, torch.float32), mask=nb.jl_from_numpy(mask, device=DEV)))
    assert ((a[:, :, 0, 0] > 0) == mask).all() and ((a[:, :, 1, 0] > 0) == mask).all()
    x = _dev(rng.random((4, 2, 3, 1), dtype=np.float32), torch.float32)
    cm = nb.make_causal_mask(x, dims=3)
    assert cm.is_cuda and cm.dtype == torch.bool and tuple(cm.shape) == (3, 3)
    cmn = cm.cpu().numpy()
    assert (cmn == O.make_causal_mask(np.zeros((4, 2, 3, 1)), dims=3)).all()
    a = nb.jl_to_numpy(nb.dot_product_attention_scores(x, x, mask=cm))
    assert ((a[:, :, 0, 0] > 0) == cmn).all() and ((a[:, :, 1, 0] > 0) == cmn).all()
    # a hand-made copy of the causal matrix is detected by content, a different matrix is not
    cm2 = nb.jl_from_numpy(cmn, device=DEV)
    a2 = nb.jl_to_numpy(nb.dot_product_attention_scores(x, x, mask=cm2))
    np.testing.assert_array_equal(a, a2)


def test_dropout_with_opaque_fdrop():
    # test/attention.jl:54-59: an arbitrary callable; returned α is post-dropout and x = V·α′
    rng = np.random.default_rng(12)
    qn = rng.random((10, 10, 10), dtype=np.float32)
    q = _dev(qn, torch.float32)
    fdrop = lambda a: (torch.rand_like(a) > 0.5) * a / (1 - 0.5)
    y, a = nb.dot_product_attention(q, q, q, nheads=2, fdrop=fdrop)
    an = nb.jl_to_numpy(a)
    assert 0.4 < (an > 0).mean() < 0.6
    v4 = O.split_heads(qn, 2)
    x4 = O.batched_mul(np.transpose(v4, (0, 2, 1, 3)), an)
    np.testing.assert_allclose(nb.jl_to_numpy(y), O.join_heads(np.transpose(x4, (0, 2, 1, 3))), atol=1e-5)


def test_bias_shapes():
    # test/attention.jl:61-68
    rng = np.random.default_rng(13)
    qn = rng.random((4, 5, 1), dtype=np.float32); kn = rng.random((4, 3, 1), dtype=np.float32)
    bn = rng.standard_normal((3, 5)).astype(np.float32)
    y, a = nb.dot_product_attention(_dev(qn, torch.float32), _dev(kn, torch.float32), _dev(kn, torch.float32),
                                    _dev(bn, torch.float32), nheads=2)
    assert tuple(a.shape) == (3, 5, 2, 1) and tuple(y.shape) == (4, 5, 1)
    yo, ao = O.dot_product_attention(qn, kn, kn, bn, nheads=2)
    np.testing.assert_allclose(nb.jl_to_numpy(y), yo, atol=1e-5)
    np.testing.assert_allclose(np.asarray(a), ao, atol=1e-5)


def test_argument_errors_on_device():
    z = lambda *s: nb.jl_zeros(s, torch.float32, DEV)
    with pytest.raises(nb.ArgumentError, match="divisible"):
        nb.dot_product_attention(z(6, 2, 1), z(6, 2, 1), z(6, 2, 1), nheads=4)
    with pytest.raises(nb.ArgumentError, match="Batch"):
        nb.dot_product_attention(z(4, 2, 1), z(4, 2, 2), z(4, 2, 2))
    with pytest.raises(nb.ArgumentError, match="query and key"):
        nb.dot_product_attention(z(4, 2, 1), z(6, 2, 1), z(6, 2, 1))
    with pytest.raises(nb.ArgumentError, match="key and value"):
        nb.dot_product_attention(z(4, 2, 1), z(4, 3, 1), z(4, 2, 1))
    with pytest.raises(TypeError):
        nb.dot_product_attention(z(4, 2, 1).cpu(), z(4, 2, 1), z(4, 2, 1))


def test_fully_masked_query_is_nan():
    rng = np.random.default_rng(14)
    for dtype, E, nheads in ((torch.float32, 8, 2), (torch.bfloat16, 128, 2)):
        qn = rng.standard_normal((E, 130, 1)).astype(np.float32)
        kn = rng.standard_normal((E, 140, 1)).astype(np.float32)
        mask = np.ones((140, 130), dtype=bool); mask[:, 5] = False; mask[:, 129] = False
        y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(kn, dtype),
                                        mask=nb.jl_from_numpy(mask, device=DEV), nheads=nheads)
        yn, an = nb.jl_to_numpy(y), np.asarray(a)
        assert np.isnan(yn[:, 5]).all() and np.isnan(yn[:, 129]).all() and np.isfinite(yn[:, 6]).all()
        assert np.isnan(an[:, 5]).all() and np.isfinite(an[:, 4]).all()


# --------------------------------------------------------------------------
# tensor-core path vs oracle on ragged and benchmark shapes
# --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype,d,Lkv", [
    (torch.bfloat16, 64, 304),     # bias rows 16-byte aligned: tiles of the bias staged by TMA
    (torch.float16, 64, 300),      # per-thread bias loads
    (torch.float16, 128, 304),
    (torch.float32, 32, 300),      # CUDA-core kernels
])
def test_plus_inf_and_nan_logits_follow_the_reference_softmax(dtype, d, Lkv):
    """src/softmax.jl:71-76 through attention: a +Inf bias means "always attend here" (equal shares on the
    +Inf keys, also when the first one shows up in a later key tile than finite logits did, and not on a
    key the mask removes); a NaN bias makes the query's scores and output NaN."""
    rng = np.random.default_rng(31)
    H, Lq, B = 2, 150, 1
    E = d * H
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    bn = _round_to(0.5 * rng.standard_normal((Lkv, Lq, H, B)), dtype)
    bn[2, 0] = np.inf                      # one key, first tile
    bn[[1, 290], 1] = np.inf               # two keys, first and last tile
    bn[200, 5] = np.inf                    # appears after a tile of finite logits
    bn[[3, 130, 131, 299], 140] = np.inf   # second query tile
    bn[7, 6] = np.inf                      # on a masked key: the mask wins
    bn[10, 9] = np.nan
    mask = np.ones((Lkv, Lq), dtype=bool)
    mask[7, 6] = False
    q, k, v, b = (_dev(a, dtype) for a in (qn, kn, vn, bn))
    m = nb.jl_from_numpy(mask, device=DEV)
    y, a = nb.dot_product_attention(q, k, v, b, mask=m, nheads=H)
    yo, ao = O.dot_product_attention(qn, kn, vn, bn, mask=mask, nheads=H)
    yn, an = nb.jl_to_numpy(y), np.asarray(a)
    assert np.isnan(an[:, 9]).all() and np.isnan(ao[:, 9]).all()
    for h in range(H):
        assert np.isnan(yn[h * d:(h + 1) * d, 9]).all()
        np.testing.assert_array_equal(an[:, 0, h, 0], ao[:, 0, h, 0])          # exactly one-hot
        np.testing.assert_array_equal(an[:, 1, h, 0], ao[:, 1, h, 0])          # exactly 0.5 / 0.5
        np.testing.assert_array_equal(an[:, 5, h, 0], ao[:, 5, h, 0])
        np.testing.assert_array_equal(an[:, 140, h, 0], ao[:, 140, h, 0])      # 0.25 each
        assert an[7, 6, h, 0] == 0
    ok = np.ones(Lq, dtype=bool); ok[9] = False
    _close(yn[:, ok], yo[:, ok], dtype, "x")
    _close(an[:, ok], ao[:, ok], dtype, "alpha")
    # the scores-only entry (statistics kernel + scores kernel)
    q4, k4 = (nb.jl_reshape(t, (d, H, t.shape[1], B)) for t in (q, k))
    a2 = nb.jl_to_numpy(nb.dot_product_attention_scores(q4, k4, b, mask=m))
    np.testing.assert_array_equal(np.isnan(a2), np.isnan(an))
    np.testing.assert_array_equal(a2[:, [0, 1, 5, 140]], an[:, [0, 1, 5, 140]])
    _close(a2[:, ok], ao[:, ok], dtype, "alpha (scores entry)")


def _run_case(dtype, E, nheads, Lq, Lkv, B, *, causal=False, mask=None, bias=None, Ev=None, seed=0,
              expect_umma=True, check_alpha=True):
    rng = np.random.default_rng(seed)
    Ev = Ev or E
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((Ev, Lkv, B)), dtype)
    q, k, v = _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype)
    if expect_umma is not None:
        want_path = {True: _lib.PATH_UMMA, False: _lib.PATH_SIMT}.get(expect_umma, expect_umma)
        assert _path(q, k, v, nheads) == want_path
    mask_np = None
    mask_arg = None
    if causal:
        mask_np = O.make_causal_mask(np.zeros((1, Lq)), dims=2)
        mask_arg = nb.make_causal_mask(q, dims=2)
    elif mask is not None:
        mask_np = mask
        mask_arg = nb.jl_from_numpy(mask, device=DEV)
    bias_np = None
    bias_arg = None
    if bias is not None:
        bias_np = _round_to(bias, dtype)
        bias_arg = _dev(bias_np, dtype)
    y, a = nb.dot_product_attention(q, k, v, bias_arg, mask=mask_arg, nheads=nheads)
    yo, ao = O.dot_product_attention(qn, kn, vn, bias_np, mask=mask_np, nheads=nheads)
    _close(nb.jl_to_numpy(y), yo, dtype, "x")
    if check_alpha:
        an = np.asarray(a)
        _close(an, ao, dtype, "alpha")
        if mask_np is not None:
            keep = np.broadcast_to(O._bcast_to_scores(mask_np), ao.shape)
            assert (an[~keep] == 0).all(), "masked scores must be exactly 0"
        np.testing.assert_allclose(an.sum(0), 1.0, atol=1e-2)
    return y, a


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d", [64, 128])
def test_umma_plain_single_tile(dtype, d):
    _run_case(dtype, d, 1, 128, 128, 1, seed=20)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d,H,Lq,Lkv,B", [
    (64, 2, 256, 256, 2),      # two query tiles, two kv tiles
    (128, 2, 384, 512, 1),     # second CTA has one live tile only
    (128, 1, 100, 200, 2),     # ragged in both directions
    (64, 3, 257, 129, 1),      # one row / one key past a tile boundary
    (128, 2, 1, 1, 1),         # smallest
    (64, 1, 700, 1500, 1),     # many kv tiles: pipeline wraps around
    (128, 4, 1, 2000, 2),      # decode-like: one query against a long key sequence
    (64, 2, 5, 777, 3),
])
def test_umma_shapes(dtype, d, H, Lq, Lkv, B):
    _run_case(dtype, d * H, H, Lq, Lkv, B, seed=21)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d,H,L,B", [(64, 2, 128, 1), (128, 2, 256, 2), (128, 1, 300, 1), (64, 1, 1000, 1)])
def test_umma_causal(dtype, d, H, L, B):
    _run_case(dtype, d * H, H, L, L, B, causal=True, seed=22)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_umma_key_padding_mask(dtype):
    # BASELINE config 2 in small: (kv_len, 1, 1, B) Bool mask with per-sample valid lengths
    rng = np.random.default_rng(23)
    Lkv, B = 384, 3
    lens = rng.integers(Lkv // 2, Lkv + 1, size=B)
    mask = (np.arange(Lkv)[:, None, None, None] < lens[None, None, None, :])
    _run_case(dtype, 128, 2, 300, Lkv, B, mask=mask, seed=23)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bias_shape", [(200, 150, 2, 2), (200, 150), (200, 1, 2, 1), (1, 150, 1, 2)])
def test_umma_bias_broadcast(dtype, bias_shape):
    rng = np.random.default_rng(24)
    bias = (0.5 * rng.standard_normal(bias_shape)).astype(np.float32)
    _run_case(dtype, 128, 2, 150, 200, 2, bias=bias, seed=24)


def test_umma_random_mask_and_bias():
    rng = np.random.default_rng(25)
    mask = rng.random((260, 130, 2, 2)) > 0.3
    mask[0] = True
    bias = rng.standard_normal((260, 130, 1, 1)).astype(np.float32)
    _run_case(torch.bfloat16, 256, 2, 130, 260, 2, mask=mask, bias=bias, seed=25)


def test_simt_matches_oracle_for_other_shapes():
    # shapes the tensor-core kernels do not take run on the CUDA-core kernels
    _run_case(torch.float32, 96, 3, 70, 90, 2, seed=26, expect_umma=False)
    _run_case(torch.bfloat16, 84, 2, 70, 90, 2, seed=27, expect_umma=False)       # d = 42: not a multiple of 8
    _run_case(torch.float16, 64, 1, 33, 65, 1, Ev=20, seed=28, expect_umma=False)  # dv = 20
    _run_case(torch.float32, 64, 2, 50, 50, 1, causal=True, seed=29, expect_umma=False)
    _run_case(torch.bfloat16, 528, 2, 40, 70, 1, seed=29, expect_umma=False)      # d = 264: beyond the tensor-core kernels


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d,dv,H,Lq,Lkv,B", [
    (32, 32, 2, 200, 264, 2),      # half a swizzle row of features
    (96, 96, 2, 130, 70, 1),       # one and a half
    (8, 8, 3, 64, 64, 1),          # smallest head the 16-byte rule allows
    (120, 40, 1, 257, 129, 2),     # dv != d, neither a power of two
    (64, 128, 2, 300, 500, 1),     # dv != d with the fused kernel's own sizes
    (128, 64, 2, 100, 1000, 1),
    (48, 72, 2, 1, 700, 2),        # decode-like
    (256, 256, 2, 200, 330, 1),    # the largest heads the tensor-core path takes (16-bit types)
    (192, 128, 2, 130, 260, 2),    # query / key heads wider than the value heads
    (160, 256, 1, 257, 129, 1),
    (64, 200, 2, 100, 300, 1),     # only the value heads are wide
    (256, 256, 2, 4, 2000, 1),     # few queries against many keys: the keys are split
])
def test_tile_kernel_other_head_sizes(dtype, d, dv, H, Lq, Lkv, B):
    """Head sizes other than 64 / 128 and value heads of another size than the query heads
    (src/attention.jl:21-23, docstring example :36, test/attention.jl:61-68) on the tensor cores: the
    one-tile kernels, forward and lazily rebuilt scores."""
    # d = dv up to 128 runs on the fused two-tile kernel (padded to 64 / 128), everything else here on the one-tile ones
    want = _lib.PATH_UMMA if (d == dv and d <= 128) else _lib.PATH_TILE
    _run_case(dtype, d * H, H, Lq, Lkv, B, Ev=dv * H, seed=70 + d, expect_umma=want)


@pytest.mark.parametrize("dtype,d,dv", [(torch.bfloat16, 96, 32), (torch.float16, 40, 72)])
def test_tile_kernel_masks_bias_dropout(dtype, d, dv):
    """Every option of the call on the one-tile kernels: causal, key-padding and full masks, bias in
    broadcast forms, Philox dropout (mask compared bit for bit), and the scores-only entry."""
    rng = np.random.default_rng(71)
    H, Lq, Lkv, B = 2, 150, 150, 2
    _run_case(dtype, d * H, H, Lq, Lq, B, Ev=dv * H, causal=True, seed=72, expect_umma=_lib.PATH_TILE)
    keypad = rng.random((Lkv, 1, 1, B)) > 0.3
    keypad[0] = True
    _run_case(dtype, d * H, H, Lq, Lkv, B, Ev=dv * H, mask=keypad, seed=73, expect_umma=_lib.PATH_TILE)
    full = rng.random((Lkv, Lq, H, B)) > 0.3
    full[0] = True
    _run_case(dtype, d * H, H, Lq, Lkv, B, Ev=dv * H, mask=full, bias=0.5 * rng.standard_normal((Lkv, Lq, H, B)),
              seed=74, expect_umma=_lib.PATH_TILE)
    _run_case(dtype, d * H, H, Lq, Lkv, B, Ev=dv * H, bias=0.5 * rng.standard_normal((Lkv, 1, H)), seed=75,
              expect_umma=_lib.PATH_TILE)
    # dropout: exact mask, then values
    p = 0.25
    qn = _round_to(rng.standard_normal((d * H, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((d * H, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((dv * H, Lkv, B)), dtype)
    fd = nb.PhiloxDropout(p, seed=77, offset=3)
    y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), nheads=H, fdrop=fd)
    keep = P.keep_mask((Lkv, Lq, H, B), p, 77, 3)
    yo, ao = O.dot_product_attention(qn, kn, vn, nheads=H, fdrop=lambda al: al * keep / np.float32(1 - p))
    an = np.asarray(a)
    assert ((an > 0) == (keep & (ao > 0))).mean() > 0.9999
    _close(nb.jl_to_numpy(y), yo, dtype, "x with dropout")
    _close(an, ao, dtype, "alpha with dropout")
    # scores-only entry: statistics kernel + scores kernel
    q4, k4 = (nb.jl_reshape(_dev(t, dtype), (d, H, t.shape[1], B)) for t in (qn, kn))
    a2 = nb.jl_to_numpy(nb.dot_product_attention_scores(q4, k4, mask=nb.jl_from_numpy(keypad, device=DEV)))
    ao2 = O.dot_product_attention_scores(O.split_heads(qn, H), O.split_heads(kn, H), mask=keypad)
    _close(a2, ao2, dtype, "alpha (scores entry)")


@pytest.fixture
def eager_scores():
    nb.set_scores_mode("eager")
    yield
    nb.set_scores_mode("lazy")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("d,H,Lq,Lkv,B,kind", [
    (64, 3, 512, 512, 2, "keypad"),     # config 2's shape class: four key tiles in tensor memory
    (64, 2, 300, 264, 1, "plain"),      # ragged: a partial last key tile, a partial query tile
    (64, 2, 384, 384, 2, "causal"),     # key tiles above the diagonal are written as zeros
    (128, 2, 200, 256, 1, "plain"),     # d = 128: two key tiles
    (128, 1, 256, 256, 2, "causal"),
    (64, 2, 130, 512, 1, "bias"),       # bias, full mask and dropout
    (64, 1, 64, 8, 1, "plain"),         # a single short tile
    (40, 3, 200, 328, 2, "keypad"),     # a head narrower than the 64-feature box: the copy engine pads it
    (96, 2, 256, 256, 1, "causal"),     # between the two compiled sizes
    (72, 2, 256, 200, 2, "bias"),
    (8, 5, 130, 512, 1, "plain"),       # the smallest head
    (64, 12, 384, 384, 12, "keypad"),   # 432 work items: every CTA walks over three or more of them
    (64, 10, 320, 320, 16, "causal"),   # 480 items of unequal length
    (64, 6, 300, 512, 16, "rowmask"),   # a mask that depends on the query, several items per CTA
    (64, 4, 256, 128, 48, "dropout"),   # dropout alone: one item per CTA
])
def test_short_sequence_kernel_x_and_alpha_in_one_pass(eager_scores, dtype, d, H, Lq, Lkv, B, kind):
    """Eager scores for key sequences that fit one CTA's tensor memory: one kernel writes x and α
    (src/attention.jl:83 returns both), checked against the oracle with every option."""
    rng = np.random.default_rng(100 + Lq + Lkv)
    E = d * H
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    q, k, v = _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype)
    lib = _lib.load()
    mask_np = bias_np = None
    mask_arg = bias_arg = None
    fdrop, fdrop_o = nb.identity, (lambda al: al)
    if kind == "keypad":
        lens = rng.integers(Lkv // 2, Lkv + 1, size=B)
        mask_np = (np.arange(Lkv)[:, None, None, None] < lens[None, None, None, :])
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)
    elif kind == "causal":
        mask_np = O.make_causal_mask(qn)
        mask_arg = nb.make_causal_mask(q)
    elif kind == "rowmask":
        mask_np = rng.random((Lkv, Lq, 1, B)) > 0.3
        mask_np[0] = True
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)
    elif kind == "dropout":
        keep = P.keep_mask((Lkv, Lq, H, B), 0.25, 9, 2)
        fdrop = nb.PhiloxDropout(0.25, seed=9, offset=2)
        fdrop_o = lambda al: al * keep / np.float32(0.75)
    elif kind == "bias":
        bias_np = _round_to(0.5 * rng.standard_normal((Lkv, Lq, H, B)), dtype)
        bias_arg = _dev(bias_np, dtype)
        mask_np = rng.random((Lkv, Lq, 1, B)) > 0.25
        mask_np[0] = True
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)
        keep = P.keep_mask((Lkv, Lq, H, B), 0.2, 21, 4)
        fdrop = nb.PhiloxDropout(0.2, seed=21, offset=4)
        fdrop_o = lambda al: al * keep / np.float32(0.8)
    n0 = lib.nnlib_b200_launch_count()
    y, a = nb.dot_product_attention(q, k, v, bias_arg, mask=mask_arg, nheads=H, fdrop=fdrop)
    assert lib.nnlib_b200_launch_count() - n0 == 1, "x and alpha must come from one kernel"
    assert isinstance(a, torch.Tensor) and tuple(a.shape) == (Lkv, Lq, H, B)
    yo, ao = O.dot_product_attention(qn, kn, vn, bias_np, mask=mask_np, nheads=H, fdrop=fdrop_o)
    an = nb.jl_to_numpy(a)
    _close(nb.jl_to_numpy(y), yo, dtype, "x")
    _close(an, ao, dtype, "alpha")
    if mask_np is not None:
        keepm = np.broadcast_to(O._bcast_to_scores(mask_np), ao.shape)
        assert (an[~keepm] == 0).all(), "masked scores must be exactly 0"
    if kind not in ("bias", "dropout"):
        np.testing.assert_allclose(an.sum(0), 1.0, atol=1e-2)


def test_eager_scores_on_longer_sequences_use_the_two_kernels(eager_scores):
    dtype = torch.bfloat16
    rng = np.random.default_rng(101)
    E, H, Lq, Lkv, B = 128, 2, 100, 700, 1
    qn, kn, vn = (_round_to(rng.standard_normal((E, L, B)), dtype) for L in (Lq, Lkv, Lkv))
    lib = _lib.load()
    n0 = lib.nnlib_b200_launch_count()
    y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), nheads=H)
    assert lib.nnlib_b200_launch_count() - n0 == 2
    yo, ao = O.dot_product_attention(qn, kn, vn, nheads=H)
    _close(nb.jl_to_numpy(y), yo, dtype, "x")
    _close(nb.jl_to_numpy(a), ao, dtype, "alpha")


@pytest.mark.parametrize("seed", range(80))
def test_random_configurations_match_the_oracle(seed):
    """Seeded random draws over everything the public call accepts — element type, head size (any, not only
    the tensor-core ones), dv != d, heads, ragged lengths, batch, mask form (none / causal matrix / offset /
    key padding / random Bool array with any broadcast shape), bias broadcast shape, Philox dropout, lazy or
    eager scores — whichever kernel family the library picks.  x and alpha against the oracle."""
    rng = np.random.default_rng(7000 + seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    d = int(rng.choice([8, 16, 24, 40, 64, 64, 72, 96, 128, 128, 20, 33, 192, 256]))
    dv = d if rng.random() < 0.6 else int(rng.choice([8, 32, 64, 128, 48, 256, 160]))
    H = int(rng.integers(1, 5))
    lmax = 330 if seed < 48 else 900                       # the later seeds walk the copy rings around several times
    Lq, Lkv = int(rng.integers(1, lmax)), int(rng.integers(1, lmax))
    if rng.random() < 0.25:
        Lkv = int(rng.choice([64, 128, 256, 264]))        # sizes the short-sequence kernel takes
    B = int(rng.integers(1, 4))
    E, Ev = d * H, dv * H
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((Ev, Lkv, B)), dtype)
    q, k, v = _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype)

    mask_np = mask_arg = None
    kind = str(rng.choice(["none", "causal", "offset", "keypad", "random", "random"]))
    if kind == "causal" and Lq == Lkv:
        mask_np, mask_arg = O.make_causal_mask(qn), nb.make_causal_mask(q)
    elif kind in ("causal", "offset"):
        off = int(rng.integers(0, max(1, Lkv)))            # key 0 stays visible to every query
        mask_np, mask_arg = _offset_mask(Lkv, Lq, off), nb.CausalMask(off)
    elif kind == "keypad":
        lens = rng.integers(1, Lkv + 1, size=B)
        mask_np = np.arange(Lkv)[:, None, None, None] < lens[None, None, None, :]
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)
    elif kind == "random":
        shape = [(Lkv, Lq), (Lkv, Lq, 1, B), (Lkv, Lq, H, B), (Lkv, 1, H, 1), (Lkv, Lq, H)][int(rng.integers(0, 5))]
        mask_np = rng.random(shape) > 0.3
        mask_np[0] = True                                   # nobody is left without a key
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)

    bias_np = bias_arg = None
    if rng.random() < 0.4:
        shape = [(Lkv, Lq, H, B), (Lkv, Lq), (Lkv, 1, 1, B), (1, Lq, H, 1), (Lkv, Lq, H)][int(rng.integers(0, 5))]
        bias_np = _round_to(0.5 * rng.standard_normal(shape), dtype)
        bias_arg = _dev(bias_np, dtype)

    fdrop, fdrop_o, p_drop = nb.identity, (lambda al: al), 0.0
    if rng.random() < 0.3:
        p_drop, dseed, doff = float(rng.choice([0.1, 0.25, 0.5])), int(rng.integers(0, 2 ** 31)), int(rng.integers(0, 1000))
        keep = P.keep_mask((Lkv, Lq, H, B), p_drop, dseed, doff)
        fdrop = nb.PhiloxDropout(p_drop, seed=dseed, offset=doff)
        fdrop_o = lambda al: al * keep / np.float32(1.0 - p_drop)

    eager = rng.random() < 0.5
    fast = dtype == torch.float32 and rng.random() < 0.5       # Float32 on the tensor cores (TF32 operands)
    nb.set_scores_mode("eager" if eager else "lazy")
    nb.set_math_mode("fast" if fast else "default")
    try:
        y, a = nb.dot_product_attention(q, k, v, bias_arg, mask=mask_arg, nheads=H, fdrop=fdrop)
        an = nb.jl_to_numpy(a) if isinstance(a, torch.Tensor) else np.asarray(a)
    finally:
        nb.set_scores_mode("lazy")
        nb.set_math_mode("default")
    yo, ao = O.dot_product_attention(qn, kn, vn, bias_np, mask=mask_np, nheads=H, fdrop=fdrop_o)
    what = f"seed {seed}: {dtype} d={d} dv={dv} H={H} Lq={Lq} Lkv={Lkv} B={B} mask={kind} bias={None if bias_np is None else bias_np.shape} p={p_drop} eager={eager} tf32={fast}"
    assert tuple(y.shape) == (Ev, Lq, B) and an.shape == (Lkv, Lq, H, B), what
    if fast:
        _close_tf32(nb.jl_to_numpy(y), yo, "x, " + what)
        _close_tf32(an, ao, "alpha, " + what)
    else:
        _close(nb.jl_to_numpy(y), yo, dtype, "x, " + what)
        _close(an, ao, dtype, "alpha, " + what)
    if mask_np is not None:
        keepm = np.broadcast_to(O._bcast_to_scores(mask_np), ao.shape)
        assert (an[~keepm] == 0).all(), "masked scores must be exactly 0, " + what
    if p_drop == 0.0:
        np.testing.assert_allclose(an.sum(0), 1.0, atol=1e-2, err_msg=what)


def _offset_mask(Lkv, Lq, off):
    """the Bool matrix the reference would be handed for `key <= query + off`"""
    return np.arange(Lkv)[:, None] <= (np.arange(Lq)[None, :] + off)


@pytest.mark.parametrize("dtype,d,Lq,Lkv,off", [
    (torch.bfloat16, 128, 300, 500, 200),     # two-tile fused kernel; last query sees the last key
    (torch.float16, 64, 300, 500, 37),
    (torch.bfloat16, 128, 260, 400, -140),    # negative: the first 140 queries see no key at all (NaN like the reference)
    (torch.bfloat16, 96, 200, 333, 133),      # one-tile kernels
    (torch.float32, 48, 70, 100, 30),         # CUDA-core kernels
])
def test_causal_offset_matches_an_explicit_mask(dtype, d, Lq, Lkv, off):
    """CausalMask(offset) — key j visible to query i iff j <= i + offset — against the oracle fed the same
    pattern as a Bool matrix, x and α, on every forward kernel family."""
    rng = np.random.default_rng(80 + d)
    H, B = 2, 2
    qn = _round_to(rng.standard_normal((d * H, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((d * H, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((d * H, Lkv, B)), dtype)
    mask = _offset_mask(Lkv, Lq, off)
    y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), mask=nb.CausalMask(off), nheads=H)
    with np.errstate(invalid="ignore"):
        yo, ao = O.dot_product_attention(qn, kn, vn, mask=mask, nheads=H)
    yn, an = nb.jl_to_numpy(y), np.asarray(a)
    live = mask.any(axis=0)
    assert np.isnan(yn[:, ~live]).all() and np.isnan(an[:, ~live]).all()       # nothing to attend to
    _close(yn[:, live], yo[:, live], dtype, "x")
    _close(an[:, live], ao[:, live], dtype, "alpha")
    assert (an[:, live][~mask[:, live]] == 0).all()


@pytest.mark.parametrize("dtype,d,dv,H,B,Lq,Lkv", [
    (torch.bfloat16, 128, 128, 2, 1, 1, 5000),      # one new token, two units: 148 SMs would see two CTAs
    (torch.float16, 64, 64, 4, 1, 5, 3000),
    (torch.bfloat16, 128, 128, 1, 2, 16, 4100),
    (torch.bfloat16, 96, 40, 2, 1, 128, 2500),      # a full query tile, other head sizes
])
def test_split_key_forward_for_few_queries(dtype, d, dv, H, B, Lq, Lkv):
    """Few queries against a long key / value history, aligned at the end (offset = Lkv - Lq): the keys of a
    unit are split over several CTAs and merged; x, the log-sum-exp (through α) and the options agree with
    the oracle."""
    rng = np.random.default_rng(90 + Lq)
    off = Lkv - Lq
    qn = _round_to(rng.standard_normal((d * H, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((d * H, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((dv * H, Lkv, B)), dtype)
    q, k, v = _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype)
    pr = nb.attention._Problem(q, k, v, None, nb.CausalMask(off), H, None, need_v=True)
    pr.alloc_x()
    assert _lib.load().nnlib_b200_attn_decode_workspace_bytes(pr.p) > 0
    mask = _offset_mask(Lkv, Lq, off)
    y, a = nb.dot_product_attention(q, k, v, mask=nb.CausalMask(off), nheads=H)
    yo, ao = O.dot_product_attention(qn, kn, vn, mask=mask, nheads=H)
    _close(nb.jl_to_numpy(y), yo, dtype, "x")
    _close(np.asarray(a), ao, dtype, "alpha")
    # with a key-padding mask, a bias and dropout on top
    keypad = rng.random((Lkv, 1, 1, B)) > 0.2
    keypad[-1] = True
    bn = _round_to(0.5 * rng.standard_normal((Lkv, Lq, H, 1)), dtype)
    pd = 0.2
    keep = P.keep_mask((Lkv, Lq, H, B), pd, 11, 2)
    y, a = nb.dot_product_attention(q, k, v, _dev(bn, dtype), mask=nb.jl_from_numpy(keypad, device=DEV), nheads=H,
                                    fdrop=nb.PhiloxDropout(pd, seed=11, offset=2))
    yo, ao = O.dot_product_attention(qn, kn, vn, bn, mask=keypad, nheads=H,
                                     fdrop=lambda al: al * keep / np.float32(1 - pd))
    _close(nb.jl_to_numpy(y), yo, dtype, "x with options")
    _close(np.asarray(a), ao, dtype, "alpha with options")


TF32_TOL = (3e-3, 1e-3)     # max-abs, mean-rel against the Float32 oracle: 10-bit mantissa operands


def _close_tf32(got, want, what):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.isfinite(got).all(), what
    assert err.max() <= TF32_TOL[0], f"{what}: max-abs {err.max():.3e}"
    assert err.mean() / np.abs(want).mean() <= TF32_TOL[1], f"{what}: mean-rel {err.mean() / np.abs(want).mean():.3e}"


@pytest.fixture
def fast_math():
    nb.set_math_mode("fast")
    yield
    nb.set_math_mode("default")


def test_tf32_path_config1_and_options(fast_math):
    """Float32 arrays in fast math mode run both products on the tensor cores with TF32 operands: BASELINE
    config 1 (E=512, nheads=8, L=128, batch=4, α returned) and a masked / biased / dropped-out case, inside
    max-abs 3e-3 and mean-rel 1e-3 of the Float32 oracle; without the switch the same call stays on the
    exact CUDA-core kernels."""
    rng = np.random.default_rng(1234)
    E, H, L, B = 512, 8, 128, 4
    qn, kn, vn = (rng.standard_normal((E, L, B), dtype=np.float32) for _ in range(3))
    q, k, v = (_dev(t, torch.float32) for t in (qn, kn, vn))
    p = _lib.AttnParams()
    p.dtype, p.d, p.dv, p.H, p.Lq, p.Lkv, p.B = _lib.F32, E // H, E // H, H, L, L, B
    x = nb.jl_empty((E, L, B), torch.float32, DEV)
    p.q, p.k, p.v, p.x = q.data_ptr(), k.data_ptr(), v.data_ptr(), x.data_ptr()
    assert _lib.load().nnlib_b200_attn_path(p) == _lib.PATH_SIMT
    p.allow_tf32 = 1
    assert _lib.load().nnlib_b200_attn_path(p) == _lib.PATH_TILE
    y, a = nb.dot_product_attention(q, k, v, nheads=H)
    yo, ao = O.dot_product_attention(qn, kn, vn, nheads=H)
    _close_tf32(nb.jl_to_numpy(y), yo, "x")
    _close_tf32(np.asarray(a), ao, "alpha")
    # options: d = 40, dv = 24, ragged lengths, full mask, bias, dropout
    d, dv, H, Lq, Lkv, B, pd = 40, 24, 2, 150, 200, 2, 0.2
    qn = rng.standard_normal((d * H, Lq, B), dtype=np.float32)
    kn = rng.standard_normal((d * H, Lkv, B), dtype=np.float32)
    vn = rng.standard_normal((dv * H, Lkv, B), dtype=np.float32)
    bn = (0.5 * rng.standard_normal((Lkv, Lq, H, B))).astype(np.float32)
    mask = rng.random((Lkv, Lq, 1, B)) > 0.3
    mask[0] = True
    keep = P.keep_mask((Lkv, Lq, H, B), pd, 9, 1)
    y, a = nb.dot_product_attention(_dev(qn, torch.float32), _dev(kn, torch.float32), _dev(vn, torch.float32),
                                    _dev(bn, torch.float32), mask=nb.jl_from_numpy(mask, device=DEV), nheads=H,
                                    fdrop=nb.PhiloxDropout(pd, seed=9, offset=1))
    yo, ao = O.dot_product_attention(qn, kn, vn, bn, mask=mask, nheads=H, fdrop=lambda al: al * keep / np.float32(1 - pd))
    _close_tf32(nb.jl_to_numpy(y), yo, "x with options")
    _close_tf32(np.asarray(a), ao, "alpha with options")


def test_tf32_path_config3_shape_row_sampled(fast_math):
    """A Float32 case of config 3's shape (E=4096, nheads=32, d=128, L=4096, causal; one batch element) on the
    TF32 path against the row-sampled Float64 oracle."""
    E, H, L, B = 4096, 32, 4096, 1
    g = torch.Generator(device=DEV).manual_seed(45)
    q, k, v = (nb.jl_empty((E, L, B), torch.float32, DEV) for _ in range(3))
    for t in (q, k, v):
        t.normal_(generator=g)
    y, a = nb.dot_product_attention(q, k, v, mask=nb.make_causal_mask(q), nheads=H)
    lse = a._problem.lse.cpu().numpy()
    qn, kn, vn, yn = (nb.jl_to_numpy(t) for t in (q, k, v, y))
    d = E // H
    rows = _sample_rows(L)
    for (b, h) in [(0, 0), (0, 31)]:
        xr, ar, lr = O.attention_rows(qn, kn, vn, H, rows, b, h, causal=True)
        _close_tf32(yn[h * d:(h + 1) * d][:, rows, b], xr.astype(np.float32), f"x rows of unit {(b, h)}")
        np.testing.assert_allclose(lse[rows, h, b], lr, atol=5e-3)


def test_nd_batch_and_lazy_alpha():
    rng = np.random.default_rng(30)
    dtype = torch.bfloat16
    qn = _round_to(rng.standard_normal((128, 130, 2, 1, 3)), dtype)
    q = _dev(qn, dtype)
    y, a = nb.dot_product_attention(q, q, q, nheads=2)
    assert isinstance(a, nb.LazyAttnScores) and not a.is_materialized
    assert tuple(y.shape) == (128, 130, 2, 1, 3) and tuple(a.shape) == (130, 130, 2, 2, 1, 3)
    yo, ao = O.dot_product_attention(qn, qn, qn, nheads=2)
    _close(nb.jl_to_numpy(y), yo, dtype, "x")
    _close(np.asarray(a), ao, dtype, "alpha")


# --------------------------------------------------------------------------
# fused Philox dropout
# --------------------------------------------------------------------------

@pytest.mark.parametrize("dtype,E,H", [(torch.float16, 128, 2), (torch.float32, 32, 2)])
def test_philox_dropout_exact_mask_and_values(dtype, E, H):
    rng = np.random.default_rng(31)
    Lq, Lkv, B, p, seed = 140, 270, 2, 0.1, 0xB200
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    fd = nb.PhiloxDropout(p, seed=seed, offset=3)
    y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), nheads=H, fdrop=fd)
    an = np.asarray(a)
    keep = P.keep_mask((Lkv, Lq, H, B), p, seed, offset=3)
    _, a0 = O.dot_product_attention(qn, kn, vn, nheads=H)
    assert abs(keep.mean() - (1 - p)) < 0.01
    # the device drew exactly the oracle's mask (scores are > 0 everywhere before dropout)
    assert ((an > 0) == keep).all()
    want_a = a0 * keep / np.float32(1 - p)
    _close(an, want_a.astype(np.float32), dtype, "alpha'")
    # x equals V·α′ for that mask
    fdrop_o = lambda al: al * keep / np.float32(1 - p)
    yo, _ = O.dot_product_attention(qn, kn, vn, nheads=H, fdrop=fdrop_o)
    _close(nb.jl_to_numpy(y), yo, dtype, "x")
    # a second object with the same (p, seed, offset) reproduces the call; the next offset differs
    y2, _ = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), nheads=H,
                                     fdrop=nb.PhiloxDropout(p, seed=seed, offset=3))
    assert torch.equal(y, y2)
    y3, _ = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), nheads=H, fdrop=fd)
    assert not torch.equal(y, y3)


def test_philox_dropout_rate_like_reference():
    # test/attention.jl:54-59 with the fused fdrop
    rng = np.random.default_rng(32)
    q = _dev(rng.random((128, 64, 10), dtype=np.float32), torch.bfloat16)
    y, a = nb.dot_product_attention(q, q, q, nheads=2, fdrop=nb.PhiloxDropout(0.5, seed=1))
    frac = (np.asarray(a) > 0).mean()
    assert 0.4 < frac < 0.6


# --------------------------------------------------------------------------
# raw C-ABI: strides, separate entry points, status word
# --------------------------------------------------------------------------

def test_abi_strided_head_slice_and_entry_points():
    """A shard that owns heads 1..2 of 4 addresses the parent arrays through
    pointer offsets and the parent's strides (no copy), and the four entry
    points agree with each other."""
    import ctypes as C
    lib = _lib.load()
    rng = np.random.default_rng(33)
    dtype = torch.bfloat16
    H, d, Lq, Lkv, B = 4, 64, 200, 333, 2
    E = H * d
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    q, k, v = _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype)
    x = nb.jl_zeros((E, Lq, B), dtype, DEV)
    h0, Hs = 1, 2
    lse = torch.empty((B, Hs, Lq), dtype=torch.float32, device=DEV)
    alpha = nb.jl_empty((Lkv, Lq, Hs, B), dtype, DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    p = _lib.AttnParams()
    p.dtype = _lib.BF16
    p.d, p.dv, p.H, p.Lq, p.Lkv, p.B = d, d, Hs, Lq, Lkv, B
    off = h0 * d * 2
    p.q, p.k, p.v, p.x = q.data_ptr() + off, k.data_ptr() + off, v.data_ptr() + off, x.data_ptr() + off
    p.q_stride_l = p.k_stride_l = p.v_stride_l = p.x_stride_l = E
    p.q_stride_b, p.x_stride_b = E * Lq, E * Lq
    p.k_stride_b = p.v_stride_b = E * Lkv
    p.lse, p.alpha, p.status = lse.data_ptr(), alpha.data_ptr(), status.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.nnlib_b200_attn_path(p) == _lib.PATH_UMMA
    assert lib.nnlib_b200_attn_fwd(C.byref(p), st) == 0
    assert lib.nnlib_b200_attn_scores(C.byref(p), st) == 0
    lse2 = torch.empty_like(lse)
    p.lse = lse2.data_ptr()
    assert lib.nnlib_b200_attn_stats(C.byref(p), st) == 0
    x2 = nb.jl_zeros((E, Lq, B), dtype, DEV)
    p.x = x2.data_ptr() + off
    assert lib.nnlib_b200_attn_apply(C.byref(p), st) == 0
    torch.cuda.synchronize()
    assert status.item() == 0
    yo, ao = O.dot_product_attention(qn, kn, vn, nheads=H)
    xs = nb.jl_to_numpy(x)
    _close(xs[h0 * d:(h0 + Hs) * d], yo[h0 * d:(h0 + Hs) * d], dtype, "x shard")
    assert (xs[:h0 * d] == 0).all() and (xs[(h0 + Hs) * d:] == 0).all(), "wrote outside the shard"
    _close(nb.jl_to_numpy(alpha), ao[:, :, h0:h0 + Hs], dtype, "alpha shard")
    np.testing.assert_allclose(lse.cpu().numpy(), lse2.cpu().numpy(), atol=2e-3)
    # lse is the natural-log sum of exponentials of the scaled logits
    logits = np.einsum("ehjb,ehib->jihb", O.split_heads(kn, H), O.split_heads(qn, H)) / math.sqrt(d)
    want_lse = np.log(np.exp(logits - logits.max(0)).sum(0)) + logits.max(0)        # (Lq, H, B)
    np.testing.assert_allclose(lse.cpu().numpy().transpose(2, 1, 0), want_lse[:, h0:h0 + Hs], atol=2e-2)
    # attn_apply (x = V·α from the stored bf16 scores) agrees with the fused x
    _close(nb.jl_to_numpy(x2)[h0 * d:(h0 + Hs) * d], yo[h0 * d:(h0 + Hs) * d], dtype, "apply x")


def test_abi_attention_one_call_with_workspace():
    import ctypes as C
    lib = _lib.load()
    rng = np.random.default_rng(34)
    dtype = torch.float16
    H, d, L, B = 2, 128, 160, 1
    qn = _round_to(rng.standard_normal((H * d, L, B)), dtype)
    q = _dev(qn, dtype)
    x = nb.jl_empty((H * d, L, B), dtype, DEV)
    alpha = nb.jl_empty((L, L, H, B), dtype, DEV)
    p = _lib.AttnParams()
    p.dtype = _lib.F16
    p.d, p.dv, p.H, p.Lq, p.Lkv, p.B = d, d, H, L, L, B
    p.q = p.k = p.v = q.data_ptr()
    p.x, p.alpha = x.data_ptr(), alpha.data_ptr()
    p.causal = 1
    need = lib.nnlib_b200_workspace_bytes(C.byref(p))
    assert need == L * H * B * 4
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.nnlib_b200_attention(C.byref(p), ws.data_ptr(), need - 1, st) == _lib.WORKSPACE_TOO_SMALL
    assert lib.nnlib_b200_attention(C.byref(p), ws.data_ptr(), need, st) == 0
    torch.cuda.synchronize()
    yo, ao = O.dot_product_attention(qn, qn, qn, mask=O.make_causal_mask(qn), nheads=H)
    _close(nb.jl_to_numpy(x), yo, dtype, "x")
    _close(nb.jl_to_numpy(alpha), ao, dtype, "alpha")


def test_bounded_wait_runout_is_reported_and_the_device_stays_usable():
    """The fail-stop path end to end, without faulting or hanging anything: a self-test kernel waits with
    the library's bounded wait (limit 5 ms here) on a barrier nobody arrives at and returns by itself.
    Then: the status word says TIMEOUT; the device is marked, so a later tensor-core launch returns at
    once, leaves its output untouched and reports through ITS status word; the Python wrapper raises at
    its next synchronisation point; device_health reports the mark once and clears it; and the next
    ordinary call is correct again."""
    import ctypes as C
    lib = _lib.load()
    rng = np.random.default_rng(35)
    dtype, H, d, L, B = torch.bfloat16, 2, 64, 200, 1
    qn, kn, vn = (_round_to(rng.standard_normal((H * d, L, B)), dtype) for _ in range(3))
    q, k, v = (_dev(a, dtype) for a in (qn, kn, vn))
    st = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    t0 = time.perf_counter()
    assert lib.nnlib_b200_selftest_wait_runout(5_000_000, status.data_ptr(), st) == _lib.OK
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 2.0, "the wait did not run out by itself"
    assert status.item() == _lib.TIMEOUT
    try:
        # a launch on the marked device: skipped, output untouched, status word set
        x = nb.jl_empty((H * d, L, B), dtype, DEV)
        x.fill_(7.0)
        status2 = torch.zeros(1, dtype=torch.int32, device=DEV)
        p = _lib.AttnParams()
        p.dtype = _lib.BF16
        p.d, p.dv, p.H, p.Lq, p.Lkv, p.B = d, d, H, L, L, B
        p.q, p.k, p.v, p.x, p.status = q.data_ptr(), k.data_ptr(), v.data_ptr(), x.data_ptr(), status2.data_ptr()
        assert lib.nnlib_b200_attn_path(p) == _lib.PATH_UMMA
        assert lib.nnlib_b200_attn_fwd(C.byref(p), st) == _lib.OK
        torch.cuda.synchronize()
        assert status2.item() == _lib.TIMEOUT
        assert (x.float() == 7.0).all()
        # the wrapper passes its own status word and raises where it synchronises anyway
        y, _ = nb.dot_product_attention(q, k, v, nheads=H)
        with pytest.raises(_lib.NNlibB200Error) as ei:
            nb.check_status(DEV)
        assert ei.value.code == _lib.TIMEOUT
    finally:
        # reported once, then clear
        assert lib.nnlib_b200_device_health(st) == _lib.TIMEOUT
    assert lib.nnlib_b200_device_health(st) == _lib.OK
    nb.check_status(DEV)
    y, a = nb.dot_product_attention(q, k, v, nheads=H)
    yo, ao = O.dot_product_attention(qn, kn, vn, nheads=H)
    _close(nb.jl_to_numpy(y), yo, dtype, "x after the mark was cleared")
    _close(np.asarray(a), ao, dtype, "alpha after the mark was cleared")


def test_causal_check_kernel():
    import ctypes as C
    lib = _lib.load()
    L = 77
    m = nb.jl_empty((L, L), torch.bool, DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.nnlib_b200_causal_fill(m.view(torch.uint8).data_ptr(), L, st) == 0
    assert lib.nnlib_b200_causal_check(m.view(torch.uint8).data_ptr(), L, flag.data_ptr(), st) == 0
    assert flag.item() == 1
    m[5, 3] = True   # below the diagonal
    assert lib.nnlib_b200_causal_check(m.view(torch.uint8).data_ptr(), L, flag.data_ptr(), st) == 0
    assert flag.item() == 0


def test_causal_matrix_is_trusted_only_while_unmodified():
    """make_causal_mask's result selects the causal mode without being read — until somebody writes to it;
    any other square Bool matrix is read each time, so neither a modified matrix nor a new matrix that
    lands on a freed one's address is ever mistaken for the causal pattern."""
    rng = np.random.default_rng(30)
    dtype, E, H, L, B = torch.bfloat16, 128, 2, 160, 1
    qn, kn, vn = (_round_to(rng.standard_normal((E, L, B)), dtype) for _ in range(3))
    q, k, v = (_dev(a, dtype) for a in (qn, kn, vn))
    lib = _lib.load()

    def run(mask_dev, mask_np):
        n0 = lib.nnlib_b200_launch_count()
        y, _ = nb.dot_product_attention(q, k, v, mask=mask_dev, nheads=H)
        launches = lib.nnlib_b200_launch_count() - n0
        yo, _ = O.dot_product_attention(qn, kn, vn, mask=mask_np, nheads=H)
        _close(nb.jl_to_numpy(y), yo, dtype, "x")
        return launches

    # (1) fresh make_causal_mask result: one launch (the fused kernel), no check
    m = nb.make_causal_mask(q)
    assert run(m, O.make_causal_mask(qn)) == 1
    # (2) written to (version counter moves): read again, and the new contents count
    m[5, 2] = True                                   # key 5 visible to query 2
    mn = O.make_causal_mask(qn).copy(); mn[5, 2] = True
    assert run(m, mn) == 3                           # flag set + check + fused kernel
    # (3) a user-built causal matrix is checked on every call, also the second time
    tri = nb.jl_from_numpy(O.make_causal_mask(qn), device=DEV)
    assert run(tri, O.make_causal_mask(qn)) == 3
    assert run(tri, O.make_causal_mask(qn)) == 3
    # (4) free it and put a random matrix of the same size where it was
    addr = tri.data_ptr()
    del tri
    rn = rng.random((L, L)) > 0.3
    rn[0, :] = True
    rnd = nb.jl_from_numpy(rn, device=DEV)
    if rnd.data_ptr() != addr:
        pytest.skip("the allocator did not reuse the freed block")
    run(rnd, rn)


# --------------------------------------------------------------------------
# benchmark configurations (BASELINE.json configs 2-5), full size where the
# oracle finishes in seconds, otherwise row-sampled
# --------------------------------------------------------------------------

def _sample_rows(L):
    base = [0, 1, 127, 128, 129, 255, 256, L // 2, L - 129, L - 128, L - 2, L - 1]
    return np.array(sorted({r for r in base if 0 <= r < L}))


def _check_rows(q, k, v, y, lse, H, units, dtype, *, causal=False, mask=None, bias=None):
    qn, kn, vn = (nb.jl_to_numpy(t) for t in (q, k, v))
    yn = nb.jl_to_numpy(y)
    d = qn.shape[0] // H
    rows = _sample_rows(qn.shape[1])
    for (b, h) in units:
        xr, ar, lr = O.attention_rows(qn, kn, vn, H, rows, b, h, causal=causal, mask=mask, bias=bias)
        _close(yn[h * d:(h + 1) * d][:, rows, b], xr.astype(np.float32), dtype, f"x rows of unit {(b, h)}")
        if lse is not None:
            np.testing.assert_allclose(lse[rows, h, b], lr, atol=2e-2)


def test_config1_float32_exact():
    """BASELINE config 1 exactly: Float32, E=512, nheads=8 (d=64), Lq=Lkv=128, batch=4, no mask / bias,
    fdrop = identity, (x, α) returned with α of size (128, 128, 8, 4); whole oracle, atol 1e-5 like the
    reference's own CPU-vs-GPU tests (test/ext_amdgpu/attention.jl:19-21)."""
    rng = np.random.default_rng(1234)
    E, H, L, B = 512, 8, 128, 4
    qn, kn, vn = (rng.standard_normal((E, L, B), dtype=np.float32) for _ in range(3))
    y, a = nb.dot_product_attention(_dev(qn, torch.float32), _dev(kn, torch.float32), _dev(vn, torch.float32),
                                    nheads=H)
    yo, ao = O.dot_product_attention(qn, kn, vn, nheads=H)
    assert tuple(y.shape) == (E, L, B) and tuple(a.shape) == (L, L, H, B)
    np.testing.assert_allclose(nb.jl_to_numpy(y), yo, atol=1e-5, rtol=0)
    np.testing.assert_allclose(np.asarray(a), ao, atol=1e-5, rtol=0)


def test_config2_encoder_key_padding():
    # bf16, E=768, nheads=12, L=512, batch=32 → batch 8 here (same shape class), α returned
    rng = np.random.default_rng(40)
    dtype, E, H, L, B = torch.bfloat16, 768, 12, 512, 8
    lens = rng.integers(256, 513, size=B)
    mask = (np.arange(L)[:, None, None, None] < lens[None, None, None, :])
    _run_case(dtype, E, H, L, L, B, mask=mask, seed=40)


def test_config3_decoder_causal_row_sampled():
    # bf16, E=4096, nheads=32, L=4096, causal; batch 2 of the 8 (each batch is an independent unit set)
    dtype, E, H, L, B = torch.bfloat16, 4096, 32, 4096, 2
    g = torch.Generator(device=DEV).manual_seed(41)
    q, k, v = (nb.jl_empty((E, L, B), dtype, DEV) for _ in range(3))
    for t in (q, k, v):
        t.normal_(generator=g)
    y, a = nb.dot_product_attention(q, k, v, mask=nb.make_causal_mask(q), nheads=H)
    assert not a.is_materialized
    lse = a._problem.lse.cpu().numpy()
    _check_rows(q, k, v, y, lse, H, [(0, 0), (1, 31), (0, 17)], dtype, causal=True)


def test_config4_cross_attention_bias_dropout():
    # fp16 q (1024, 256, B), k/v (1024, 2048, B), nheads=16, bias (Lkv, Lq, H, B) ~ N(0, 0.5), p=0.1; B=2 of 16
    rng = np.random.default_rng(42)
    dtype, E, H, Lq, Lkv, B, p = torch.float16, 1024, 16, 256, 2048, 2, 0.1
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    bn = _round_to(0.5 * rng.standard_normal((Lkv, Lq, H, B)), dtype)
    fd = nb.PhiloxDropout(p, seed=0xB200, offset=0)
    y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), _dev(bn, dtype),
                                    nheads=H, fdrop=fd)
    keep = P.keep_mask((Lkv, Lq, H, B), p, 0xB200, 0)
    fdrop_o = lambda al: al * keep / np.float32(1 - p)
    yo, ao = O.dot_product_attention(qn, kn, vn, bn, nheads=H, fdrop=fdrop_o)
    _close(nb.jl_to_numpy(y), yo, dtype, "x")
    an = np.asarray(a)
    assert ((an > 0) == (keep & (ao > 0))).mean() > 0.9999   # f16 underflow may zero a few tiny scores
    _close(an, ao, dtype, "alpha'")


def test_config5_long_context_row_sampled():
    # bf16, E=2048, nheads=16, L=32768, causal; one batch of the 8
    dtype, E, H, L, B = torch.bfloat16, 2048, 16, 32768, 1
    g = torch.Generator(device=DEV).manual_seed(43)
    q, k, v = (nb.jl_empty((E, L, B), dtype, DEV) for _ in range(3))
    for t in (q, k, v):
        t.normal_(generator=g)
    y, a = nb.dot_product_attention(q, k, v, mask=nb.CausalMask(), nheads=H)
    lse = a._problem.lse.cpu().numpy()
    _check_rows(q, k, v, y, lse, H, [(0, 0), (0, 15)], dtype, causal=True)


def test_linearity_in_v_full_size():
    """Size-independent property at config-3 size: attention is linear in v, so
    x(v1 + v2) = x(v1) + x(v2) up to rounding, and x(v = const) = const."""
    dtype, E, H, L, B = torch.bfloat16, 4096, 32, 4096, 1
    g = torch.Generator(device=DEV).manual_seed(44)
    q, k = (nb.jl_empty((E, L, B), dtype, DEV) for _ in range(2))
    q.normal_(generator=g); k.normal_(generator=g)
    ones = nb.jl_empty((E, L, B), dtype, DEV); ones.fill_(1.0)
    y, _ = nb.dot_product_attention(q, k, ones, mask=nb.CausalMask(), nheads=H)
    assert (y.float() - 1).abs().max().item() <= 2e-2


# --------------------------------------------------------------------------
# multi-GPU driver on real devices (one host thread per entry of `devices`)
# --------------------------------------------------------------------------

def test_sharded_driver_on_device_matches_single_call():
    """Three shards (worker threads) over the visible GPUs — with one GPU they share it — so that the
    unit ranges cut through a batch: head-range rectangles, pointer-free slicing, and the dropout
    origin of each shard are exercised.  The sharded x must equal the unsharded call bit for bit."""
    from nnlib_jl_b200.shard import ShardedAttention
    ndev = torch.cuda.device_count()
    devices = [f"cuda:{i % ndev}" for i in range(3)]
    rng = np.random.default_rng(50)
    dtype, E, H, Lq, Lkv, B = torch.bfloat16, 256, 4, 200, 260, 2      # 8 units over 3 shards: 3 + 3 + 2
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    mask = rng.random((Lkv, 1, 1, B)) > 0.2
    mask[0] = True
    q, k, v = (nb.jl_from_numpy(a, dtype=dtype) for a in (qn, kn, vn))           # host arrays
    m_host = nb.jl_from_numpy(mask)
    drv = ShardedAttention(devices)
    x = drv(q, k, v, mask=m_host, nheads=H, fdrop=nb.PhiloxDropout(0.2, seed=5, offset=9))
    assert not x.is_cuda and tuple(x.shape) == (E, Lq, B)
    y, _ = nb.dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), mask=m_host.to(DEV), nheads=H,
                                    fdrop=nb.PhiloxDropout(0.2, seed=5, offset=9))
    assert torch.equal(x, y.cpu())
    keep = P.keep_mask((Lkv, Lq, H, B), 0.2, 5, 9)
    yo, _ = O.dot_product_attention(qn, kn, vn, mask=mask, nheads=H, fdrop=lambda a: a * keep / np.float32(0.8))
    _close(nb.jl_to_numpy(x), yo, dtype, "sharded x")


@pytest.mark.parametrize("causal", [False, True])
def test_sharded_driver_pipelines_whole_batch_shards(causal):
    """Shards that are ranges of whole batch elements, with inputs and output in pinned host memory and no side
    input, go through a per-device pipeline (copies and kernels of neighbouring batch elements overlap): the
    same bits as one device call."""
    from nnlib_jl_b200.shard import ShardedAttention
    ndev = torch.cuda.device_count()
    devices = [f"cuda:{i % ndev}" for i in range(2)]
    dtype, E, H, L, B = torch.bfloat16, 256, 2, 700, 6                     # 12 units over 2 shards: 3 batch elements each
    g = torch.Generator().manual_seed(57)
    hq, hk, hv = (torch.randn((B, L, E), generator=g).to(dtype).pin_memory().permute(2, 1, 0) for _ in range(3))
    hx = torch.zeros((B, L, E), dtype=dtype).pin_memory().permute(2, 1, 0)
    mask = nb.CausalMask() if causal else None
    drv = ShardedAttention(devices)
    for _ in range(2):
        x = drv(hq, hk, hv, mask=mask, nheads=H, out=hx)
    assert x is hx and len(drv._pipes) == len(devices)
    y, _ = nb.dot_product_attention(hq.to(DEV), hk.to(DEV), hv.to(DEV), mask=mask, nheads=H)
    assert torch.equal(hx, y.cpu())


@pytest.mark.parametrize("seed", range(12))
def test_random_shard_partitions_match_the_single_call(seed):
    """Seeded random draws of (heads, batch, shard count, head size, options): the driver cuts the unit grid into
    head-range rectangles and each shard addresses its slice of the parent arrays through pointer offsets and
    the parent's strides — bit-identical x to the unsharded call, whatever the cut."""
    from nnlib_jl_b200.shard import ShardedAttention
    rng = np.random.default_rng(13000 + seed)
    ndev = torch.cuda.device_count()
    nshards = int(rng.integers(1, 6))
    devices = [f"cuda:{i % ndev}" for i in range(nshards)]
    dtype = [torch.bfloat16, torch.float16][seed % 2]
    d = int(rng.choice([64, 128, 96, 40, 72]))
    H, B = int(rng.integers(1, 6)), int(rng.integers(1, 4))
    Lq, Lkv = int(rng.integers(1, 300)), int(rng.integers(1, 400))
    E = d * H
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    kind = str(rng.choice(["none", "causal", "keypad", "full"]))
    mask_np = None
    mask_host = None
    if kind == "causal":
        mask_host = nb.CausalMask(int(rng.integers(0, max(1, Lkv))))
    elif kind == "keypad":
        mask_np = rng.random((Lkv, 1, 1, B)) > 0.3
    elif kind == "full":
        mask_np = rng.random((Lkv, Lq, H, B)) > 0.3
    if mask_np is not None:
        mask_np[0] = True
        mask_host = nb.jl_from_numpy(mask_np)
    bias_host = None
    if rng.random() < 0.4:
        shape = [(Lkv, Lq, H, B), (Lkv, 1, H, 1), (Lkv, Lq)][int(rng.integers(0, 3))]
        bias_host = nb.jl_from_numpy(_round_to(0.5 * rng.standard_normal(shape), dtype), dtype=dtype)
    fd = (lambda: nb.PhiloxDropout(0.2, seed=7 + seed, offset=seed)) if rng.random() < 0.4 else (lambda: nb.identity)
    q, k, v = (nb.jl_from_numpy(a, dtype=dtype) for a in (qn, kn, vn))           # host arrays
    what = f"seed {seed}: {dtype} d={d} H={H} B={B} Lq={Lq} Lkv={Lkv} shards={nshards} mask={kind} bias={None if bias_host is None else tuple(bias_host.shape)}"
    x = ShardedAttention(devices)(q, k, v, bias_host, mask=mask_host, nheads=H, fdrop=fd())
    to_dev = lambda t: t if (t is None or isinstance(t, nb.CausalMask)) else t.to(DEV)
    y, _ = nb.dot_product_attention(q.to(DEV), k.to(DEV), v.to(DEV), to_dev(bias_host), mask=to_dev(mask_host), nheads=H, fdrop=fd())
    assert torch.equal(x, y.cpu()), what


@pytest.mark.parametrize("B,chunk,causal", [(5, 2, True), (3, 1, False), (2, 4, True)])
def test_host_pipelined_attention_matches_device_call(B, chunk, causal):
    """q, k, v in pinned host memory, batch cut into chunks whose copies and kernels overlap: the same
    result as one device call, whatever the chunk size (the last chunk may be partial)."""
    dtype, E, H, L = torch.bfloat16, 256, 2, 300
    g = torch.Generator().manual_seed(55)
    hq, hk, hv = (torch.randn((B, L, E), generator=g).to(dtype).pin_memory() for _ in range(3))
    hx = torch.zeros((B, L, E), dtype=dtype).pin_memory()
    mask = nb.CausalMask() if causal else None
    pipe = nb.HostPipelinedAttention(E, E, L, L, B, dtype, nheads=H, mask=mask, chunk=chunk, device=DEV)
    for _ in range(2):                      # the second call reuses the staging buffers
        pipe(hq, hk, hv, hx)
    pipe.synchronize()
    q, k, v = (t.to(DEV).permute(2, 1, 0) for t in (hq, hk, hv))
    y, _ = nb.dot_product_attention(q, k, v, mask=mask, nheads=H)
    torch.cuda.synchronize()
    assert torch.equal(hx, y.permute(2, 1, 0).cpu())
    with pytest.raises(nb.ArgumentError):
        pipe(hq.clone(), hk, hv, hx)        # not pinned


@pytest.mark.parametrize("B,chunk,kind,tail_split", [
    (3, 1, "causal_matrix", 4), (2, 2, "sentinel", 3), (1, 1, "none", 4), (3, 2, "bool", 4), (2, 1, "bool3", 2),
    (2, 1, "offset", 4),
])
def test_host_pipeline_takes_the_last_batch_element_in_query_ranges(B, chunk, kind, tail_split):
    """The queries of the last batch element go through the pipeline in ranges (their kernels and copies
    back overlap the rest of the input): bit-identical to one device call for every form of mask — the
    causal matrix (recognised, replaced by the pattern with the range's offset), the sentinel with and
    without an offset, and Bool arrays (column ranges of them)."""
    dtype, E, H, L = torch.bfloat16, 256, 2, 1100
    g = torch.Generator().manual_seed(56)
    hq, hk, hv = (torch.randn((B, L, E), generator=g).to(dtype).pin_memory() for _ in range(3))
    hx = torch.zeros((B, L, E), dtype=dtype).pin_memory()
    probe = nb.jl_empty((E, L, 1), dtype, DEV)
    if kind == "causal_matrix":
        mask = nb.make_causal_mask(probe)
    elif kind == "sentinel":
        mask = nb.CausalMask()
    elif kind == "offset":
        mask = nb.CausalMask(37)
    elif kind == "bool":
        m = torch.rand((L, L), generator=g) > 0.3
        m[0] = True
        mask = nb.jl_from_numpy(m.numpy().T.copy().T, device=DEV)
    elif kind == "bool3":
        m = torch.rand((L, L, H), generator=g) > 0.3
        m[0] = True
        mask = nb.jl_from_numpy(m.numpy(), device=DEV)
    else:
        mask = None
    pipe = nb.HostPipelinedAttention(E, E, L, L, B, dtype, nheads=H, mask=mask, chunk=chunk, device=DEV,
                                     tail_split=tail_split)
    assert pipe.tail_split == tail_split
    for _ in range(2):
        pipe(hq, hk, hv, hx)
    pipe.synchronize()
    q, k, v = (t.to(DEV).permute(2, 1, 0) for t in (hq, hk, hv))
    y, _ = nb.dot_product_attention(q, k, v, mask=mask, nheads=H)
    torch.cuda.synchronize()
    assert torch.equal(hx, y.permute(2, 1, 0).cpu())


# --------------------------------------------------------------------------
# backward (pullback) against the gradient oracle
# --------------------------------------------------------------------------

def _grad_close(got, want, dtype, what):
    """Gradients scale with the problem: compare relative to the oracle's magnitude."""
    rel = {torch.float32: 2e-4, torch.float16: 1e-2, torch.bfloat16: 4e-2}[dtype]
    g, w = got.astype(np.float64), want.astype(np.float64)
    scale = np.abs(w).max() + 1e-30
    assert np.isfinite(g).all(), what
    assert np.abs(g - w).max() <= rel * scale, f"{what}: {np.abs(g - w).max() / scale:.3e} of max |grad|"


def test_pullback_reference_gradtest_shapes():
    # test/attention.jl:70-76: q (4,5,1), k = v (4,3,1), bias (3,5), nheads = 2 — Float32 on the device
    rng = np.random.default_rng(60)
    qn = rng.random((4, 5, 1), dtype=np.float32); kn = rng.random((4, 3, 1), dtype=np.float32)
    bn = rng.standard_normal((3, 5)).astype(np.float32)
    dyn = rng.standard_normal((4, 5, 1)).astype(np.float32)
    f32 = torch.float32
    x, a, back = nb.dot_product_attention_pullback(_dev(qn, f32), _dev(kn, f32), _dev(kn, f32), _dev(bn, f32), nheads=2)
    dq, dk, dv, db = back(_dev(dyn, f32))
    # k and v are the same array in the reference's test: its gradient is the sum of both roles
    gq, gk, gv, gb = O.dot_product_attention_grad(qn, kn, kn, dyn, bn, nheads=2)
    _grad_close(nb.jl_to_numpy(dq), gq, f32, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, f32, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, f32, "dv")
    _grad_close(nb.jl_to_numpy(db), gb, f32, "dbias")
    assert tuple(db.shape) == (3, 5)


@pytest.mark.parametrize("dtype,E,H,Lq,Lkv,B,causal,drop", [
    (torch.float32, 48, 3, 37, 50, 2, False, 0.0),
    (torch.float32, 32, 2, 40, 40, 1, True, 0.25),
    (torch.bfloat16, 128, 2, 130, 150, 2, False, 0.1),     # forward on the tensor-core kernels
    (torch.float16, 256, 2, 129, 129, 1, True, 0.0),
])
def test_pullback_matches_gradient_oracle(dtype, E, H, Lq, Lkv, B, causal, drop):
    rng = np.random.default_rng(61)
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    bn = _round_to(0.5 * rng.standard_normal((Lkv, Lq, 1, B)), dtype)
    pad = (np.arange(Lkv)[:, None, None, None] < rng.integers(Lkv // 2, Lkv + 1, size=B)[None, None, None, :])
    mask_np = pad
    if causal:
        mask_np = pad & O.make_causal_mask(np.zeros((1, Lq)), dims=2)[:, :, None, None]
    fd = nb.PhiloxDropout(drop, seed=77, offset=2) if drop > 0 else nb.identity
    x, a, back = nb.dot_product_attention_pullback(
        _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), _dev(bn, dtype),
        mask=nb.jl_from_numpy(mask_np, device=DEV), nheads=H, fdrop=fd)
    dq, dk, dv, db = back(_dev(dyn, dtype))
    keep = P.keep_mask((Lkv, Lq, H, B), drop, 77, 2) if drop > 0 else None
    gq, gk, gv, gb = O.dot_product_attention_grad(qn, kn, vn, dyn, bn, mask=mask_np, nheads=H, keep=keep, p=drop)
    _grad_close(nb.jl_to_numpy(dq), gq, dtype, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, dtype, "dv")
    _grad_close(nb.jl_to_numpy(db), gb, dtype, "dbias")
    assert tuple(db.shape) == (Lkv, Lq, 1, B)


@pytest.mark.parametrize("dtype,E,H,Lq,Lkv,B,causal", [
    (torch.bfloat16, 128, 2, 200, 264, 2, False),    # d = 64, ragged tiles
    (torch.bfloat16, 256, 2, 300, 300, 1, True),     # d = 128, causal with a partial last tile
    (torch.float16, 128, 1, 129, 520, 1, False),     # d = 128, many key tiles
    (torch.float16, 128, 2, 384, 384, 2, True),      # d = 64, whole tiles
])
def test_pullback_on_tensor_cores(dtype, E, H, Lq, Lkv, B, causal):
    """Plain / causal attention of 16-bit arrays: the backward runs on the tcgen05 kernels and matches the
    gradient oracle (and the CUDA-core backward, which the other pullback tests pin)."""
    rng = np.random.default_rng(62)
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    mask = nb.make_causal_mask(_dev(qn, dtype)) if causal else None
    mask_np = (np.arange(Lkv)[:, None] <= np.arange(Lq)[None, :]) if causal else None
    x, a, back = nb.dot_product_attention_pullback(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype),
                                                   mask=mask, nheads=H)
    dq, dk, dv, db = back(_dev(dyn, dtype))
    assert back.path == nb._lib.PATH_UMMA
    assert db is None
    nb.device_health()
    gq, gk, gv, _ = O.dot_product_attention_grad(qn, kn, vn, dyn, None, mask=mask_np, nheads=H)
    _grad_close(nb.jl_to_numpy(dq), gq, dtype, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, dtype, "dv")


@pytest.mark.parametrize("seed", range(32))
def test_random_configurations_of_the_pullback_match_the_gradient_oracle(seed):
    """Seeded random draws for the backward: element type, head size (tensor-core sizes and others), dv != d,
    ragged lengths with several key / query tiles, mask form, bias broadcast shape (dbias has the bias's own
    shape), Philox dropout replayed from the forward — whichever backward the library picks."""
    rng = np.random.default_rng(9000 + seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    d = int(rng.choice([64, 128, 64, 128, 32, 48, 8, 20]))
    dv = d if rng.random() < 0.7 else int(rng.choice([16, 64, 128]))
    H = int(rng.integers(1, 4))
    Lq, Lkv = int(rng.integers(1, 420)), int(rng.integers(1, 420))
    if dtype == torch.float32:
        Lq, Lkv = min(Lq, 90), min(Lkv, 90)                # the Float32 kernels are the slow exact ones
    B = int(rng.integers(1, 3))
    E, Ev = d * H, dv * H
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((Ev, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((Ev, Lq, B)), dtype)
    q, k, v = _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype)

    mask_np = mask_arg = None
    kind = str(rng.choice(["none", "causal", "offset", "keypad", "random"]))
    if kind == "causal" and Lq == Lkv:
        mask_np, mask_arg = O.make_causal_mask(qn), nb.make_causal_mask(q)
    elif kind in ("causal", "offset"):
        off = int(rng.integers(0, max(1, Lkv)))
        mask_np, mask_arg = _offset_mask(Lkv, Lq, off), nb.CausalMask(off)
    elif kind == "keypad":
        lens = rng.integers(1, Lkv + 1, size=B)
        mask_np = np.arange(Lkv)[:, None, None, None] < lens[None, None, None, :]
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)
    elif kind == "random":
        shape = [(Lkv, Lq), (Lkv, Lq, 1, B), (Lkv, Lq, H, B)][int(rng.integers(0, 3))]
        mask_np = rng.random(shape) > 0.3
        mask_np[0] = True
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)

    bias_np = bias_arg = None
    if rng.random() < 0.4:
        shape = [(Lkv, Lq, H, B), (Lkv, Lq), (Lkv, 1, 1, B), (Lkv, Lq, H)][int(rng.integers(0, 4))]
        bias_np = _round_to(0.5 * rng.standard_normal(shape), dtype)
        bias_arg = _dev(bias_np, dtype)

    fdrop, keep, p_drop = nb.identity, None, 0.0
    if rng.random() < 0.3:
        p_drop, dseed, doff = float(rng.choice([0.1, 0.25])), int(rng.integers(0, 2 ** 31)), int(rng.integers(0, 1000))
        keep = P.keep_mask((Lkv, Lq, H, B), p_drop, dseed, doff)
        fdrop = nb.PhiloxDropout(p_drop, seed=dseed, offset=doff)

    what = f"seed {seed}: {dtype} d={d} dv={dv} H={H} Lq={Lq} Lkv={Lkv} B={B} mask={kind} bias={None if bias_np is None else bias_np.shape} p={p_drop}"
    x, a, back = nb.dot_product_attention_pullback(q, k, v, bias_arg, mask=mask_arg, nheads=H, fdrop=fdrop)
    dq, dk, dv_, db = back(_dev(dyn, dtype))
    gq, gk, gv, gb = O.dot_product_attention_grad(qn, kn, vn, dyn, bias_np, mask=mask_np, nheads=H, keep=keep, p=p_drop)
    _grad_close(nb.jl_to_numpy(dq), gq, dtype, "dq, " + what)
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk, " + what)
    _grad_close(nb.jl_to_numpy(dv_), gv, dtype, "dv, " + what)
    if bias_np is None:
        assert db is None, what
    else:
        assert tuple(db.shape) == bias_np.shape, what
        _grad_close(nb.jl_to_numpy(db), gb, dtype, "dbias, " + what)


def test_pullback_at_config3_size_unit_sampled():
    """The tcgen05 backward at the size its throughput is quoted on: bf16, E=4096, nheads=32 (d=128),
    L=4096, causal (32 key / query tiles per unit: causal tile skipping, ring wrap-around, the lse / D
    double buffer of the dk/dv half).  Two whole units are compared with the Float64 gradient oracle of a
    single unit, every row and column of them — rows / keys 0, 127, 128, L-129, L-1 included."""
    dtype, E, H, L, B = torch.bfloat16, 4096, 32, 4096, 2
    g = torch.Generator(device=DEV).manual_seed(66)
    q, k, v, dx = (nb.jl_empty((E, L, B), dtype, DEV) for _ in range(4))
    for t in (q, k, v, dx):
        t.normal_(generator=g)
    x, a, back = nb.dot_product_attention_pullback(q, k, v, mask=nb.make_causal_mask(q), nheads=H)
    dq, dk, dv, _ = back(dx)
    assert back.path == nb._lib.PATH_UMMA
    nb.device_health()
    d = E // H
    for (b, h) in [(0, 0), (1, 31)]:
        sl = slice(h * d, (h + 1) * d)
        qn, kn, vn, dyn = (t[sl, :, b:b + 1].float().cpu().numpy() for t in (q, k, v, dx))
        gq, gk, gv = O.attention_grad_unit(qn, kn, vn, dyn, 1, 0, 0, causal=True)
        for name, got, want in (("dq", dq, gq), ("dk", dk, gk), ("dv", dv, gv)):
            got_n = got[sl, :, b].float().cpu().numpy()
            _grad_close(got_n, want, dtype, f"{name} of unit {(b, h)}")
            # single rows / keys on their own scale (floored at 5 % of the unit's: query 0 attends to one
            # key only, so its dq is an exact zero in the oracle and pure rounding noise on the device)
            for pos in (0, 127, 128, L - 129, L - 1):
                scale = max(np.abs(want[:, pos]).max(), 0.05 * np.abs(want).max())
                err = np.abs(got_n[:, pos].astype(np.float64) - want[:, pos]).max()
                assert err <= 4e-2 * scale, f"{name}[:, {pos}] of unit {(b, h)}: {err / scale:.3e}"


@pytest.mark.parametrize("dtype,E,H,Lq,Lkv,B,kind", [
    (torch.bfloat16, 128, 2, 200, 264, 2, "keypad"),     # (Lkv, 1, 1, B): one byte per key in the dk/dv half
    (torch.float16, 256, 2, 130, 150, 2, "full"),        # (Lkv, Lq, H, B): gathered per step
    (torch.bfloat16, 128, 2, 257, 136, 1, "matrix"),     # (Lkv, Lq) broadcast over heads and batch
])
def test_pullback_with_mask_on_tensor_cores(dtype, E, H, Lq, Lkv, B, kind):
    """Bool mask arrays (src/attention.jl:133-138) in the tcgen05 backward."""
    rng = np.random.default_rng(64)
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    if kind == "keypad":
        mask_np = np.arange(Lkv)[:, None, None, None] < rng.integers(Lkv // 2, Lkv + 1, size=B)[None, None, None, :]
    elif kind == "full":
        mask_np = rng.random((Lkv, Lq, H, B)) > 0.4
        mask_np[0] = True
    else:
        mask_np = rng.random((Lkv, Lq)) > 0.5
        mask_np[3] = True
    x, a, back = nb.dot_product_attention_pullback(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype),
                                                   mask=nb.jl_from_numpy(mask_np, device=DEV), nheads=H)
    dq, dk, dv, db = back(_dev(dyn, dtype))
    assert back.path == _lib.PATH_UMMA
    nb.device_health()
    gq, gk, gv, _ = O.dot_product_attention_grad(qn, kn, vn, dyn, None, mask=mask_np, nheads=H)
    _grad_close(nb.jl_to_numpy(dq), gq, dtype, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, dtype, "dv")


@pytest.mark.parametrize("dtype,E,H,Lq,Lkv,B,causal,keypad,drop", [
    (torch.bfloat16, 128, 2, 200, 264, 2, False, False, 0.2),
    (torch.float16, 256, 2, 300, 300, 1, True, False, 0.1),
    (torch.bfloat16, 192, 3, 140, 333, 2, False, True, 0.3),
])
def test_pullback_with_dropout_on_tensor_cores(dtype, E, H, Lq, Lkv, B, causal, keypad, drop):
    """The tcgen05 backward replays the forward's Philox mask (src/dropout.jl:106-122 pullback): the dq half
    draws rows of scores like the forward, the dk/dv half columns (lanes trade the calls by shuffles)."""
    rng = np.random.default_rng(66)
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    mask, mask_np = None, None
    if causal:
        mask = nb.make_causal_mask(_dev(qn, dtype))
        mask_np = np.arange(Lkv)[:, None] <= np.arange(Lq)[None, :]
    if keypad:
        mask_np = np.arange(Lkv)[:, None, None, None] < rng.integers(Lkv // 2, Lkv + 1, size=B)[None, None, None, :]
        mask = nb.jl_from_numpy(mask_np, device=DEV)
    fd = nb.PhiloxDropout(drop, seed=91, offset=3)
    x, a, back = nb.dot_product_attention_pullback(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype),
                                                   mask=mask, nheads=H, fdrop=fd)
    dq, dk, dv, db = back(_dev(dyn, dtype))
    assert back.path == _lib.PATH_UMMA
    nb.device_health()
    keep = P.keep_mask((Lkv, Lq, H, B), drop, 91, 3)
    gq, gk, gv, _ = O.dot_product_attention_grad(qn, kn, vn, dyn, None, mask=mask_np, nheads=H, keep=keep, p=drop)
    _grad_close(nb.jl_to_numpy(dq), gq, dtype, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, dtype, "dv")


@pytest.mark.parametrize("dtype,bias_dtype,E,H,Lq,Lkv,B,bias_shape,causal,drop", [
    (torch.bfloat16, torch.bfloat16, 128, 2, 200, 264, 2, (264, 200, 2, 2), False, 0.0),   # own element per score
    (torch.float16, torch.float16, 256, 2, 130, 150, 2, (150, 130), False, 0.2),           # summed over heads, batch
    (torch.bfloat16, torch.bfloat16, 128, 2, 140, 333, 2, (333, 1, 1, 2), False, 0.0),     # key bias: summed over queries
    (torch.bfloat16, torch.float32, 128, 2, 257, 257, 1, (257, 257, 2, 1), True, 0.1),     # Float32 bias, causal, odd rows
])
def test_pullback_with_bias_on_tensor_cores(dtype, bias_dtype, E, H, Lq, Lkv, B, bias_shape, causal, drop):
    """Additive bias in the tcgen05 backward: the logits are rebuilt with it and dbias = dS reduced over the
    bias' broadcast dimensions (test/attention.jl:61-76 checks shapes and gradients w.r.t. bias)."""
    rng = np.random.default_rng(67)
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    bn = _round_to(0.5 * rng.standard_normal(bias_shape), bias_dtype)
    mask, mask_np = None, None
    if causal:
        mask = nb.make_causal_mask(_dev(qn, dtype))
        mask_np = np.arange(Lkv)[:, None] <= np.arange(Lq)[None, :]
    fd = nb.PhiloxDropout(drop, seed=92, offset=1) if drop > 0 else nb.identity
    x, a, back = nb.dot_product_attention_pullback(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype),
                                                   _dev(bn, bias_dtype), mask=mask, nheads=H, fdrop=fd)
    dq, dk, dv, db = back(_dev(dyn, dtype))
    assert back.path == _lib.PATH_UMMA
    nb.device_health()
    keep = P.keep_mask((Lkv, Lq, H, B), drop, 92, 1) if drop > 0 else None
    gq, gk, gv, gb = O.dot_product_attention_grad(qn, kn, vn, dyn, bn, mask=mask_np, nheads=H, keep=keep, p=drop)
    _grad_close(nb.jl_to_numpy(dq), gq, dtype, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, dtype, "dv")
    assert tuple(db.shape) == tuple(bias_shape)
    _grad_close(nb.jl_to_numpy(db), gb, bias_dtype if bias_dtype != torch.float32 else dtype, "dbias")


def test_pullback_fully_masked_query_gives_no_gradient():
    """A query that attends to nothing has NaN output (src/softmax.jl:71-76); the library lets no gradient
    flow through it (both backward paths), so the other queries' gradients stay finite."""
    rng = np.random.default_rng(65)
    dtype, E, H, Lq, Lkv, B = torch.bfloat16, 128, 2, 140, 136, 1
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    mask_np = rng.random((Lkv, Lq)) > 0.3
    mask_np[0] = True
    dead = 77
    mask_np[:, dead] = False
    x, a, back = nb.dot_product_attention_pullback(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype),
                                                   mask=nb.jl_from_numpy(mask_np, device=DEV), nheads=H)
    assert np.isnan(nb.jl_to_numpy(x)[:, dead]).all()
    dq, dk, dv, _ = back(_dev(dyn, dtype))
    assert back.path == _lib.PATH_UMMA
    live = np.arange(Lq) != dead
    gq, gk, gv, _ = O.dot_product_attention_grad(qn[:, live], kn, vn, dyn[:, live], None, mask=mask_np[:, live], nheads=H)
    dqn = nb.jl_to_numpy(dq)
    assert (dqn[:, dead] == 0).all()
    _grad_close(dqn[:, live], gq, dtype, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, dtype, "dv")


@pytest.mark.parametrize("Lq,Lkv", [(100, 300), (515, 130)])
def test_abi_backward_causal_flag_on_a_head_slice(Lq, Lkv):
    """C ABI: causal flag with kv_len != q_len (keys past the last query get zero gradient) on a shard that
    owns heads 1..2 of 4 through pointer offsets and the parent's strides; tcgen05 backward kernels."""
    import ctypes as C
    lib = _lib.load()
    rng = np.random.default_rng(63)
    dtype = torch.bfloat16
    H, d, B = 4, 128, 2
    E = H * d
    h0, Hs = 1, 2
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    dyn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    q, k, v, dx = _dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), _dev(dyn, dtype)
    x = nb.jl_zeros((E, Lq, B), dtype, DEV)
    lse = torch.empty((B, Hs, Lq), dtype=torch.float32, device=DEV)
    delta = torch.empty((B, Hs, Lq), dtype=torch.float32, device=DEV)
    dq = nb.jl_zeros((Hs * d, Lq, B), dtype, DEV)
    dk = nb.jl_zeros((Hs * d, Lkv, B), dtype, DEV)
    dv = nb.jl_zeros((Hs * d, Lkv, B), dtype, DEV)
    p = _lib.AttnParams()
    p.dtype = _lib.BF16
    p.d, p.dv, p.H, p.Lq, p.Lkv, p.B = d, d, Hs, Lq, Lkv, B
    off = h0 * d * 2
    p.q, p.k, p.v, p.x = q.data_ptr() + off, k.data_ptr() + off, v.data_ptr() + off, x.data_ptr() + off
    p.q_stride_l = p.k_stride_l = p.v_stride_l = p.x_stride_l = E
    p.q_stride_b, p.x_stride_b = E * Lq, E * Lq
    p.k_stride_b = p.v_stride_b = E * Lkv
    p.lse = lse.data_ptr()
    p.causal = 1
    g = _lib.AttnGrads()
    g.dx = dx.data_ptr() + off
    g.dx_stride_l, g.dx_stride_b = E, E * Lq
    g.dq, g.dk, g.dv, g.delta = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr()
    st = torch.cuda.current_stream().cuda_stream
    assert lib.nnlib_b200_attn_fwd(C.byref(p), st) == 0
    assert lib.nnlib_b200_attn_bwd_path(C.byref(p), C.byref(g)) == _lib.PATH_UMMA
    assert lib.nnlib_b200_attn_bwd(C.byref(p), C.byref(g), st) == 0
    nb.device_health()
    mask_np = np.arange(Lkv)[:, None] <= np.arange(Lq)[None, :]
    sl = slice(h0 * d, (h0 + Hs) * d)
    gq, gk, gv, _ = O.dot_product_attention_grad(qn[sl], kn[sl], vn[sl], dyn[sl], None, mask=mask_np, nheads=Hs)
    _grad_close(nb.jl_to_numpy(dq), gq, dtype, "dq")
    _grad_close(nb.jl_to_numpy(dk), gk, dtype, "dk")
    _grad_close(nb.jl_to_numpy(dv), gv, dtype, "dv")
    if Lkv > Lq:
        assert (nb.jl_to_numpy(dk)[:, Lq:] == 0).all() and (nb.jl_to_numpy(dv)[:, Lq:] == 0).all()
    # D_i = dx_i · x_i is left in the scratch array
    dl = (nb.jl_to_numpy(dx).astype(np.float64)[sl] * nb.jl_to_numpy(x).astype(np.float64)[sl])
    want_delta = dl.reshape(Hs, d, Lq, B).sum(1).transpose(2, 0, 1)          # (B, Hs, Lq)
    np.testing.assert_allclose(delta.cpu().numpy(), want_delta, rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("dtype,E,H,Lq,Lkv,B", [(torch.bfloat16, 256, 2, 200, 264, 2), (torch.float16, 128, 2, 129, 520, 1)])
def test_opaque_fdrop_on_tensor_cores(dtype, E, H, Lq, Lkv, B):
    """fdrop is an arbitrary callable: stats -> scores -> fdrop -> x = V·α′ (src/attention.jl:91-98), with the
    last product on the tcgen05 apply kernel (16-bit types, 16-byte aligned score rows)."""
    rng = np.random.default_rng(70)
    qn = _round_to(rng.standard_normal((E, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((E, Lkv, B)), dtype)
    keep_np = rng.random((Lkv, Lq, H, B)) > 0.3
    keep = nb.jl_from_numpy(keep_np, device=DEV)
    fdrop = lambda al: al * keep / 0.7
    y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), nheads=H, fdrop=fdrop)
    an = nb.jl_to_numpy(a)
    assert ((an > 0) == keep_np).mean() > 0.999       # returned scores are post-fdrop
    # x must be V·α′ for the α′ that was returned (rounded to the element type)
    v4 = O.split_heads(vn, H)
    x4 = O.batched_mul(np.transpose(v4, (0, 2, 1, 3)), an)
    _close(nb.jl_to_numpy(y), O.join_heads(np.transpose(x4, (0, 2, 1, 3))), dtype, "x = V·alpha'")
    yo, _ = O.dot_product_attention(qn, kn, vn, nheads=H, fdrop=lambda al: al * keep_np / np.float32(0.7))
    _close(nb.jl_to_numpy(y), yo, dtype, "x vs oracle")


@pytest.mark.parametrize("seed", range(16))
def test_random_configurations_with_an_opaque_fdrop(seed):
    """fdrop as an arbitrary callable over seeded random shapes and options: statistics -> scores -> fdrop -> x = V alpha'
    (src/attention.jl:91-98), whichever kernels the shapes select for the three steps."""
    rng = np.random.default_rng(14000 + seed)
    dtype = [torch.bfloat16, torch.float16, torch.float32][seed % 3]
    d = int(rng.choice([64, 128, 96, 40, 8, 20, 256]))
    dv = d if rng.random() < 0.7 else int(rng.choice([32, 64, 128]))
    H, B = int(rng.integers(1, 4)), int(rng.integers(1, 3))
    Lq, Lkv = int(rng.integers(1, 260)), int(rng.integers(1, 330))
    if rng.random() < 0.5:
        Lkv = int(8 * rng.integers(1, 40))          # 16-byte aligned score rows: the tensor-core apply kernel
    qn = _round_to(rng.standard_normal((d * H, Lq, B)), dtype)
    kn = _round_to(rng.standard_normal((d * H, Lkv, B)), dtype)
    vn = _round_to(rng.standard_normal((dv * H, Lkv, B)), dtype)
    mask_np = mask_arg = None
    if rng.random() < 0.5:
        mask_np = rng.random((Lkv, Lq, 1, B)) > 0.3
        mask_np[0] = True
        mask_arg = nb.jl_from_numpy(mask_np, device=DEV)
    keep_np = rng.random((Lkv, Lq, H, B)) > 0.3
    keep = nb.jl_from_numpy(keep_np, device=DEV)
    what = f"seed {seed}: {dtype} d={d} dv={dv} H={H} B={B} Lq={Lq} Lkv={Lkv} mask={mask_np is not None}"
    y, a = nb.dot_product_attention(_dev(qn, dtype), _dev(kn, dtype), _dev(vn, dtype), mask=mask_arg, nheads=H,
                                    fdrop=lambda al: al * keep / 0.7)
    an = nb.jl_to_numpy(a)
    yo, ao = O.dot_product_attention(qn, kn, vn, mask=mask_np, nheads=H, fdrop=lambda al: al * keep_np / np.float32(0.7))
    _close(an, ao, dtype, "alpha', " + what)
    _close(nb.jl_to_numpy(y), yo, dtype, "x, " + what)
