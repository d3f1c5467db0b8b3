"""Pins the CPU oracle against every known-answer vector the reference's own
tests hold for the attention path, and re-states the reference's remaining
attention tests (test/attention.jl) on the oracle."""
import numpy as np
import pytest

from oracle import attention_oracle as O
from oracle import philox_oracle as P


def _mat(rows):
    return np.array([[float(v) for v in r] for r in rows], dtype=np.float32)


def test_specific_results(golden):
    # test/attention.jl:25-34
    g = golden["attention_specific"]
    q = (np.arange(1, 13, dtype=np.float64).reshape(g["q_shape"], order="F") / 12)
    y, a = O.dot_product_attention(q, q, q, nheads=g["nheads"])
    ytrue = np.array(g["ytrue_colmajor"]).reshape(g["ytrue_shape"], order="F")
    atrue = np.array(g["alphatrue_colmajor"]).reshape(g["alphatrue_shape"], order="F")
    assert y.shape == ytrue.shape and a.shape == atrue.shape
    np.testing.assert_allclose(y, ytrue, atol=g["atol"], rtol=0)
    np.testing.assert_allclose(a, atrue, atol=g["atol"], rtol=0)
    # same in Float32, the precision the parity tests use
    y32, a32 = O.dot_product_attention(*(q.astype(np.float32),) * 3, nheads=2)
    assert y32.dtype == np.float32
    np.testing.assert_allclose(y32, ytrue, atol=g["atol"], rtol=0)
    np.testing.assert_allclose(a32, atrue, atol=g["atol"], rtol=0)


def test_softmax_inf_nan_tables(golden):
    # test/softmax.jl:61-68
    for case in golden["softmax_inf_nan"]["cases"]:
        x, y = _mat(case["x"]), _mat(case["y"])
        got = O.softmax(x, dims=case["dims"] - 1)
        np.testing.assert_allclose(got, y, rtol=1e-6, equal_nan=case["nans"])


def test_softmax_basic(golden):
    for case in golden["softmax_basic"]["cases"]:
        np.testing.assert_allclose(O.softmax(np.array(case["x"])), case["y"])
    xs = np.random.default_rng(0).random((5, 5))
    np.testing.assert_allclose(O.softmax(xs).sum(0), 1)
    np.testing.assert_allclose(O.softmax(xs, dims=1).sum(1), 1)
    v = np.random.default_rng(1).random(5)
    np.testing.assert_allclose(O.softmax(v), np.exp(v) / np.exp(v).sum())


def test_masked_softmax_regression():
    # test/ext_cuda/softmax.jl:34-78: big negative fill stays finite, -Inf gives exact zeros
    rng = np.random.default_rng(2)
    x = rng.standard_normal((128, 32)).astype(np.float32)
    x[:64] = -1e3
    y = O.softmax(x)
    assert np.isfinite(y).all()
    xi = rng.standard_normal((128, 32)).astype(np.float32)
    xi[:64] = -np.inf
    yi = O.softmax(xi)
    assert np.isfinite(yi).all() and (yi[:64] == 0).all()


@pytest.mark.parametrize("batch_size", [(), (1,), (2,), (2, 1, 3)])
@pytest.mark.parametrize("nheads", [1, 3, 5])
def test_different_batchsizes(batch_size, nheads):
    # test/attention.jl:1-15
    rng = np.random.default_rng(3)
    n, lenq, lenkv = 15, 3, 4
    q = rng.random((n, lenq) + batch_size, dtype=np.float32)
    k = rng.random((n, lenkv) + batch_size, dtype=np.float32)
    v = rng.random((n, lenkv) + batch_size, dtype=np.float32)
    y, a = O.dot_product_attention(q, k, v, nheads=nheads)
    assert y.dtype == np.float32
    assert y.shape == (n, lenq) + batch_size
    assert a.shape == (lenkv, lenq, nheads) + batch_size
    np.testing.assert_allclose(a.sum(0), np.ones((lenq, nheads) + batch_size), rtol=1e-5)


def test_scores_match_3d_entry():
    # test/attention.jl:17-23
    q = np.arange(1, 25, dtype=np.float64).reshape((4, 2, 3, 1), order="F") / 24
    a = O.dot_product_attention_scores(q, q)
    q2 = q.reshape((8, 3, 1), order="F")
    _, a2 = O.dot_product_attention(q2, q2, q2, nheads=2)
    np.testing.assert_allclose(a, a2)


def test_mask_and_causal():
    # test/attention.jl:36-52
    rng = np.random.default_rng(4)
    q = rng.random((4, 2, 3, 1))
    k = rng.random((4, 2, 5, 1))
    mask = rng.random((5, 3)) > 0.5
    mask[0] = True
    a = O.dot_product_attention_scores(q, k, mask=mask)
    assert ((a[:, :, 0, 0] > 0) == mask).all() and ((a[:, :, 1, 0] > 0) == mask).all()
    x = rng.random((4, 2, 3, 1))
    cm = O.make_causal_mask(x, dims=3)
    assert cm.shape == (3, 3) and cm[0, 2] and not cm[2, 0]
    a = O.dot_product_attention_scores(x, x, mask=cm)
    assert ((a[:, :, 0, 0] > 0) == cm).all() and ((a[:, :, 1, 0] > 0) == cm).all()


def test_fully_masked_query_is_nan():
    # src/softmax.jl:71-76: max = -Inf gives exp(-Inf - -Inf) = NaN for the column
    rng = np.random.default_rng(5)
    q = rng.random((4, 1, 3, 1)); k = rng.random((4, 1, 5, 1))
    mask = np.ones((5, 3), dtype=bool); mask[:, 1] = False
    a = O.dot_product_attention_scores(q, k, mask=mask)
    assert np.isnan(a[:, 1]).all() and np.isfinite(a[:, 0]).all()


def test_dropout_rate_and_post_dropout_alpha():
    # test/attention.jl:54-59
    rng = np.random.default_rng(6)
    q = rng.random((10, 10, 10))
    fdrop = lambda a: O.dropout_apply(a, rng.random(a.shape), 0.5)
    y, a = O.dot_product_attention(q, q, q, nheads=2, fdrop=fdrop)
    assert 0.4 < (a > 0).mean() < 0.6
    # x is computed from the returned (post-dropout) scores
    v4 = O.split_heads(q, 2)
    x4 = O.batched_mul(np.transpose(v4, (0, 2, 1, 3)), a)
    np.testing.assert_allclose(O.join_heads(np.transpose(x4, (0, 2, 1, 3))), y)


def test_bias_shapes():
    # test/attention.jl:61-68
    rng = np.random.default_rng(7)
    q = rng.random((4, 5, 1)); k = rng.random((4, 3, 1))
    bias = rng.standard_normal((3, 5))
    y, a = O.dot_product_attention(q, k, k, bias, nheads=2)
    assert a.shape == (3, 5, 2, 1) and y.shape == (4, 5, 1)
    # bias really is added to the scaled logits
    y0, a0 = O.dot_product_attention(q, k, k, nheads=2)
    assert not np.allclose(a, a0)


def test_argument_errors():
    # src/attention.jl:42,55-78
    z = np.zeros
    with pytest.raises(O.ArgumentError, match="divisible"):
        O.dot_product_attention(z((6, 2, 1)), z((6, 2, 1)), z((6, 2, 1)), nheads=4)
    with pytest.raises(O.ArgumentError, match="Batch"):
        O.dot_product_attention(z((4, 2, 1)), z((4, 2, 2)), z((4, 2, 2)))
    with pytest.raises(O.ArgumentError, match="query and key"):
        O.dot_product_attention(z((4, 2, 1)), z((6, 2, 1)), z((6, 2, 1)))
    with pytest.raises(O.ArgumentError, match="key and value"):
        O.dot_product_attention(z((4, 2, 1)), z((4, 3, 1)), z((4, 2, 1)))
    with pytest.raises(O.ArgumentError, match="Batch"):
        O.dot_product_attention(z((4, 2, 1, 2)), z((4, 2, 2, 1)), z((4, 2, 2, 1)))


def test_attention_rows_matches_full():
    rng = np.random.default_rng(8)
    q = rng.standard_normal((16, 9, 2)); k = rng.standard_normal((16, 11, 2)); v = rng.standard_normal((24, 11, 2))
    bias = rng.standard_normal((11, 9, 1, 2)); mask = rng.random((11, 1, 1, 2)) > 0.3
    mask[0] = True
    y, a = O.dot_product_attention(q, k, v, bias, mask=mask, nheads=4)
    rows = np.array([0, 3, 8])
    xr, ar, lse = O.attention_rows(q, k, v, 4, rows, b=1, h=2, mask=mask, bias=bias)
    np.testing.assert_allclose(ar, a[:, rows, 2, 1], rtol=1e-10)
    np.testing.assert_allclose(xr, y[12:18][:, rows, 1], rtol=1e-10)


# ---- Philox4x32-10 known answers (Random123 kat_vectors) -------------------
KAT = [
    ((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
    ((0xffffffff,) * 4, (0xffffffff, 0xffffffff), (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
    ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
     (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)),
]


def test_philox_known_answers():
    for ctr, key, want in KAT:
        assert P.philox4x32_10_scalar(ctr, key) == want
        got = P.philox4x32_10_np(*[np.array([c]) for c in ctr], *key)
        assert tuple(int(g[0]) for g in got) == want


def test_keep_mask_rate():
    m = P.keep_mask((64, 16, 2, 2), 0.1, seed=0xB200)
    assert abs(m.mean() - 0.9) < 0.02


# ---- gradient oracle: pinned by central finite differences, like the reference's gradtest
#      (test/attention.jl:70-76 uses FiniteDifferences on q (4,5,1), k = v (4,3,1), bias (3,5), nheads = 2)
def _fd(fun, x, eps=1e-6):
    out = np.zeros_like(x)
    it = np.nditer(x, flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        xp, xm = x.copy(), x.copy()
        xp[i] += eps
        xm[i] -= eps
        out[i] = (fun(xp) - fun(xm)) / (2 * eps)
    return out


@pytest.mark.parametrize("with_mask,with_drop", [(False, False), (True, False), (True, True)])
def test_gradient_oracle_against_finite_differences(with_mask, with_drop):
    rng = np.random.default_rng(20)
    q = rng.random((4, 5, 1)); k = rng.random((4, 3, 1)); v = rng.random((4, 3, 1))
    bias = rng.standard_normal((3, 5))
    dy = rng.standard_normal((4, 5, 1))
    mask = None
    if with_mask:
        mask = np.ones((3, 5), dtype=bool); mask[1, 2] = False; mask[2, 0] = False
    keep, p = None, 0.0
    fdrop = lambda a: a
    if with_drop:
        p = 0.3
        keep = P.keep_mask((3, 5, 2, 1), p, seed=4)
        fdrop = lambda a: a * keep / (1 - p)
    f = lambda q_, k_, v_, b_: (O.dot_product_attention(q_, k_, v_, b_, mask=mask, nheads=2, fdrop=fdrop)[0] * dy).sum()
    dq, dk, dv, db = O.dot_product_attention_grad(q, k, v, dy, bias, mask=mask, nheads=2, keep=keep, p=p)
    np.testing.assert_allclose(dq, _fd(lambda t: f(t, k, v, bias), q), atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(dk, _fd(lambda t: f(q, t, v, bias), k), atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(dv, _fd(lambda t: f(q, k, t, bias), v), atol=1e-6, rtol=1e-6)
    np.testing.assert_allclose(db, _fd(lambda t: f(q, k, v, t), bias), atol=1e-6, rtol=1e-6)


def test_config1_on_the_oracle():
    """BASELINE config 1 exactly: Float32 q, k, v ~ N(0,1), E=512, nheads=8 (d=64), Lq=Lkv=128, batch=4, no
    mask / bias, fdrop = identity; returns (x, α) with α of size (128, 128, 8, 4).  The Float32 oracle must
    agree with its own Float64 row-restricted form and keep the reference's structural properties
    (test/attention.jl:1-15: sizes, columns of α sum to 1)."""
    rng = np.random.default_rng(1234)
    E, H, L, B = 512, 8, 128, 4
    q, k, v = (rng.standard_normal((E, L, B), dtype=np.float32) for _ in range(3))
    x, a = O.dot_product_attention(q, k, v, nheads=H)
    assert x.shape == (E, L, B) and a.shape == (L, L, H, B) and x.dtype == np.float32
    np.testing.assert_allclose(a.sum(0), 1.0, atol=1e-5)
    assert (a > 0).all()
    rows = np.arange(L)
    d = E // H
    for (b, h) in [(0, 0), (3, 7), (1, 4)]:
        xr, ar, _ = O.attention_rows(q, k, v, H, rows, b, h)
        np.testing.assert_allclose(x[h * d:(h + 1) * d, :, b], xr, atol=1e-5)
        np.testing.assert_allclose(a[:, :, h, b], ar, atol=1e-5)


@pytest.mark.parametrize("causal", [False, True])
def test_gradient_of_one_unit_matches_full_gradient(causal):
    rng = np.random.default_rng(7)
    E, H, L, B = 24, 3, 11, 2
    q, k, v, dy = (rng.standard_normal((E, L, B)) for _ in range(4))
    mask = O.make_causal_mask(q) if causal else None
    gq, gk, gv, _ = O.dot_product_attention_grad(q, k, v, dy, mask=mask, nheads=H)
    d = E // H
    for b in range(B):
        for h in range(H):
            dq, dk, dv = O.attention_grad_unit(q, k, v, dy, H, b, h, causal=causal)
            sl = slice(h * d, (h + 1) * d)
            np.testing.assert_allclose(dq, gq[sl, :, b], atol=1e-12)
            np.testing.assert_allclose(dk, gk[sl, :, b], atol=1e-12)
            np.testing.assert_allclose(dv, gv[sl, :, b], atol=1e-12)


def test_plus_inf_bias_is_always_attend_here():
    """src/softmax.jl:73-75 reached through attention: a +Inf bias puts the whole weight of that query on
    the +Inf keys in equal shares (masked keys excepted: the mask is applied after the bias,
    src/attention.jl:122-123), a NaN logit makes the query's column NaN."""
    rng = np.random.default_rng(8)
    E, H, Lq, Lkv, B = 8, 2, 5, 6, 1
    q, k, v = (rng.standard_normal((E, L, B)).astype(np.float32) for L in (Lq, Lkv, Lkv))
    bias = np.zeros((Lkv, Lq, H, B), dtype=np.float32)
    bias[2, 0] = np.inf                       # query 0: one-hot on key 2
    bias[[1, 4], 1] = np.inf                  # query 1: halves on keys 1 and 4
    bias[3, 2] = np.inf                       # query 2: +Inf on a key the mask removes
    bias[0, 3] = np.nan                       # query 3: NaN
    mask = np.ones((Lkv, Lq), dtype=bool)
    mask[3, 2] = False
    x, a = O.dot_product_attention(q, k, v, bias, mask=mask, nheads=H)
    d = E // H
    for h in range(H):
        np.testing.assert_array_equal(a[:, 0, h, 0], np.eye(Lkv, dtype=np.float32)[2])
        want = np.zeros(Lkv, dtype=np.float32); want[[1, 4]] = 0.5
        np.testing.assert_array_equal(a[:, 1, h, 0], want)
        assert a[3, 2, h, 0] == 0 and abs(a[:, 2, h, 0].sum() - 1) < 1e-6
        assert np.isnan(a[:, 3, h, 0]).all() and np.isnan(x[h * d:(h + 1) * d, 3, 0]).all()
        np.testing.assert_allclose(x[h * d:(h + 1) * d, 0, 0], v[h * d:(h + 1) * d, 2, 0], rtol=1e-6)
        assert np.isfinite(a[:, 4, h, 0]).all()
