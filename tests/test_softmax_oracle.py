"""The softmax oracle against the reference's own known-answer tests (NNlib.jl test/softmax.jl:16-75)."""
import numpy as np

from oracle import softmax_oracle as S


def test_basic_properties_and_identities():
    rng = np.random.default_rng(0)
    xs = rng.random((5, 5))
    assert np.allclose(S.softmax(xs).sum(0), 1)                               # test/softmax.jl:18
    assert np.allclose(S.softmax(xs, dims=2).sum(1), 1)                       # :19
    assert np.allclose(np.log(S.softmax(xs, dims=2)), S.logsoftmax(xs, dims=2))   # :21
    v = rng.random(5)
    assert np.allclose(S.softmax(v), np.exp(v) / np.exp(v).sum())             # :28
    assert np.allclose(S.softmax(np.array([-100000.0, -100000.0])), [0.5, 0.5])           # :23-25
    assert np.allclose(S.logsoftmax(np.array([-100000.0, -100000.0])), np.log([0.5, 0.5]))


def test_large_inputs_and_pullbacks_of_ones():
    assert np.allclose(S.logsoftmax(np.float32([1, 2, 3000.0])), [-2999, -2998, 0])       # :31-32
    xs = np.float32([[1, 2, 3], [1000, 2000, 3000]])
    assert np.allclose(S.logsoftmax(xs), [[-999, -1998, -2997], [0, 0, 0.0]])             # :34-35
    y = S.logsoftmax(xs)
    assert np.allclose(S.logsoftmax_pullback(np.ones_like(xs), y), np.float32([[1, 1, 1], [-1, -1, -1]]))   # :37-38
    y = S.softmax(xs)
    assert np.allclose(S.softmax_pullback(np.ones_like(xs), y), 0)                        # :40-41


def test_values_precalculated_with_pytorch():
    # test/softmax.jl:43-59
    xs = np.array([[-0.238639, 0.748142, -0.283194, -0.525461, -1.5348, -0.797842],
                   [0.690384, 0.211427, 0.254794, -0.213572, -0.314174, -0.372663],
                   [-1.146370, -0.577988, 0.718952, 0.919720, -0.620773, 0.929977]])
    ys = np.array([[0.237703, -0.621474, 0.448193, 0.546047, 0.564185, 0.632273],
                   [-0.930163, 0.0519798, 0.0549979, 0.3799, -0.477112, 0.437428],
                   [0.69246, 0.569494, -0.503191, -0.925947, -0.0870738, -1.0697]])
    y = S.logsoftmax(xs)
    np.testing.assert_allclose(S.logsoftmax_pullback(np.ones_like(xs), y), ys, rtol=1e-5, atol=1e-6)
    y = S.softmax(xs)
    np.testing.assert_allclose(S.softmax_pullback(np.ones_like(xs), y), 0, atol=1e-6)


def test_inf_and_nan_table():
    # test/softmax.jl:62-75
    f = np.float32
    inf, nan = np.inf, np.nan
    np.testing.assert_allclose(S.softmax(f([[1, 2], [3, inf]])), f([[0.11920292, 0.0], [0.880797, 1.0]]), rtol=1e-6)
    np.testing.assert_allclose(S.softmax(f([[1, -inf], [3, inf]])), f([[0.11920292, 0.0], [0.880797, 1.0]]), rtol=1e-6)
    np.testing.assert_allclose(S.softmax(f([[1, inf], [3, inf]])), f([[0.11920292, 0.5], [0.880797, 0.5]]), rtol=1e-6)
    got = S.softmax(f([[1, 2], [3, nan]]))
    np.testing.assert_allclose(got[:, 0], f([0.11920292, 0.880797]), rtol=1e-6)
    assert np.isnan(got[:, 1]).all()
    np.testing.assert_allclose(S.softmax(f([[1, 2], [3, inf]]), dims=2), f([[0.26894143, 0.7310586], [0.0, 1.0]]), rtol=1e-6)
    np.testing.assert_allclose(S.softmax(f([[1, 2], [3, inf]]), dims=None), f([[0, 0], [0, 1.0]]))
    np.testing.assert_allclose(S.softmax(f([[1, 2], [3, inf]]), dims=(1, 2)), f([[0, 0], [0, 1.0]]))
    for x in (f([[1, 2], [3, inf]]), f([[1, -inf], [3, inf]]), f([[1, inf], [3, inf]])):
        np.testing.assert_allclose(np.exp(S.logsoftmax(x)), S.softmax(x), rtol=1e-6)
    # a column of -Inf (a fully masked attention query): NaN, src/softmax.jl:71-76
    assert np.isnan(S.softmax(f([[-inf, 1], [-inf, 2]]))[:, 0]).all()
