"""Host-side logic that needs no GPU: column-major tensors, the package's
Philox copy against the oracle's, the reference's argument checks, and the
multi-GPU driver's partitioning, slicing and per-shard failure reporting
(with a CPU stand-in injected for the per-device computation)."""
import numpy as np
import pytest
import torch

import nnlib_jl_b200 as nb
from nnlib_jl_b200 import attention as A
from nnlib_jl_b200 import dropout as D
from nnlib_jl_b200 import shard as S
from oracle import attention_oracle as O
from oracle import philox_oracle as P


# ---- layout ----------------------------------------------------------------
def test_column_major_roundtrip():
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = nb.jl_from_numpy(a)
    assert tuple(t.shape) == (2, 3, 4) and t.stride() == (1, 2, 6) and nb.is_column_major(t)
    # memory order is the reference's: linear offset e + E*l + E*L*b
    flat = t.permute(2, 1, 0).contiguous().view(-1).numpy()
    np.testing.assert_array_equal(flat, a.ravel(order="F"))
    np.testing.assert_array_equal(nb.jl_to_numpy(t), a)
    r = nb.jl_reshape(t, (6, 4))
    np.testing.assert_array_equal(nb.jl_to_numpy(r), a.reshape((6, 4), order="F"))
    assert r.data_ptr() == t.data_ptr()
    r2 = nb.jl_reshape(t, (2, 3, 2, 1, 2))
    np.testing.assert_array_equal(nb.jl_to_numpy(r2), a.reshape((2, 3, 2, 1, 2), order="F"))
    assert not nb.is_column_major(torch.zeros(2, 3))
    assert nb.is_column_major(nb.as_column_major(torch.zeros(2, 3)))
    with pytest.raises(ValueError):
        nb.jl_reshape(torch.zeros(2, 3), (3, 2))


def test_split_heads_is_a_pure_reshape():
    a = np.arange(4 * 6 * 2, dtype=np.float32).reshape(12, 2, 2)
    t = nb.jl_from_numpy(a)
    np.testing.assert_array_equal(nb.jl_to_numpy(nb.jl_reshape(t, (3, 4, 2, 2))), O.split_heads(a, 4))


# ---- dropout ---------------------------------------------------------------
def test_package_philox_matches_oracle_and_kat():
    got = D.philox4x32_10(np.array([0x243f6a88]), np.array([0x85a308d3]), np.array([0x13198a2e]),
                          np.array([0x03707344]), 0xa4093822, 0x299f31d0)
    assert tuple(int(g[0]) for g in got) == (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1)
    for args in [dict(shape4=(37, 5, 3, 2), p=0.3, seed=1234, offset=7, h0=1, b0=2, H_total=8),
                 dict(shape4=(8, 2, 1, 1), p=0.9, seed=(1 << 40) + 5, offset=(3 << 32) + 1)]:
        np.testing.assert_array_equal(D.keep_mask(**args), P.keep_mask(**args))


def test_sharded_mask_equals_slice_of_whole():
    whole = D.keep_mask((16, 4, 6, 5), 0.25, seed=9)
    part = D.keep_mask((16, 4, 2, 3), 0.25, seed=9, h0=3, b0=1, H_total=6)
    np.testing.assert_array_equal(part, whole[:, :, 3:5, 1:4])


def test_philox_dropout_on_host_arrays():
    rng = np.random.default_rng(0)
    a = rng.random((12, 5, 2, 3)).astype(np.float32) + 0.1
    fd = nb.PhiloxDropout(0.5, seed=3)
    out = fd(a)
    keep = P.keep_mask(a.shape, 0.5, 3, 0)
    np.testing.assert_allclose(out, a * keep * 2.0)
    out2 = fd(torch.from_numpy(a))            # second call: next offset
    keep2 = P.keep_mask(a.shape, 0.5, 3, 1)
    np.testing.assert_allclose(out2.numpy(), a * keep2 * 2.0)
    assert not (keep == keep2).all()
    assert 0.4 < keep.mean() < 0.6
    with pytest.raises(ValueError):
        nb.PhiloxDropout(1.0)
    # usable as the reference-style fdrop of the oracle
    q = rng.random((10, 10, 10))
    y, al = O.dot_product_attention(q, q, q, nheads=2, fdrop=nb.PhiloxDropout(0.5, seed=1))
    assert 0.4 < (al > 0).mean() < 0.6


# ---- argument checks of src/attention.jl:55-78 --------------------------------
def test_validation_messages():
    z = lambda *s: torch.zeros(*s)
    with pytest.raises(nb.ArgumentError, match="divisible by `nheads`"):
        A._validate_3d(z(6, 2, 1), z(6, 2, 1), z(6, 2, 1), 4)
    with pytest.raises(nb.ArgumentError, match="Batch dimensions have to be the same"):
        A._validate_3d(z(4, 2, 1), z(4, 2, 2), z(4, 2, 2), 1)
    with pytest.raises(nb.ArgumentError, match="First dimension in query and key"):
        A._validate_3d(z(4, 2, 1), z(6, 2, 1), z(6, 2, 1), 1)
    with pytest.raises(nb.ArgumentError, match="Second dimension in key and value"):
        A._validate_3d(z(4, 2, 1), z(4, 3, 1), z(4, 2, 1), 1)
    A._validate_3d(z(4, 2, 1), z(4, 3, 1), z(8, 3, 1), 2)     # Ev != E and Lq != Lkv are fine
    # non-CUDA arrays do not dispatch to this method
    with pytest.raises(TypeError, match="CUDA arrays only"):
        nb.dot_product_attention(z(4, 2, 1), z(4, 2, 1), z(4, 2, 1))
    with pytest.raises(TypeError):
        nb.make_causal_mask(z(4, 2, 1))


def test_bias_mask_broadcast_strides():
    full = (7, 5, 3, 2)
    t = nb.jl_empty((7, 5))
    assert A._bcast_strides("bias", t, full) == [1, 7, 0, 0]
    t = nb.jl_empty((7, 1, 1, 2))
    assert A._bcast_strides("mask", t, full) == [1, 0, 0, 7]
    t = nb.jl_empty((1, 5, 3, 1))
    assert A._bcast_strides("bias", t, full) == [0, 1, 5, 0]
    with pytest.raises(nb.ArgumentError):
        A._bcast_strides("bias", nb.jl_empty((6, 5)), full)
    with pytest.raises(nb.ArgumentError):
        A._bcast_strides("bias", nb.jl_empty((7, 5, 3, 2, 1)), full)


# ---- sharding --------------------------------------------------------------
@pytest.mark.parametrize("B,H,n", [(8, 16, 8), (8, 16, 3), (1, 5, 4), (3, 2, 8), (7, 3, 2), (8, 32, 1)])
def test_partition_covers_every_unit_once(B, H, n):
    plan = S.partition_units(B, H, n)
    assert len(plan) == n
    seen = np.zeros((B, H), dtype=int)
    sizes = []
    for rects in plan:
        sizes.append(sum(r.units for r in rects))
        assert len(rects) <= 3
        for r in rects:
            seen[r.b0:r.b0 + r.nb, r.h0:r.h0 + r.nh] += 1
    assert (seen == 1).all()
    assert max(sizes) - min(sizes) <= 1
    if B % n == 0:
        assert all(len(rects) == 1 and rects[0].nh == H and rects[0].nb == B // n for rects in plan)
    assert S.rank_rects(B, H, n - 1, n) == plan[-1]


def _cpu_compute(dev, q, k, v, bias, mask, nheads, dropout, rng_origin):
    """Stand-in for the per-rectangle GPU call: the oracle on the shard's slices."""
    to_np = lambda t: None if t is None else nb.jl_to_numpy(t)
    fdrop = (lambda a: a)
    if dropout is not None:
        h0, b0, H = rng_origin
        Lkv, Lq, B = k.shape[1], q.shape[1], q.shape[2]
        keep = P.keep_mask((Lkv, Lq, nheads, B), dropout.p, dropout.seed, dropout.offset, h0=h0, b0=b0, H_total=H)
        fdrop = lambda a: a * keep / np.float32(1 - dropout.p)
    m = mask if not isinstance(mask, torch.Tensor) else to_np(mask)
    y, _ = O.dot_product_attention(to_np(q), to_np(k), to_np(v), to_np(bias), mask=m, nheads=nheads, fdrop=fdrop)
    return nb.jl_from_numpy(y.astype(np.float32))


@pytest.mark.parametrize("ndev", [1, 2, 3, 8])
def test_sharded_driver_assembles_the_unsharded_result(ndev):
    rng = np.random.default_rng(5)
    E, H, Lq, Lkv, B = 12, 3, 5, 7, 4
    qn, kn, vn = (rng.standard_normal(s).astype(np.float32) for s in ((E, Lq, B), (E, Lkv, B), (2 * E, Lkv, B)))
    bias = rng.standard_normal((Lkv, Lq, H, B)).astype(np.float32)
    mask = rng.random((Lkv, 1, 1, B)) > 0.2
    mask[0] = True
    drv = S.ShardedAttention([f"cpu:{i}" for i in range(ndev)], compute=_cpu_compute, out_device="cpu")
    fd = nb.PhiloxDropout(0.2, seed=77, offset=5)
    x = drv(nb.jl_from_numpy(qn), nb.jl_from_numpy(kn), nb.jl_from_numpy(vn), nb.jl_from_numpy(bias),
            mask=nb.jl_from_numpy(mask), nheads=H, fdrop=fd)
    keep = P.keep_mask((Lkv, Lq, H, B), 0.2, 77, 5)
    want, _ = O.dot_product_attention(qn, kn, vn, bias, mask=mask, nheads=H,
                                      fdrop=lambda a: a * keep / np.float32(0.8))
    np.testing.assert_allclose(nb.jl_to_numpy(x), want, rtol=1e-5, atol=1e-6)
    assert fd.offset == 6     # the call consumed exactly one offset


def test_sharded_driver_reports_a_failing_shard_and_keeps_the_others():
    rng = np.random.default_rng(6)
    E, H, L, B = 8, 2, 4, 4
    qn = rng.standard_normal((E, L, B)).astype(np.float32)

    def flaky(dev, *args):
        if dev == "cpu:1":
            raise RuntimeError("injected: device lost")      # host-side failure injection
        return _cpu_compute(dev, *args)

    drv = S.ShardedAttention(["cpu:0", "cpu:1", "cpu:2", "cpu:3"], compute=flaky, out_device="cpu")
    q = nb.jl_from_numpy(qn)
    with pytest.raises(S.ShardError) as ei:
        drv(q, q, q, nheads=H)
    err = ei.value
    assert [r.ok for r in err.results] == [True, False, True, True]
    assert "injected" in str(err) and "cpu:1" in str(err)
    want, _ = O.dot_product_attention(qn, qn, qn, nheads=H)
    got = nb.jl_to_numpy(err.x)
    for r in (0, 2, 3):     # each device owns one batch here
        np.testing.assert_allclose(got[:, :, r], want[:, :, r], rtol=1e-5, atol=1e-6)


def test_sharded_driver_rejects_opaque_fdrop():
    q = nb.jl_zeros((4, 2, 2))
    drv = S.ShardedAttention(["cpu:0"], compute=_cpu_compute)
    with pytest.raises(nb.ArgumentError):
        drv(q, q, q, fdrop=lambda a: a)
