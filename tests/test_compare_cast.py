"""Comparisons, Tensor::to(DType), ones, rand and operator[] (src/Tensor.cpp:985-1309, 1462-1591,
199-243, 422-479, 175-189).

CPU part: the numpy restatement against the golden record made from the reference and against the
reference library run now; the front end's host tensors against the same record; error behaviour.
GPU part: the kernels through the C ABI and the front end's device tensors, bit for bit; rand by its
distribution (the reference seeds from std::random_device: no sequence of it can be reproduced)."""
import numpy as np
import pytest

import oracle
from conftest import assert_exact

CMP_CODE = {c: i for i, c in enumerate(oracle.CMP_NAMES)}


def _frontend():
    from ctorch_b200 import frontend as F
    F.set_quiet(True)
    return F


# ---- CPU -------------------------------------------------------------------------------------------
def test_restatement_against_golden_and_reference(golden):
    G = golden
    a, b, s = G["cmp.a"], G["cmp.b"], float(G["cmp.s"])
    ref = oracle.Reference() if oracle.Reference.available() else None
    for c in oracle.CMP_NAMES:
        for key, got in ((f"cmp.{c}.tt", oracle.compare(c, a, b)), (f"cmp.{c}.ts", oracle.compare(c, a, s)),
                         (f"cmp.{c}.st", oracle.compare(c, a, s, scalar_left=True))):
            assert_exact(got, G[key], key)
        if ref:
            assert_exact(ref.compare(c, a, b), G[f"cmp.{c}.tt"], f"reference now: {c}")
    x = G["cast.x"]
    for d in (1, 2, 3, 4):
        assert_exact(oracle.cast_from_float(x, d), G[f"cast.{d}"], f"to(dtype {d})")
        assert oracle.cast_from_float(x, d).dtype == G[f"cast.{d}"].dtype
    assert_exact(np.asarray([oracle.index_1d(x, i)[0] for i in (0, 2, 1002)], np.float32), G["index.values"])
    with pytest.raises(ValueError):
        oracle.compare("gt", a, b[:, :3])
    with pytest.raises(IndexError):
        oracle.index_1d(x, x.size)
    with pytest.raises(ValueError):
        oracle.index_1d(a, 0)


def test_front_end_host_tensors(golden):
    F = _frontend()
    G = golden
    A, B = F.Tensor.from_numpy(G["cmp.a"], F.CPU), F.Tensor.from_numpy(G["cmp.b"], F.CPU)
    s = float(G["cmp.s"])
    for c in oracle.CMP_NAMES:
        code = CMP_CODE[c]
        r = A._cmp(code, B)
        assert r.dtype == F.BOOL and r.shape == A.shape
        assert_exact(r.numpy(), G[f"cmp.{c}.tt"], f"{c} tensor/tensor")
        assert_exact(A._cmp(code, s).numpy(), G[f"cmp.{c}.ts"], f"{c} tensor/scalar")
        assert_exact(A.scalar_cmp(code, s).numpy(), G[f"cmp.{c}.st"], f"{c} scalar/tensor")
    X = F.Tensor.from_numpy(G["cast.x"], F.CPU)
    for d in (1, 2, 3, 4):
        r = X.to_dtype(d)
        assert r.dtype == d
        assert_exact(r.numpy(), G[f"cast.{d}"], f"to(dtype {d})")
    assert X.to_dtype(F.FLOAT).dtype == F.FLOAT
    assert_exact(np.asarray([X[i].numpy()[0] for i in (0, 2, 1002)], np.float32), G["index.values"])
    assert X[5].shape == (1,)
    for d in range(5):
        t = F.Tensor.empty((5,), d, F.CPU)
        assert_exact(t.numpy().astype(np.float64), np.zeros(5), "zero-initialised")
        assert_exact(t.ones().numpy().astype(np.float64), G[f"ones.{d}"], f"ones of dtype {d}")
    # a non-float source converts to nothing and compares to all-false, as in the reference
    I = X.to_dtype(F.INT)
    assert_exact(I.to_dtype(F.DOUBLE).numpy(), np.zeros(X.shape, np.float64))
    assert not I._cmp(0, 0.0).numpy().any()


def test_front_end_errors():
    F = _frontend()
    a = F.Tensor.from_numpy(np.zeros((2, 3), np.float32), F.CPU)
    b = F.Tensor.from_numpy(np.zeros((3, 2), np.float32), F.CPU)
    with pytest.raises(F.FrontendError, match="shapes differ"):
        a > b
    with pytest.raises(F.FrontendError, match="dtypes differ"):
        a == a.to_dtype(F.INT)
    with pytest.raises(F.FrontendError, match="1-D"):
        a[0]
    v = F.Tensor.from_numpy(np.zeros(4, np.float32), F.CPU)
    with pytest.raises(F.FrontendError, match="out of range"):
        v[4]


# ---- GPU -------------------------------------------------------------------------------------------
@pytest.mark.gpu
@pytest.mark.parametrize("n,off", [(1, 0), (1000003, 0), (4099, 1), (77, 3), (1 << 22, 0)])
def test_compare_kernels(cb, n, off):
    rng = np.random.default_rng(n)
    a = rng.integers(-3, 4, n + off).astype(np.float32)
    b = rng.integers(-3, 4, n + off).astype(np.float32)
    a[off:off + 3] = [np.nan, np.inf, -0.0][:min(3, n)]
    b[off:off + 3] = [np.nan, np.inf, 0.0][:min(3, n)]
    dA, dB = cb.to_device(a).view(off, (n,)), cb.to_device(b).view(off, (n,))
    for c in oracle.CMP_NAMES:
        assert_exact(cb.ops.compare(c, dA, dB).numpy().astype(np.bool_), oracle.compare(c, a[off:], b[off:]), f"{c} tensor/tensor n={n}")
        assert_exact(cb.ops.compare(c, dA, 1.0).numpy().astype(np.bool_), oracle.compare(c, a[off:], 1.0), f"{c} tensor/scalar")
        assert_exact(cb.ops.compare(c, dA, 1.0, scalar_left=True).numpy().astype(np.bool_), oracle.compare(c, a[off:], 1.0, True), f"{c} scalar/tensor")


@pytest.mark.gpu
@pytest.mark.parametrize("n,off", [(1, 0), (1000003, 0), (4099, 1), (1 << 22, 0)])
def test_cast_kernels(cb, n, off):
    rng = np.random.default_rng(n + 1)
    x = (rng.standard_normal(n + off) * 1000).astype(np.float32)
    x[off:off + 4] = [0.0, -0.0, 0.5, -1.5][:min(4, n)]
    dX = cb.to_device(x).view(off, (n,))
    for d in (1, 2, 3, 4):
        got = cb.ops.cast(dX, d).numpy()
        want = oracle.cast_from_float(x[off:], d)
        assert_exact(got.astype(np.bool_) if d == 4 else got, want, f"to(dtype {d}) n={n}")
    for d, v in ((0, 1.0), (1, 1.0), (2, 1), (3, 1), (4, 1)):
        out = cb.DeviceArray((257,), cb.ops.DTYPES[d])
        assert_exact(cb.ops.fill_dtype(out, d, v).numpy().astype(np.float64), np.ones(257), f"typed fill {d}")


@pytest.mark.gpu
def test_rand_uniform_kernel(cb):
    n = 1 << 22
    a = cb.ops.rand_uniform((n,), seed=7).numpy()
    assert a.min() >= 0.0 and a.max() < 1.0
    assert abs(a.mean() - 0.5) < 1e-3 and abs(a.var() - 1 / 12) < 1e-3
    hist = np.histogram(a, bins=64, range=(0, 1))[0]
    assert np.abs(hist / (n / 64) - 1).max() < 0.02
    assert abs(np.corrcoef(a[:-1], a[1:])[0, 1]) < 2e-3
    assert_exact(cb.ops.rand_uniform((n,), seed=7).numpy(), a, "same seed, same numbers")
    # element i depends on (seed, offset + i) alone: a later window of the same stream
    assert_exact(cb.ops.rand_uniform((1000,), seed=7, offset=12345).numpy(), a[12345:13345], "offset continues the stream")
    assert not np.array_equal(cb.ops.rand_uniform((1000,), seed=8).numpy(), a[:1000])


@pytest.mark.gpu
def test_front_end_device_tensors(cb, golden):
    F = _frontend()
    G = golden
    A, B = F.Tensor.from_numpy(G["cmp.a"]), F.Tensor.from_numpy(G["cmp.b"])
    s = float(G["cmp.s"])
    for c in oracle.CMP_NAMES:
        code = CMP_CODE[c]
        r = A._cmp(code, B)
        assert r.dtype == F.BOOL and r.info()["device"] == F.CUDA
        assert_exact(r.numpy(), G[f"cmp.{c}.tt"], f"{c} tensor/tensor")
        assert_exact(A._cmp(code, s).numpy(), G[f"cmp.{c}.ts"], f"{c} tensor/scalar")
        assert_exact(A.scalar_cmp(code, s).numpy(), G[f"cmp.{c}.st"], f"{c} scalar/tensor")
    assert_exact((A > B).numpy(), G["cmp.gt.tt"])
    assert_exact((A != 1.0).numpy(), G["cmp.ne.ts"])
    X = F.Tensor.from_numpy(G["cast.x"])
    for d in (1, 2, 3, 4):
        r = X.to_dtype(d)
        assert r.dtype == d and r.info()["device"] == F.CUDA
        assert_exact(r.numpy(), G[f"cast.{d}"], f"to(dtype {d})")
    assert_exact(np.asarray([X[i].numpy()[0] for i in (0, 2, 1002)], np.float32), G["index.values"])
    for d in range(5):
        assert_exact(F.Tensor.empty((5,), d).ones().numpy().astype(np.float64), G[f"ones.{d}"], f"ones of dtype {d}")
    with pytest.raises(F.FrontendError, match="different devices"):
        A > F.Tensor.from_numpy(G["cmp.b"], F.CPU)


@pytest.mark.gpu
def test_front_end_rand(cb):
    F = _frontend()
    F.manual_seed(11)
    t = F.Tensor.empty((1 << 20,)).rand()
    a = t.numpy()
    assert a.min() >= 0.0 and a.max() < 1.0 and abs(a.mean() - 0.5) < 2e-3
    u = F.Tensor.empty((1 << 20,)).rand().numpy()
    assert not np.array_equal(a, u), "consecutive calls continue the stream"
    F.manual_seed(11)
    assert_exact(F.Tensor.empty((1 << 20,)).rand().numpy(), a, "manual_seed restarts the stream")
    d = F.Tensor.empty((4096,), F.DOUBLE).rand().numpy()
    assert d.dtype == np.float64 and d.min() >= 0.0 and d.max() < 1.0 and abs(d.mean() - 0.5) < 0.02
    i = F.Tensor.empty((16,), F.INT)
    assert_exact(i.rand().numpy(), np.zeros(16, np.int32), "other dtypes are left alone, as in the reference")
