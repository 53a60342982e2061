import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden():
    return dict(np.load(os.path.join(ROOT, "tests", "golden", "golden.npz")))


@pytest.fixture(scope="session")
def orc():
    import oracle
    return oracle.Oracle()


@pytest.fixture(scope="session")
def cb():
    """The product library on cuda:0.  GPU tests fail (not skip) if it cannot run."""
    import ctorch_b200 as m
    import ctypes
    n = ctypes.c_int()
    m.check(m.lib.ctk_device_count(ctypes.byref(n)))
    assert n.value >= 1, "no CUDA device"
    m.check(m.lib.ctk_set_device(0))
    return m


# ---- tolerances (written once, used by every parity test) -------------------------------------
def assert_exact(got, ref, what=""):
    got, ref = np.asarray(got), np.asarray(ref)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    same = (got == ref) | (np.isnan(got) & np.isnan(ref))
    assert same.all(), f"{what}: {np.count_nonzero(~same)} of {got.size} elements differ, first at {np.argwhere(~same)[0]}"


def assert_close(got, ref, rel=1e-5, abs_=1e-6, what=""):
    """|got - ref| <= rel*|ref| + abs_ elementwise (elementwise / reduction tolerance: rel 1e-5)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    err = np.abs(got - ref)
    bound = rel * np.abs(ref) + abs_
    bad = ~((err <= bound) | (np.isnan(got) & np.isnan(ref)) | ((got == ref)))
    assert not bad.any(), f"{what}: {np.count_nonzero(bad)} of {got.size} out of tolerance, worst err {err[bad].max():.3e} (rel={rel}, abs={abs_})"


def assert_matmul_close(got, ref, tol, what=""):
    """max|got - ref| / max|ref| <= tol (MatMul and gradient tolerance: 1e-4 for 3xTF32, 5e-3 for TF32)."""
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    denom = max(np.abs(ref).max(), 1e-30)
    e = np.abs(got - ref).max() / denom
    assert e <= tol, f"{what}: normwise error {e:.3e} > {tol}"
    return e


def assert_sum_close(got, ref_seq, values64, what=""):
    """A scalar sum passes if it is within rel 1e-5 of the fp64 sum, or at least as accurate as the
    reference's sequential fp32 sum (whose own error grows with n)."""
    s64 = float(values64)
    eg, er = abs(float(got) - s64), abs(float(ref_seq) - s64)
    assert eg <= 1e-5 * abs(s64) + 1e-6 or eg <= er, f"{what}: gpu {got} ref {ref_seq} fp64 {s64}"
