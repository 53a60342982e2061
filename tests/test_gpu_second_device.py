"""One process driving two GPUs through ctk_set_device: set-up that belongs to a (kernel, device) pair
-- the opt-in shared-memory size of the tensor-core and long-row kernels, occupancy queries, the
library's per-device scratch and the caches of device buffers -- has to be repeated per device.
Skips on a box with one GPU."""
import ctypes

import numpy as np
import pytest

from conftest import assert_close, assert_matmul_close

pytestmark = pytest.mark.gpu


def _workload(cb, orc, tag):
    rng = np.random.default_rng(5)
    A = rng.standard_normal((384, 200)).astype(np.float32)
    B = rng.standard_normal((200, 512)).astype(np.float32)
    for mode, tol in (("3xtf32", 1e-4), ("tf32", 5e-3)):
        C = cb.ops.matmul(cb.to_device(A), cb.to_device(B), mode=mode).numpy()       # CTA-pair kernel
        assert_matmul_close(C, orc.matmul(A, B), tol, f"{tag}: {mode} product")
    S = rng.standard_normal((96, 40)).astype(np.float32)
    assert_matmul_close(cb.ops.matmul(cb.to_device(S), cb.to_device(B[:40]), mode="3xtf32").numpy(), orc.matmul(S, B[:40]), 1e-4, f"{tag}: single-CTA kernel")
    for cols in (12, 1000, 3000, 8196, 40000):                                        # every row holder
        L = (2 * rng.standard_normal((130, cols))).astype(np.float32)
        assert_close(cb.ops.softmax(cb.to_device(L)).numpy(), orc.softmax(L), 1e-5, 1e-9, f"{tag}: softmax, {cols} columns")
    x = rng.uniform(-4, 4, 100003).astype(np.float32)
    assert abs(float(cb.ops.sum(cb.to_device(x)).numpy()) - float(x.sum(dtype=np.float64))) <= 1e-5 * np.abs(x).sum()
    assert cb.ops.matmul_status() == 0 and cb.ops.rowwise_status() == 0


def test_kernels_on_a_second_device_of_the_same_process(cb, orc):
    n = ctypes.c_int()
    cb.check(cb.lib.ctk_device_count(ctypes.byref(n)))
    if n.value < 2:
        pytest.skip("needs 2 GPUs")
    from ctorch_b200 import frontend as F
    F.set_quiet(True)
    try:
        _workload(cb, orc, "device 0")
        t0 = F.Tensor.from_numpy(np.ones((64, 64), np.float32))      # parks buffers of device 0 in the caches when freed
        del t0
        cb.check(cb.lib.ctk_set_device(1))
        _workload(cb, orc, "device 1")
        t1 = F.Tensor.from_numpy(np.full((64, 64), 3.0, np.float32))  # same size: must not get device 0's buffer
        assert float(t1.sum().numpy()) == 3.0 * 64 * 64
        del t1
        cb.synchronize()
        cb.check(cb.lib.ctk_set_device(0))
        _workload(cb, orc, "device 0 again")
    finally:
        cb.check(cb.lib.ctk_set_device(0))
