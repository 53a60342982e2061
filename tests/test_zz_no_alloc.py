"""GPU test of ctk_matmul_3xtf32_noalloc_f32, the 3xTF32 MatMul for hosts that must not allocate.

Some callers of this library cannot tolerate a device allocation made on their behalf: code that is
recording a CUDA graph, servers that give all GPU memory to their own allocator at start-up, and
tight loops where a workspace that grows means a device-wide stall.  For them the split scratch of
the 3xTF32 product sits in a 16 MiB array inside the library (enough for 1024 x 1024 operands).  This file checks, through the C ABI,
that the entry point returns what the ordinary one returns -- twice in a row on different operands,
because the array keeps whatever the previous call left in it -- and that operands too large for the
array are refused before anything is launched.

Kept in a file of its own that sorts last, so a run that stops at the first failure has already been
through every other test."""
import ctypes

import numpy as np
import pytest

from conftest import assert_matmul_close

pytestmark = pytest.mark.gpu

i64 = ctypes.c_int64
LIMIT_BYTES = (16 << 20) + 1024  # 16 MiB of split floats plus the workspace's 1 KiB alignment slack


def _noalloc(cb, A, B, ta=False, tb=False):
    m, k = (A.shape[1], A.shape[0]) if ta else A.shape
    n = B.shape[0] if tb else B.shape[1]
    sa = (1, m) if ta else (k, 1)
    sb = (1, k) if tb else (n, 1)
    C = cb.empty((m, n))
    cb.check(cb.lib.ctk_matmul_3xtf32_noalloc_f32(A.p, B.p, C.p, i64(m), i64(n), i64(k), i64(sa[0]), i64(sa[1]), i64(sb[0]), i64(sb[1]), None))
    return C


def test_same_result_as_the_allocating_entry_point_twice_in_a_row(cb, orc):
    rng = np.random.default_rng(123)
    # second call: other shapes, other major-ness, so it reads scratch the first call left dirty
    for (m, k, n, ta, tb) in ((384, 200, 512, False, False), (256, 320, 136, True, True)):
        A = rng.standard_normal((m, k)).astype(np.float32)
        B = rng.standard_normal((k, n)).astype(np.float32)
        sa = A.T.copy() if ta else A
        sb = B.T.copy() if tb else B
        dA, dB = cb.to_device(sa), cb.to_device(sb)
        assert cb.ops.matmul_path(dA, dB, ta, tb, "3xtf32") == 0, "this shape should take the tensor-core path"
        got = _noalloc(cb, dA, dB, ta, tb).numpy()
        want = cb.ops.matmul(dA, dB, ta, tb, "3xtf32").numpy()
        assert_matmul_close(got, want, 1e-4, "fixed-scratch entry point vs ctk_matmul_f32")
        assert np.array_equal(got, want), "same kernels on the same data: the bits should agree too"
        assert_matmul_close(got, orc.matmul(sa, sb, ta, tb), 1e-4, "fixed-scratch entry point vs the oracle")
    assert cb.ops.matmul_status() == 0


def _free_bytes(cb):
    sms, total, free = ctypes.c_int(), ctypes.c_size_t(), ctypes.c_size_t()
    cb.check(cb.lib.ctk_device_info(ctypes.byref(sms), ctypes.byref(total), ctypes.byref(free)))
    return free.value


def test_largest_admissible_shape_and_nothing_is_allocated(cb, orc):
    """1024 x 1024 by 1024 x 1024 fills the fixed array to the last byte.  The first call may set
    kernel attributes; across the second and third the device's free memory must not move (the
    library neither grows a workspace nor takes anything from the driver on this path)."""
    rng = np.random.default_rng(7)
    A = rng.standard_normal((1024, 1024)).astype(np.float32)
    B = rng.standard_normal((1024, 1024)).astype(np.float32)
    dA, dB = cb.to_device(A), cb.to_device(B)
    C = cb.empty((1024, 1024))
    want = cb.ops.matmul(dA, dB, mode="3xtf32").numpy()
    args = (dA.p, dB.p, C.p, i64(1024), i64(1024), i64(1024), i64(1024), i64(1), i64(1024), i64(1), None)
    cb.check(cb.lib.ctk_matmul_3xtf32_noalloc_f32(*args))
    cb.synchronize()
    free0 = _free_bytes(cb)
    for _ in range(2):
        C.fill_bytes(0)
        cb.check(cb.lib.ctk_matmul_3xtf32_noalloc_f32(*args))
        cb.synchronize()
        assert _free_bytes(cb) == free0, "the call changed the device's free memory"
        got = C.numpy()
        assert np.array_equal(got, want)
    assert_matmul_close(got, orc.matmul(A, B), 1e-4, "1024^3 through the fixed scratch vs the oracle")
    assert cb.ops.matmul_status() == 0


def test_operands_beyond_the_fixed_scratch_are_refused(cb):
    m = n = k = 2048  # 2*(m*k + k*n)*4 bytes = 64 MiB of split scratch
    assert cb.lib.ctk_matmul_workspace_bytes(m, n, k, 0) > LIMIT_BYTES
    # real-size operands: should the size check ever move behind a launch, the call computes a product
    # (and this test fails on the return code) instead of reading past small buffers
    a, b, c = cb.empty((m, k)), cb.empty((k, n)), cb.empty((m, n))
    before = cb.launch_count()
    rc = cb.lib.ctk_matmul_3xtf32_noalloc_f32(a.p, b.p, c.p, i64(m), i64(n), i64(k), i64(k), i64(1), i64(n), i64(1), None)
    assert rc == 5, "CTK_ERR_LIMIT expected"
    msg = cb.lib.ctk_last_error().decode()
    assert "fixed array" in msg and str(LIMIT_BYTES) in msg, msg
    assert cb.launch_count() == before, "nothing may be launched for a refused call"
    # the largest square that still fits: 1024^3
    assert cb.lib.ctk_matmul_workspace_bytes(1024, 1024, 1024, 0) <= LIMIT_BYTES
