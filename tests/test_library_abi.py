"""CPU tests of the drop-in boundary: the shared library loads and exports every symbol the public
header declares (no compute calls: there is no GPU here)."""
import ctypes
import os

import pytest


def test_library_is_built_and_exports_every_declared_symbol():
    import ctorch_b200 as cb
    from ctorch_b200._lib import declared_symbols
    assert os.path.exists(cb.LIB_PATH), "run `python -m ctorch_b200.build`"
    L = cb.load()
    names = declared_symbols()
    assert len(names) >= 50
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_no_cpu_fallback_without_a_device():
    """Without a usable CUDA device every entry point reports an error instead of computing."""
    import ctorch_b200 as cb
    n = ctypes.c_int(-1)
    st = cb.lib.ctk_device_count(ctypes.byref(n))
    if st == 0 and n.value > 0:
        pytest.skip("a CUDA device is present")
    with pytest.raises(cb.CtkError):
        cb.check(cb.lib.ctk_device_sync())
    assert cb.lib.ctk_last_error()


def test_argument_validation_needs_no_device():
    import ctorch_b200 as cb
    L = cb.load()
    i64 = ctypes.c_int64
    assert L.ctk_binary_f32(0, None, None, None, i64(-1), 0, i64(0), None) == 1       # negative size
    assert L.ctk_binary_f32(99, ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), i64(4), 0, i64(0), None) in (1, 2)
    assert L.ctk_set_matmul_mode(7) == 1
    assert L.ctk_set_matmul_mode(0) == 0
    assert L.ctk_matmul_f32(None, None, None, i64(-1), i64(1), i64(1), i64(1), i64(1), i64(1), i64(1), 0, None, None) == 1
    assert b"negative" in L.ctk_last_error()
    assert L.ctk_matmul_workspace_bytes(i64(8), i64(8), i64(8), 1) == 0
    assert L.ctk_matmul_workspace_bytes(i64(8), i64(8), i64(8), 0) >= 2 * 128 * 4


def test_buffer_caches_are_keyed_by_device():
    """The caches that recycle device buffers never hand a buffer parked on one GPU to a request made
    with another GPU current (a fake allocator and a fake current device: no GPU is touched)."""
    import ctorch_b200 as cb
    failed = ctypes.c_int(-1)
    assert cb.lib.cth_selftest_cache_keying(ctypes.byref(failed)) == 0, cb.lib.cth_last_error()
    assert failed.value == 0


def test_oracle_is_not_reachable_from_the_product():
    """No file of the product package mentions the oracle."""
    import ctorch_b200 as cb
    pkg = os.path.dirname(cb.__file__)
    for root, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(root, f), errors="replace").read()
                assert "oracle" not in text.lower() or f == "__init__.py" and "oracle" not in text, os.path.join(root, f)
