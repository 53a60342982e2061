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


def test_matmul_path_choice_is_host_logic():
    """ctk_matmul_path only looks at pointers, extents and strides (it launches nothing): the four paths of
    ctk_matmul_f32 -- 0 tcgen05, 1 CUDA cores, 2 the K <= 16 kernel, 3 the N <= 16 kernels -- on made-up
    addresses."""
    import ctorch_b200 as cb
    L = cb.load()
    i64, P = ctypes.c_int64, ctypes.c_void_p
    MODE_3X, MODE_TF32 = 0, 1

    def path(m, k, n, ta=False, tb=False, mode=MODE_3X, a=1 << 20, b=1 << 24):
        sa = (1, m) if ta else (k, 1)
        sb = (1, k) if tb else (n, 1)
        return L.ctk_matmul_path(P(a), P(b), i64(m), i64(n), i64(k), i64(sa[0]), i64(sa[1]), i64(sb[0]), i64(sb[1]), mode)

    assert path(8192, 4096, 4096) == 0 and path(8192, 4096, 4096, ta=True, tb=True) == 0
    assert path(8192, 784, 4096, mode=MODE_TF32) == 0
    # neither stride of A is 1: the CUDA-core kernel
    assert L.ctk_matmul_path(P(1 << 20), P(1 << 24), i64(64), i64(64), i64(64), i64(130), i64(2), i64(64), i64(1), MODE_3X) == 1
    # dX of the 10-class layer: [B,10].[10,H] with both operands K-major
    assert path(8192, 10, 4096, tb=True) == 2
    assert path(64, 10, 4096, tb=True) == 0, "below 2^20 outputs the tensor-core kernel keeps it"
    assert path(8192, 10, 4096, tb=True, mode=MODE_TF32) != 2
    # logits and weight gradient of the 10-class layer
    assert path(8192, 4096, 10) == 3 and path(4096, 8192, 10, ta=True) == 3
    assert path(8192, 4096, 10, mode=MODE_TF32) != 3
    assert path(8192, 4096, 10, a=(1 << 20) + 4) == 0, "A not on a 16-byte boundary"
    assert path(8192, 4094, 10) == 0 and path(8192, 128, 10) == 0 and path(128, 4096, 10) == 0 and path(8192, 4096, 17) == 0


def test_split_tags_follow_the_setting_and_the_operand():
    """The tag a kept split carries: 1 + the correction setting, + 2 where the array itself serves as the
    split's hi part (16-byte aligned rows)."""
    import ctorch_b200 as cb
    L = cb.load()
    i64, P = ctypes.c_int64, ctypes.c_void_p
    start = L.ctk_get_matmul_correction()
    try:
        for setting in (0, 1):
            assert L.ctk_set_matmul_correction(setting) == 0
            base = L.ctk_matmul_split_tag()
            assert base == 1 + setting
            in_place = L.ctk_matmul_split_tag_for(P(1 << 20), i64(4096), i64(4096))
            assert in_place in (base, base + 2)          # base when CTORCH_MATMUL_HI_IN_PLACE=0
            if os.environ.get("CTORCH_MATMUL_HI_IN_PLACE", "1") != "0":
                assert in_place == base + 2
            assert L.ctk_matmul_split_tag_for(P((1 << 20) + 4), i64(4096), i64(4096)) == base   # unaligned start
            assert L.ctk_matmul_split_tag_for(P(1 << 20), i64(10), i64(10)) == base            # 40-byte rows
        assert L.ctk_set_matmul_correction(2) != 0
    finally:
        L.ctk_set_matmul_correction(start)
    # room for a split: 8 bytes per element of the larger padded view, whatever the setting
    assert L.ctk_matmul_split_bytes(i64(4096), i64(4096)) >= 8 * 4096 * 4096
    assert L.ctk_matmul_split_bytes(i64(8192), i64(10)) >= 8 * 8192 * 16
