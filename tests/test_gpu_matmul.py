"""GPU parity: MatMul forward and the two backward products, every operand major-ness, both tensor
core modes and the CUDA-core path, vs the oracle's fp32 recurrence.

Tolerances (normwise, max|C - C_ref| / max|C_ref|): 1e-4 for 3xTF32, 5e-3 for TF32, 1e-5 for the
fp32 CUDA-core path."""
import ctypes

import numpy as np
import pytest

from conftest import assert_exact, assert_matmul_close

pytestmark = pytest.mark.gpu

TOL = {"3xtf32": 1e-4, "tf32": 5e-3, "fp32_simt": 1e-5}


@pytest.fixture(autouse=True, params=["tf32-corrections", "bf16-corrections"])
def correction(cb, request):
    """Every test of this file runs with the correction terms of the fp32-accurate mode on either path."""
    before = cb.lib.ctk_get_matmul_correction()
    cb.ops.set_matmul_correction(1 if request.param.startswith("bf16") else 0)
    yield request.param
    cb.ops.set_matmul_correction(before)


def _mats(m, k, n, seed=0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32),
            rng.standard_normal((m, n)).astype(np.float32))


def _check_status(cb):
    assert cb.ops.matmul_status() == 0, "a bounded wait in the tensor-core kernel ran out"


@pytest.mark.parametrize("mode", ["tf32", "3xtf32"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,k,n", [(128, 32, 64), (128, 64, 128), (256, 96, 256), (384, 256, 512)])
def test_tensor_core_all_major_combinations(cb, orc, mode, ta, tb, m, k, n):
    A, B, _ = _mats(m, k, n, 1)
    sa = A.T.copy() if ta else A   # stored [k,m], viewed through t()
    sb = B.T.copy() if tb else B   # stored [n,k], viewed through t()
    dA, dB = cb.to_device(sa), cb.to_device(sb)
    assert cb.ops.matmul_path(dA, dB, ta, tb, mode) == 0, "expected the tcgen05 path"
    C = cb.ops.matmul(dA, dB, ta, tb, mode).numpy()
    _check_status(cb)
    assert_matmul_close(C, orc.matmul(sa, sb, ta, tb), TOL[mode], f"{mode} ta={ta} tb={tb} {m}x{k}x{n}")


@pytest.mark.parametrize("mode", ["tf32", "3xtf32"])
@pytest.mark.parametrize("m,k,n", [(64, 784, 128), (100, 40, 72), (129, 36, 260), (1, 8, 16), (300, 1000, 20), (130, 784, 4096)])
def test_tensor_core_ragged_extents(cb, orc, mode, m, k, n):
    """M, N, K that are not multiples of the tile: TMA zero fill on load, masked store."""
    A, B, _ = _mats(m, k, n, 2)
    dA, dB = cb.to_device(A), cb.to_device(B)
    assert cb.ops.matmul_path(dA, dB, False, False, mode) == 0
    C = cb.ops.matmul(dA, dB, mode=mode).numpy()
    _check_status(cb)
    assert_matmul_close(C, orc.matmul(A, B), TOL[mode], f"{mode} {m}x{k}x{n}")


@pytest.mark.parametrize("mode", ["tf32", "3xtf32"])
def test_forward_and_both_backward_products(cb, orc, mode):
    """C = A.B, dA = dC.B^T, dB = A^T.dC with the transposes as stride-swapped views (no copies)."""
    m, k, n = 320, 200, 264
    A, B, dC = _mats(m, k, n, 3)
    dA_, dB_, dC_ = cb.to_device(A), cb.to_device(B), cb.to_device(dC)
    assert_matmul_close(cb.ops.matmul(dA_, dB_, mode=mode).numpy(), orc.matmul(A, B), TOL[mode], "C")
    assert_matmul_close(cb.ops.matmul(dC_, dB_, tb=True, mode=mode).numpy(), orc.matmul(dC, B, tb=True), TOL[mode], "dA")
    assert_matmul_close(cb.ops.matmul(dA_, dC_, ta=True, mode=mode).numpy(), orc.matmul(A, dC, ta=True), TOL[mode], "dB")
    _check_status(cb)


def test_persistent_scheduler_many_tiles(cb, orc):
    """More tiles than SMs so each CTA loops over several tiles and both TMEM accumulators are used."""
    m, k, n = 2560, 64, 2304   # 20 x 9 = 180 tiles of 128 x 256
    A, B, _ = _mats(m, k, n, 4)
    rows = np.asarray([0, 1, 127, 128, 1279, 2559])
    for mode in ("tf32", "3xtf32"):
        C = cb.ops.matmul(cb.to_device(A), cb.to_device(B), mode=mode).numpy()
        _check_status(cb)
        assert_matmul_close(C[rows], orc.matmul_rows(A, B, rows), TOL[mode], mode + " sampled rows")
        # every tile against an fp64 product (catches a mis-addressed tile anywhere)
        ref64 = A.astype(np.float64) @ B.astype(np.float64)
        assert_matmul_close(C, ref64, TOL[mode] * 1.5, mode + " all tiles vs fp64")


@pytest.mark.parametrize("mode", ["tf32", "3xtf32"])
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_cta_pair_kernel_agrees_with_single_cta_kernel(cb, orc, mode, ta, tb):
    """The 256 x 256 CTA-pair kernel (default when m > 128 and n > 128) against the single-CTA kernel
    on the same operands: odd tile counts, ragged M/N/K, enough tiles that clusters loop and both
    accumulators are used; then both against the fp64 product and sampled oracle rows."""
    m, k, n = 2 * 256 * 5 + 130, 232, 256 * 17 + 72
    A, B, _ = _mats(m, k, n, 11)
    sa = A.T.copy() if ta else A
    sb = B.T.copy() if tb else B
    dA, dB = cb.to_device(sa), cb.to_device(sb)
    try:
        cb.ops.set_matmul_pairing(1)
        single = cb.ops.matmul(dA, dB, ta, tb, mode).numpy()
        cb.ops.set_matmul_pairing(0)
        paired = cb.ops.matmul(dA, dB, ta, tb, mode).numpy()
    finally:
        cb.ops.set_matmul_pairing(0)
    _check_status(cb)
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    assert_matmul_close(paired, ref64, TOL[mode] * 1.5, f"pair kernel vs fp64 {mode} ta={ta} tb={tb}")
    assert_matmul_close(single, ref64, TOL[mode] * 1.5, f"single-CTA kernel vs fp64 {mode} ta={ta} tb={tb}")
    assert_matmul_close(paired, single, 1e-6, "pair vs single-CTA kernel")
    rows = np.asarray([0, 127, 128, 255, 256, m - 1])
    assert_matmul_close(paired[rows], orc.matmul_rows(A, B, rows), TOL[mode], "sampled oracle rows")


@pytest.mark.parametrize("mode", ["tf32", "3xtf32"])
@pytest.mark.parametrize("pairing,m,k,n,ta,tb", [
    (0, 384, 520, 600, False, False),      # 4 pair tiles: every tile computed as two K-halves
    (0, 2560, 552, 2304, False, True),     # 90 pair tiles on 74 pairs: 74 whole + 16 halved
    (0, 2304, 1000, 2560, True, False),    # the weight-gradient shape: A^T.dC
    (1, 2560, 520, 2304, False, False),    # single-CTA kernel: 180 tiles on 148 SMs, 148 whole + 32 halved
    (0, 8192, 640, 20, False, False),      # a 20-class layer forward: 64 tiles of 128 x 64, all halved
    (0, 1024, 4100, 20, True, False),      # its weight gradient: 8 tiles, ragged K
])
def test_last_wave_in_k_halves(cb, orc, mode, pairing, m, k, n, ta, tb):
    """Tiles of a last wave that would fill at most half the machine are computed as two K-halves added
    into zeroed C: right, as close to the whole-tile result as two ways of cutting a long fp32 sum are,
    and bit-identical from call to call."""
    A, B, _ = _mats(m, k, n, 12)
    sa = A.T.copy() if ta else A
    sb = B.T.copy() if tb else B
    dA, dB = cb.to_device(sa), cb.to_device(sb)
    out = cb.empty((m, n))
    cb.ops.fill(out, 7.0)                  # stale contents must not leak into the sum
    try:
        cb.ops.set_matmul_pairing(pairing)
        cb.ops.set_matmul_tail_split(0)
        whole = cb.ops.matmul(dA, dB, ta, tb, mode).numpy()
        cb.ops.set_matmul_tail_split(2)    # halves wherever the shape allows (the default asks for a long contraction)
        halves = cb.ops.matmul(dA, dB, ta, tb, mode, out=out).numpy()
        again = cb.ops.matmul(dA, dB, ta, tb, mode, out=out).numpy()
    finally:
        cb.ops.set_matmul_pairing(0)
        cb.ops.set_matmul_tail_split(1)
    _check_status(cb)
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    assert_matmul_close(halves, ref64, TOL[mode] * 1.5, f"K-halves vs fp64 {mode} {m}x{k}x{n}")
    # (the tensor core's running fp32 sum is not correctly rounded, so where K is cut shows at the 1e-6..2e-5 level)
    assert_matmul_close(halves, whole, 5e-5, "K-halves vs whole tiles")
    assert np.array_equal(halves, again), "two addends: the result does not depend on which half lands first"


def test_three_tf32_terms_reach_fp32_accuracy(cb, orc):
    """K = 4096, N(0,1): 3xTF32 must sit with the fp32 recurrence, TF32 visibly must not need to."""
    m, k, n = 128, 4096, 256
    A, B, _ = _mats(m, k, n, 5)
    ref64 = A.astype(np.float64) @ B.astype(np.float64)
    e3 = assert_matmul_close(cb.ops.matmul(cb.to_device(A), cb.to_device(B), mode="3xtf32").numpy(), ref64, 1e-4, "3xtf32 vs fp64")
    e1 = assert_matmul_close(cb.ops.matmul(cb.to_device(A), cb.to_device(B), mode="tf32").numpy(), ref64, 5e-3, "tf32 vs fp64")
    eref = np.abs(orc.matmul(A, B) - ref64).max() / np.abs(ref64).max()
    assert e3 < 20 * max(eref, 1e-7), (e3, eref)
    assert e1 > e3
    _check_status(cb)


SKINNY = [(64, 128, 10, False, False), (64, 10, 128, False, True), (128, 64, 10, True, False), (5, 7, 3, False, False),
          (70, 33, 65, True, True), (1, 1, 1, False, False), (8192, 64, 10, False, False), (96, 2048, 10, True, False)]


@pytest.mark.parametrize("m,k,n,ta,tb", SKINNY)
def test_operands_tma_cannot_address_in_place(cb, orc, m, k, n, ta, tb):
    """The 10-class layer: row pitches of 40 bytes.  3xTF32 reads its own hi/lo copies, which are
    laid out for TMA whatever the source pitch, so these still run on the tensor cores; TF32 reads the
    caller's operands in place and hands them to the CUDA-core kernel (fp32 FMA, rel 1e-5)."""
    A, B, _ = _mats(m, k, n, 6)
    sa = A.T.copy() if ta else A
    sb = B.T.copy() if tb else B
    dA, dB = cb.to_device(sa), cb.to_device(sb)
    ref = orc.matmul(sa, sb, ta, tb)
    assert cb.ops.matmul_path(dA, dB, ta, tb, "3xtf32") == 0
    assert_matmul_close(cb.ops.matmul(dA, dB, ta, tb, "3xtf32").numpy(), ref, 1e-4, "3xTF32 through padded split copies")
    assert cb.ops.matmul_path(dA, dB, ta, tb, "tf32") == 1
    assert_matmul_close(cb.ops.matmul(dA, dB, ta, tb, "tf32").numpy(), ref, 1e-5, "CUDA cores (TF32 mode, not TMA-addressable)")
    assert_matmul_close(cb.ops.matmul(dA, dB, ta, tb, "fp32_simt").numpy(), ref, 1e-5, "CUDA cores forced")
    _check_status(cb)


def test_unaligned_base_pointers(cb, orc):
    """Operands that start 4 bytes into an allocation: no 16-byte alignment anywhere."""
    A, B, _ = _mats(130, 72, 40, 7)
    bufA = cb.to_device(np.concatenate([[0], A.ravel()]).astype(np.float32))
    bufB = cb.to_device(np.concatenate([[0], B.ravel()]).astype(np.float32))
    vA, vB = bufA.view(1, (130, 72)), bufB.view(1, (72, 40))
    ref = orc.matmul(A, B)
    assert_matmul_close(cb.ops.matmul(vA, vB, mode="3xtf32").numpy(), ref, 1e-4, "3xTF32, unaligned operands")
    assert_matmul_close(cb.ops.matmul(vA, vB, mode="tf32").numpy(), ref, 1e-5, "TF32 mode falls to CUDA cores")
    _check_status(cb)


def test_degenerate_extents(cb):
    A = cb.to_device(np.ones((4, 0), np.float32).reshape(4, 0))
    B = cb.to_device(np.ones((0, 8), np.float32).reshape(0, 8))
    C = cb.ops.matmul(cb.empty((4, 0)), cb.empty((0, 8)))
    assert (C.numpy() == 0).all()
    assert cb.ops.matmul(cb.empty((0, 5)), cb.empty((5, 3))).numpy().shape == (0, 3)


def test_against_golden_fixture(cb, golden):
    G = golden
    for tag in ("mm33x47x29", "mm64x100x16"):
        A, B, dC = cb.to_device(G[tag + ".A"]), cb.to_device(G[tag + ".B"]), cb.to_device(G[tag + ".dC"])
        assert_matmul_close(cb.ops.matmul(A, B).numpy(), G[tag + ".C"], 1e-4, tag + " C")
        assert_matmul_close(cb.ops.matmul(dC, B, tb=True).numpy(), G[tag + ".dA"], 1e-4, tag + " dA")
        assert_matmul_close(cb.ops.matmul(A, dC, ta=True).numpy(), G[tag + ".dB"], 1e-4, tag + " dB")
    _check_status(cb)


def test_a_wait_that_runs_out_is_reported_not_hung(cb):
    """Failure detection without a fault: the kernels' own bounded wait, on a barrier that nothing ever
    arrives on, gives up after its limit, records a code, raises the CTA-wide abort flag (which a second
    waiter honours at once), and the kernel returns normally: the context stays usable."""
    import ctypes
    res = (ctypes.c_int * 4)()
    cb.check(cb.lib.ctk_matmul_selftest_wait_timeout(res))
    assert list(res) == [0, 1, 0, 0x7e57]
    assert cb.ops.matmul_status() == 0, "the self-test restores the status word"
    A, B, _ = _mats(128, 64, 64, 13)
    C = cb.ops.matmul(cb.to_device(A), cb.to_device(B)).numpy()       # the device still works
    assert_matmul_close(C, A.astype(np.float64) @ B.astype(np.float64), 1e-4, "product after the self-test")


@pytest.mark.parametrize("pairing", [0, 1])
@pytest.mark.parametrize("m,k,n,ta,tb", [
    (256, 96, 320, False, False),
    (130, 64, 132, False, True),        # ragged rows, last column chunk of 4
    (384, 520, 600, True, False),
    (700, 40, 1000, False, True),       # the gradient product's shape: g.W^T
    (96, 33, 36, False, False),
])
def test_fused_epilogue_equals_the_separate_kernels(cb, m, k, n, ta, tb, pairing):
    """ctk_matmul_3xtf32_fused_f32: bias add, ReLU, the ReLU backward mask and the hi/lo split of the
    result in the product's epilogue, against the same product followed by the separate kernels (whole
    tiles on both sides) -- bit for bit, for every combination the front end uses."""
    A, B, _ = _mats(m, k, n, 21)
    rng = np.random.default_rng(m * n)
    bias = rng.standard_normal(n).astype(np.float32)
    y_act = np.maximum(rng.standard_normal((m, n)), 0).astype(np.float32)     # a ReLU output: zeros and positives
    dA, dB = cb.to_device(A.T.copy() if ta else A), cb.to_device(B.T.copy() if tb else B)
    dbias, dmask = cb.to_device(bias), cb.to_device(y_act)
    try:
        cb.ops.set_matmul_pairing(pairing)
        cb.ops.set_matmul_tail_split(0)
        plain = cb.ops.matmul(dA, dB, ta, tb, "3xtf32")
        biased = cb.ops.binary("Add", plain, dbias, cb.ops.B_ROW)
        relu = cb.ops.unary("ReLU", biased).numpy()
        masked = cb.ops.unary_backward("ReLU", dmask, plain).numpy()
        f_relu, hi, lo = cb.ops.matmul_fused(dA, dB, bias=dbias, relu=True, want_split=True, ta=ta, tb=tb)
        f_bias = cb.ops.matmul_fused(dA, dB, bias=dbias, ta=ta, tb=tb).numpy()
        f_mask, mhi, mlo = cb.ops.matmul_fused(dA, dB, mask=dmask, want_split=True, ta=ta, tb=tb)
    finally:
        cb.ops.set_matmul_pairing(0)
        cb.ops.set_matmul_tail_split(1)
    _check_status(cb)
    assert_exact(f_bias, biased.numpy(), "product + bias")
    assert_exact(f_relu.numpy(), relu, "relu(product + bias)")
    assert_exact(f_mask.numpy(), masked, "product * (y > 0)")
    for c, h, l, name in ((relu, hi, lo, "relu"), (masked, mhi, mlo, "masked")):
        eh, el = oracle_split(c)
        assert_exact(h, eh, f"{name}: hi part written by the epilogue")
        assert_exact(l, el, f"{name}: lo part written by the epilogue")


def oracle_split(x):
    """The split the library keeps of x, in the form ops._decode_split returns it.  hi = cvt.rna.tf32.f32
    of x (round to nearest, ties away from zero, 10 mantissa bits) where hi is an array of its own, x
    truncated to those bits where x itself is read as hi.  Correction terms on the TF32 path:
    lo = the same rounding of x - hi.  On the bf16 path: the bf16 bit patterns (round to nearest even)
    of hi and of x - hi."""
    import ctorch_b200 as cb_

    def rna(v):
        u = v.view(np.uint32).astype(np.uint64)
        r = ((u + 0x1000) & 0xFFFFE000).astype(np.uint32)
        out = r.view(np.float32).copy()
        special = ~np.isfinite(v)
        out[special] = v[special]
        return out

    def bf16_bits(v):
        u = np.ascontiguousarray(v, np.float32).view(np.uint32).astype(np.uint64)
        r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        nan = np.isnan(v)
        r[nan] = ((u[nan] >> 16) | 0x40).astype(np.uint16)
        return r

    x = np.ascontiguousarray(x, np.float32)
    # rows a multiple of 16 bytes apart (device arrays start on 256): the array itself is the hi part, read
    # by the tensor core with its low 13 mantissa bits ignored
    inner = x.shape[-1]
    in_place = cb_.lib.ctk_matmul_split_tag_for(None, ctypes.c_int64(inner), ctypes.c_int64(inner)) >= 3
    hi = (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32) if in_place else rna(x)
    lo = (x - hi).astype(np.float32)
    if cb_.lib.ctk_get_matmul_correction() == 0:
        return hi, rna(lo)
    return hi, np.stack([bf16_bits(hi), bf16_bits(lo)])


@pytest.mark.parametrize("outer,inner", [(784, 4096), (130, 132), (3, 4)])
def test_sgd_update_with_split_equals_update_then_split(cb, outer, inner):
    """ctk_sgd_update_split_f32: the same p as ctk_sgd_update_f32 bit for bit, and the hi/lo parts of
    that p; a product that takes the buffer as a kept split equals one that splits p itself."""
    rng = np.random.default_rng(outer)
    p0 = rng.standard_normal((outer, inner)).astype(np.float32)
    g = rng.standard_normal((outer, inner)).astype(np.float32)
    a, b, dg = cb.to_device(p0), cb.to_device(p0), cb.to_device(g)
    cb.ops.sgd_update(a, dg, 0.0123)
    hi, lo = cb.ops.sgd_update_split(b, dg, 0.0123)
    assert_exact(b.numpy(), a.numpy(), "updated weights")
    eh, el = oracle_split(a.numpy())
    assert_exact(hi, eh, "hi part of the updated weights")
    assert_exact(lo, el, "lo part of the updated weights")
    with pytest.raises(cb.CtkError):
        cb.ops.sgd_update_split(cb.to_device(p0[:, :inner - 1].copy()), dg, 0.1)   # rows not 16-byte aligned


@pytest.mark.parametrize("m,k,n,ta,tb", [
    (8192, 4096, 10, False, False),    # the logits of the 10-class layer
    (4096, 8192, 10, True, False),     # its weight gradient: H^T.dY
    (1027, 1028, 1, False, False), (2050, 516, 3, False, True), (4100, 260, 16, False, False), (33, 32768, 7, False, False),
    (1028, 1027, 1, True, False), (516, 2050, 13, True, True), (4096, 257, 16, True, False), (2052, 70000, 4, True, False),
])
def test_narrow_output_kernels(cb, orc, m, k, n, ta, tb):
    """N <= 16 over a long contraction (the 10-class layer's logits and weight gradient): the CUDA-core
    kernels that read A once as fp32 -- against float64, against sampled rows of the oracle's recurrence,
    and bit for bit against a second call (the partial sums over k are added in a fixed order)."""
    A, B, _ = _mats(m, k, n, 11)
    sa = A.T.copy() if ta else A
    sb = B.T.copy() if tb else B
    dA, dB = cb.to_device(sa), cb.to_device(sb)
    assert cb.ops.matmul_path(dA, dB, ta, tb, "3xtf32") == 3
    C = cb.ops.matmul(dA, dB, ta, tb, "3xtf32").numpy()
    again = cb.ops.matmul(dA, dB, ta, tb, "3xtf32").numpy()
    assert_exact(again, C, "two calls, same bits")
    assert_matmul_close(C, A.astype(np.float64) @ B.astype(np.float64), 1e-5, f"{m}x{k}x{n} vs float64")
    rows = np.asarray([0, m // 2, m - 1])
    assert_matmul_close(C[rows], orc.matmul_rows(sa, sb, rows, ta, tb), 1e-4, "sampled rows of the reference's recurrence")
    assert cb.ops.matmul_path(dA, dB, ta, tb, "tf32") != 3, "only the fp32-accurate mode"


def test_narrow_output_kernels_leave_the_other_shapes_alone(cb, orc):
    """An A that does not start on a 16-byte boundary, rows that are not whole 16-byte pieces, a short
    contraction, a small A or a wider output stay on the tensor-core kernel -- with the same result."""
    m, k, n = 2048, 1024, 10
    A, B, _ = _mats(m, k, n, 12)
    flat = cb.to_device(np.concatenate([np.zeros(1, np.float32), A.ravel()]))
    shifted = flat.view(1, (m, k))
    dB = cb.to_device(B)
    assert cb.ops.matmul_path(cb.to_device(A), dB, False, False, "3xtf32") == 3
    assert cb.ops.matmul_path(shifted, dB, False, False, "3xtf32") == 0
    assert_matmul_close(cb.ops.matmul(shifted, dB, mode="3xtf32").numpy(), A.astype(np.float64) @ B.astype(np.float64), 1e-4, "unaligned A")
    for mm, kk, nn in ((2048, 1022, 10), (8192, 128, 10), (512, 1024, 10), (2048, 1024, 17)):
        a, b, _ = _mats(mm, kk, nn, 13)
        assert cb.ops.matmul_path(cb.to_device(a), cb.to_device(b), False, False, "3xtf32") == 0, (mm, kk, nn)
    _check_status(cb)


@pytest.mark.parametrize("m,k,n", [(8192, 10, 4096), (2048, 16, 512), (4099, 1, 256), (1030, 7, 1020)])
def test_short_contraction_kernel_is_the_reference_recurrence(cb, orc, m, k, n):
    """K <= 16 with a large output (dX of the 10-class layer): the CUDA-core kernel, whose products and
    sums are rounded one by one in l order -- bit-identical to the reference's MatMul loop -- plain, with
    the ReLU-backward mask, and with the split of the result, each against the separate kernels."""
    rng = np.random.default_rng(m + k)
    g = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((n, k)).astype(np.float32)            # the right operand is w.t()
    y_act = np.maximum(rng.standard_normal((m, n)), 0).astype(np.float32)
    dG, dW, dM = cb.to_device(g), cb.to_device(w), cb.to_device(y_act)
    assert cb.ops.matmul_path(dG, dW, False, True, "3xtf32") == 2
    plain = cb.ops.matmul(dG, dW, tb=True, mode="3xtf32")
    rows = np.asarray([0, 1, m // 2, m - 1])
    assert_exact(plain.numpy()[rows], orc.matmul_rows(g, w, rows, tb=True), "sampled rows == the reference's recurrence")
    assert_matmul_close(plain.numpy(), g.astype(np.float64) @ w.T.astype(np.float64), 1e-6, "vs fp64")
    masked = cb.ops.unary_backward("ReLU", dM, plain).numpy()
    f_mask, hi, lo = cb.ops.matmul_fused(dG, dW, mask=dM, want_split=True, tb=True)
    assert_exact(f_mask.numpy(), masked, "product * (y > 0)")
    eh, el = oracle_split(masked)
    assert_exact(hi, eh, "hi part")
    assert_exact(lo, el, "lo part")
    _check_status(cb)
    # below 2^20 outputs, with another major-ness, or in TF32 mode the tensor-core kernel keeps the product
    small = cb.to_device(g[:64].copy())
    assert cb.ops.matmul_path(small, dW, False, True, "3xtf32") == 0
    assert cb.ops.matmul_path(dG, cb.to_device(w.T.copy()), False, False, "3xtf32") == 0
    assert cb.ops.matmul_path(dG, dW, False, True, "tf32") != 2
