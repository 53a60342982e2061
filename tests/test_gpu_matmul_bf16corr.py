"""GPU parity of the fp32-accurate MatMul with its correction terms on the bf16 path
(ctk_set_matmul_correction(1)): hi.hi as one TF32 product plus l16.h16 + h16.l16 as two bf16
products, against the oracle's fp32 recurrence and float64 -- every operand major-ness, both
tensor-core kernels, ragged extents, K-chunks and K-halves, the fused epilogues, kept splits through
the front end, and a training run.  Tolerance: the 1e-4 (normwise) of the fp32-accurate mode."""
import numpy as np
import pytest

import oracle
from conftest import assert_close, assert_exact, assert_matmul_close

pytestmark = pytest.mark.gpu
TOL = 1e-4


@pytest.fixture(autouse=True)
def bf16_corrections(cb):
    cb.ops.set_matmul_correction(1)
    yield
    cb.ops.set_matmul_correction(0)


def _mats(m, k, n, seed=0):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32),
            rng.standard_normal((m, n)).astype(np.float32))


def _ok(cb):
    assert cb.ops.matmul_status() == 0, "a bounded wait in the tensor-core kernel ran out"


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,k,n", [(128, 32, 64), (128, 64, 128), (256, 96, 256), (384, 256, 512), (130, 72, 40), (520, 200, 300)])
def test_all_major_combinations(cb, orc, ta, tb, m, k, n):
    A, B, _ = _mats(m, k, n, 1)
    sa = A.T.copy() if ta else A
    sb = B.T.copy() if tb else B
    dA, dB = cb.to_device(sa), cb.to_device(sb)
    assert cb.ops.matmul_path(dA, dB, ta, tb, "3xtf32") == 0, "expected the tcgen05 path"
    C = cb.ops.matmul(dA, dB, ta, tb, "3xtf32").numpy()
    _ok(cb)
    assert_matmul_close(C, orc.matmul(sa, sb, ta, tb), TOL, f"ta={ta} tb={tb} {m}x{k}x{n}")
    assert_matmul_close(C, A.astype(np.float64) @ B.astype(np.float64), TOL, "vs float64")


@pytest.mark.parametrize("m,k,n", [(64, 784, 128), (100, 40, 72), (129, 36, 260), (1, 8, 16), (300, 1000, 20), (130, 784, 4096), (8192, 784, 10)])
def test_ragged_extents(cb, orc, m, k, n):
    A, B, _ = _mats(m, k, n, 2)
    C = cb.ops.matmul(cb.to_device(A), cb.to_device(B), mode="3xtf32").numpy()
    _ok(cb)
    assert_matmul_close(C, A.astype(np.float64) @ B.astype(np.float64), TOL, f"{m}x{k}x{n}")


@pytest.mark.parametrize("pairing,m,k,n,ta,tb", [
    (0, 384, 520, 600, False, False),      # 4 pair tiles: every tile computed as two K-halves
    (0, 2560, 552, 2304, False, True),     # 90 pair tiles on 74 pairs: 74 whole + 16 halved
    (0, 2304, 1000, 2560, True, False),    # the weight-gradient shape: A^T.dC
    (1, 2560, 520, 2304, False, False),    # single-CTA kernel: 148 whole + 32 halved
    (0, 512, 5000, 512, False, False),     # K-chunks (three per tile) and K-halves together
    (0, 1024, 4500, 2560, True, True),     # whole tiles with three K-chunks each
])
def test_halves_chunks_and_pairs(cb, orc, pairing, m, k, n, ta, tb):
    A, B, _ = _mats(m, k, n, 5)
    sa = A.T.copy() if ta else A
    sb = B.T.copy() if tb else B
    dA, dB = cb.to_device(sa), cb.to_device(sb)
    try:
        cb.ops.set_matmul_pairing(pairing)
        cb.ops.set_matmul_tail_split(2)    # halves wherever the shape allows
        C = cb.ops.matmul(dA, dB, ta, tb, "3xtf32").numpy()
        again = cb.ops.matmul(dA, dB, ta, tb, "3xtf32").numpy()
    finally:
        cb.ops.set_matmul_pairing(0)
        cb.ops.set_matmul_tail_split(1)
    _ok(cb)
    assert_exact(again, C, "two calls, same bits")
    assert_matmul_close(C, A.astype(np.float64) @ B.astype(np.float64), TOL, f"{m}x{k}x{n} vs float64")
    rows = np.asarray([0, 127, 128, m - 1])
    assert_matmul_close(C[rows], orc.matmul_rows(sa, sb, rows, ta, tb), TOL, "sampled oracle rows")


def test_accuracy_next_to_the_tf32_corrections(cb):
    """4096^3, N(0,1): the error of both variants of the fp32-accurate mode against float64 on sampled
    rows (printed), each within 1e-4."""
    m = k = n = 4096
    A, B, _ = _mats(m, k, n, 9)
    dA, dB = cb.to_device(A), cb.to_device(B)
    rows = np.asarray([0, 1, 777, 2048, 4095])
    ref = A[rows].astype(np.float64) @ B.astype(np.float64)
    errs = {}
    for corr in (0, 1):
        cb.ops.set_matmul_correction(corr)
        C = cb.ops.matmul(dA, dB, mode="3xtf32").numpy()
        errs["bf16" if corr else "tf32"] = float(np.abs(C[rows] - ref).max() / np.abs(ref).max())
    _ok(cb)
    print(f"\nnormwise error vs float64 at 4096^3, correction terms on the tf32 / bf16 path: {errs['tf32']:.2e} / {errs['bf16']:.2e}")
    assert errs["tf32"] <= TOL and errs["bf16"] <= TOL


def _device_masks(F, x, Ws, bs):
    h = F.Tensor.from_numpy(x)
    masks = []
    for l in range(len(Ws) - 1):
        h = h.linear(F.Tensor.from_numpy(Ws[l]), F.Tensor.from_numpy(bs[l]), True)
        masks.append(h.numpy() > 0)
    return masks


def test_fused_epilogues_and_kept_splits_through_the_front_end(cb):
    """Two training steps of a small MLP (fused linear layers, the ReLU-backward mask and the split of
    results written by epilogues, the weights' split written by the SGD update and read by the second
    step): loss, gradients and weights of each step against a float64 evaluation of that step with the
    reference's semantics.  (float64 with the device's own on/off decisions of the hidden units, not a
    multi-step oracle run: one unit within rounding distance of 0 changes a gradient column by ~1 %.)"""
    from ctorch_b200 import frontend as F
    from test_gpu_fullsize import _fp64_step
    F.set_quiet(True)
    dims, batch, lr = [784, 256, 192, 10], 512, 1e-4
    rng = np.random.default_rng(21)
    Ws, bs = [], []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        Ws.append(rng.uniform(-lim, lim, (i, j)).astype(np.float32))
        bs.append((0.01 * rng.standard_normal(j)).astype(np.float32))
    W0 = [w.copy() for w in Ws]
    tr = F.MlpTrainer(dims, oracle.pack_params(Ws, bs), lr)
    for step in range(2):
        x = rng.integers(0, 256, (batch, dims[0])).astype(np.float32) / np.float32(255.0)
        lab = rng.integers(0, dims[-1], batch).astype(np.float32)
        masks = _device_masks(F, x, Ws, bs)
        _, loss64, gW, gb, newW, newb, flips = _fp64_step(dims, x, lab, Ws, bs, lr, masks, Ws_back=W0)
        loss = tr.step_host(x, lab)
        assert abs(loss - loss64) <= 1e-4 * abs(loss64), (step, loss, loss64)
        gW_d, gb_d = oracle.unpack_params(tr.grads(), dims)
        W_d, b_d = oracle.unpack_params(tr.params(), dims)
        for l in range(len(Ws)):
            assert_matmul_close(gW_d[l], gW[l], TOL, f"step {step}: dW{l}")
            assert_matmul_close(gb_d[l], gb[l], TOL, f"step {step}: db{l}")
            assert_matmul_close(W_d[l], newW[l], TOL, f"step {step}: updated W{l}")
        Ws, bs = [w.copy() for w in W_d], [b.copy() for b in b_d]   # the next step starts from the device's weights
    _ok(cb)


def test_switching_the_setting_refills_kept_splits(cb):
    """A split kept under one setting is not reused under the other (its tag differs): the same tensors
    multiplied before and after a switch give each setting's own result."""
    from ctorch_b200 import frontend as F
    F.set_quiet(True)
    A, B, _ = _mats(256, 320, 384, 3)
    X, W = F.Tensor.from_numpy(A), F.Tensor.from_numpy(B)
    c1 = X.matmul(W).numpy()                 # bf16 corrections (the fixture), splits kept with tag 2
    cb.ops.set_matmul_correction(0)
    c0 = X.matmul(W).numpy()                 # must refill: tag 1
    fresh0 = F.Tensor.from_numpy(A).matmul(F.Tensor.from_numpy(B)).numpy()
    assert_exact(c0, fresh0, "after the switch the kept splits were made again")
    cb.ops.set_matmul_correction(1)
    assert_exact(X.matmul(W).numpy(), c1, "and again on the way back")
    ref = A.astype(np.float64) @ B.astype(np.float64)
    assert_matmul_close(c0, ref, TOL, "tf32 corrections")
    assert_matmul_close(c1, ref, TOL, "bf16 corrections")
