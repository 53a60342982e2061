"""GPU parity: row-wise Softmax / CrossEntropy forward and backward vs the oracle (rel 1e-5)."""
import numpy as np
import pytest

from conftest import assert_close, assert_exact

pytestmark = pytest.mark.gpu

# cols chosen to hit every kernel shape: sub-warp groups (<=8, <=16, <=32), CTA register rows up to
# 4096, the streamed long-row kernel (4097..32768, rows 16-byte aligned: whole and ragged 8 KiB
# chunks, more rows than SMs so every CTA walks several rows and the ring wraps), shared-memory rows
# (unaligned, up to 48K) and the re-reading path (>48K); odd values exercise the unaligned-row loads.
SHAPES = [(1, 1), (5, 3), (300, 10), (7, 16), (9, 31), (33, 100), (64, 1000), (17, 1024), (6, 1025), (700, 2048), (5, 4095),
          (310, 4100), (160, 8196), (40, 16384), (21, 20000), (5, 32000), (300, 32768), (4, 5001), (3, 50001)]


def _case(rows, cols, seed=0):
    rng = np.random.default_rng(seed)
    L = (2 * rng.standard_normal((rows, cols))).astype(np.float32)
    lab = rng.integers(0, cols, rows)
    oh = np.zeros((rows, cols), np.float32)
    oh[np.arange(rows), lab] = 1
    g = rng.standard_normal((rows, cols)).astype(np.float32)
    return L, lab.astype(np.float32), oh, g


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_softmax_forward_backward(cb, orc, rows, cols):
    L, _, _, g = _case(rows, cols)
    y = cb.ops.softmax(cb.to_device(L))
    ref = orc.softmax(L)
    assert_close(y.numpy(), ref, 1e-5, 1e-9, f"softmax {rows}x{cols}")
    assert_close(y.numpy().sum(axis=1), np.ones(rows), 1e-5, 0, "rows sum to 1")
    dx = cb.ops.softmax_backward(cb.to_device(ref), cb.to_device(g))
    # y*(g - dot) cancels: bound the error by the size of the terms, rel 1e-5 of max|g|*y
    refdx = orc.grad_unary("Softmax", L, g)
    assert np.abs(dx.numpy() - refdx).max() <= 1e-5 * np.abs(g).max() * ref.max() + 1e-9, "softmax backward"
    assert cb.ops.rowwise_status() == 0, "a bounded wait in the long-row kernel ran out"


@pytest.mark.parametrize("rows,cols", SHAPES)
def test_cross_entropy_forward_backward(cb, orc, rows, cols):
    L, lab, oh, _ = _case(rows, cols, 1)
    dL, dlab, doh = cb.to_device(L), cb.to_device(lab), cb.to_device(oh)
    assert_close(cb.ops.cross_entropy(dL, doh).numpy(), orc.ce(L, oh), 1e-5, 1e-6, f"CE one-hot {rows}x{cols}")
    assert_close(cb.ops.cross_entropy(dL, dlab).numpy(), orc.ce(L, lab), 1e-5, 1e-6, "CE index")
    ref_d = orc.grad_loss("CE", L, oh, 1.0)
    assert_close(cb.ops.cross_entropy_backward(dL, doh).numpy(), ref_d, 1e-5, 1e-7, "CE backward")
    gdev = cb.to_device(np.asarray(0.37, np.float32))
    assert_close(cb.ops.cross_entropy_backward(dL, doh, gdev).numpy(), orc.grad_loss("CE", L, oh, 0.37), 1e-5, 1e-7, "CE backward * g")
    loss, d = cb.ops.cross_entropy_fused(dL, dlab)
    assert_close(loss.numpy(), orc.ce(L, oh), 1e-5, 1e-6, "fused loss == one-hot reference")
    assert_close(d.numpy(), ref_d, 1e-5, 1e-7, "fused dlogits == one-hot reference")
    assert cb.ops.rowwise_status() == 0, "a bounded wait in the long-row kernel ran out"


def test_soft_targets_and_probability_clamp(cb, orc):
    rng = np.random.default_rng(2)
    L = (2 * rng.standard_normal((40, 50))).astype(np.float32)
    t = rng.uniform(0, 1, (40, 50)).astype(np.float32)
    assert_close(cb.ops.cross_entropy(cb.to_device(L), cb.to_device(t)).numpy(), orc.ce(L, t), 1e-5, 1e-6, "soft targets")
    L2 = np.zeros((2, 4), np.float32)
    L2[:, 0] = 200.0  # p of the other classes underflows to 0 -> clamped at 1e-10
    t2 = np.zeros((2, 4), np.float32)
    t2[:, 3] = 1
    assert_close(cb.ops.cross_entropy(cb.to_device(L2), cb.to_device(t2)).numpy(), orc.ce(L2, t2), 1e-5, 1e-6, "clamp")
    assert_close(cb.ops.cross_entropy(cb.to_device(L2), cb.to_device(np.asarray([3, 3], np.float32))).numpy(),
                 orc.ce(L2, np.asarray([3, 3], np.float32)), 1e-5, 1e-6, "clamp, index labels")


def test_out_of_range_label_is_reported(cb, orc):
    L = np.zeros((3, 5), np.float32)
    flag = cb.zeros((1,), np.int32)
    out = cb.ops.cross_entropy(cb.to_device(L), cb.to_device(np.asarray([0, 5, 1], np.float32)), bad_flag=flag)
    assert np.isnan(out.numpy())
    assert flag.numpy()[0] == 1
    with pytest.raises(ValueError):
        orc.ce(L, np.asarray([0, 5, 1], np.float32))


def test_empty_rows(cb):
    e = cb.empty((0, 7))
    assert cb.ops.softmax(e).numpy().shape == (0, 7)
    out = cb.ops.cross_entropy(e, cb.empty((0, 7)))
    assert float(out.numpy()) == 0.0


def test_config_shapes_at_reduced_rows(cb, orc):
    """[rows, C] for C in {10, 1000, 32000} as in the row-wise benchmark config, logits ~ N(0, 2^2)."""
    for rows, C in ((4096, 10), (512, 1000), (24, 32000)):
        L, lab, oh, g = _case(rows, C, 3)
        assert_close(cb.ops.softmax(cb.to_device(L)).numpy(), orc.softmax(L), 1e-5, 1e-9, f"softmax C={C}")
        assert_close(cb.ops.cross_entropy(cb.to_device(L), cb.to_device(lab)).numpy(), orc.ce(L, lab), 1e-5, 1e-6, f"CE C={C}")


def test_against_golden_fixture(cb, golden):
    G = golden
    for C in (10, 130):
        L, oh, lab = cb.to_device(G[f"rw{C}.logits"]), cb.to_device(G[f"rw{C}.onehot"]), cb.to_device(G[f"rw{C}.labels"])
        assert_close(cb.ops.softmax(L).numpy(), G[f"rw{C}.softmax"], 1e-5, 1e-9, "softmax")
        assert_close(cb.ops.cross_entropy(L, oh).numpy(), G[f"rw{C}.ce_onehot"], 1e-5, 1e-6, "ce onehot")
        assert_close(cb.ops.cross_entropy(L, lab).numpy(), G[f"rw{C}.ce_index"], 1e-5, 1e-6, "ce index")
        assert_close(cb.ops.cross_entropy_backward(L, oh).numpy(), G[f"rw{C}.ce.dlogits"], 1e-5, 1e-7, "ce dlogits")
    # known answer of the reference's own test (src/tests/test_activation_loss.cpp:156-189)
    z, t = cb.to_device(G["ka.ce.z"]), cb.to_device(G["ka.ce.t"])
    assert_close(cb.ops.cross_entropy(z, t).numpy(), G["ka.ce"], 1e-5, 1e-6, "CE({2,1,0.1},{1,0,0})")
    assert np.abs(cb.ops.cross_entropy_backward(z, t).numpy() - G["ka.ce.grad"]).max() < 1e-4


@pytest.mark.parametrize("rows,cols", [(1, 1), (2, 3), (37, 19), (1000, 10), (64, 33), (5, 1000), (4099, 70), (257, 5), (8192, 64)])
def test_softmax_down_the_columns(cb, orc, rows, cols):
    """Tensor::softmax(0) (src/Tensor.cpp:1728-1743) and its backward (src/AutoDiff.cpp:1473-1484),
    through the kernels and through the front end's tape."""
    from ctorch_b200 import frontend as F
    rng = np.random.default_rng(rows * 31 + cols)
    x = (2 * rng.standard_normal((rows, cols))).astype(np.float32)
    g = rng.standard_normal((rows, cols)).astype(np.float32)
    ref_y, ref_dx = orc.softmax_dim0(x, g)
    with F.AutoDiff():
        X = F.Tensor.from_numpy(x).requires_grad()
        Y = X.softmax(0)
        assert_close(Y.numpy(), ref_y, 1e-5, 1e-9, f"softmax(0) {rows}x{cols}")
        assert_close(Y.numpy().sum(axis=0), np.ones(cols), 1e-5, 0, "columns sum to 1")
        F.backward(Y, F.Tensor.from_numpy(g))
        dx = F.grad(X).numpy()
    assert np.abs(dx - ref_dx).max() <= 1e-5 * np.abs(g).max() * ref_y.max() * max(1.0, np.sqrt(rows) / 8) + 1e-9, "softmax(0) backward"
