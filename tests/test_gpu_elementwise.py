"""GPU parity: elementwise forward/backward and scalar reductions through the C ABI vs the oracle."""
import numpy as np
import pytest

from conftest import assert_exact, assert_close, assert_sum_close

pytestmark = pytest.mark.gpu

EXACT_UN = ("Neg", "ReLU")
TRANS_UN = ("Sigmoid", "Tanh", "Sin", "Cos")
SIZES = [0, 1, 3, 4, 1031, (1 << 20) + 5]


def _data(n, seed=0):
    rng = np.random.default_rng(seed)
    a = rng.uniform(-4, 4, n).astype(np.float32)
    b = rng.uniform(-4, 4, n).astype(np.float32)
    d = rng.uniform(0.5, 4, n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    return a, b, d, g


@pytest.mark.parametrize("n", SIZES)
def test_binary_same_shape_bit_exact(cb, orc, n):
    a, b, d, g = _data(n)
    da_, db_, dd_ = cb.to_device(a), cb.to_device(b), cb.to_device(d)
    for op in ("Add", "Sub", "Mul"):
        assert_exact(cb.ops.binary(op, da_, db_).numpy(), orc.binary(op, a, b), f"{op} n={n}")
    assert_exact(cb.ops.binary("Div", da_, dd_).numpy(), orc.binary("Div", a, d), f"Div n={n}")


def test_binary_broadcast_layouts_bit_exact(cb, orc):
    rng = np.random.default_rng(1)
    for rows, inner in ((1024, 1024), (7, 10), (33, 128), (5, 3)):
        A = rng.uniform(-4, 4, (rows, inner)).astype(np.float32)
        r = rng.uniform(0.5, 4, inner).astype(np.float32)
        dA, dr = cb.to_device(A), cb.to_device(r)
        for op in ("Add", "Sub", "Mul", "Div"):
            assert_exact(cb.ops.binary(op, dA, dr, cb.ops.B_ROW).numpy(), orc.binary(op, A, r, 2), f"{op} row {rows}x{inner}")
            assert_exact(cb.ops.binary(op, dA, dr.view(0, (1,)), cb.ops.B_SCALAR).numpy(), orc.binary(op, A, r[:1], 1), f"{op} b-scalar")
            assert_exact(cb.ops.binary(op, dr.view(0, (1,)), dA, cb.ops.A_SCALAR).numpy(), orc.binary(op, r[:1], A, 3), f"{op} a-scalar")


def test_division_by_zero_is_ieee(cb, orc):
    a = np.asarray([1, -1, 0, 2], np.float32)
    b = np.asarray([0, 0, 0, 1], np.float32)
    with np.errstate(all="ignore"):
        assert_exact(cb.ops.binary("Div", cb.to_device(a), cb.to_device(b)).numpy(), orc.binary("Div", a, b), "x/0")


def test_unaligned_operands_take_the_scalar_path(cb, orc):
    a, b, d, g = _data(4101, 3)
    buf_a, buf_b = cb.to_device(np.concatenate([[0], a]).astype(np.float32)), cb.to_device(np.concatenate([[0, 0, 0], b]).astype(np.float32))
    va, vb = buf_a.view(1, (4101,)), buf_b.view(3, (4101,))
    assert_exact(cb.ops.binary("Add", va, vb).numpy(), orc.binary("Add", a, b), "unaligned Add")
    assert_exact(cb.ops.unary("ReLU", va).numpy(), orc.unary("ReLU", a), "unaligned ReLU")
    out = cb.empty((4102,))
    cb.ops.unary("Neg", vb, out=out.view(1, (4101,)))
    assert_exact(out.numpy()[1:], orc.unary("Neg", b), "unaligned output")


@pytest.mark.parametrize("n", SIZES)
def test_unary_forward(cb, orc, n):
    a, _, _, _ = _data(n, 4)
    da_ = cb.to_device(a)
    for op in EXACT_UN:
        assert_exact(cb.ops.unary(op, da_).numpy(), orc.unary(op, a), f"{op} n={n}")
    for op in TRANS_UN:  # tolerance: rel 1e-5 (+1e-6 absolute: Tanh cancels near 0)
        assert_close(cb.ops.unary(op, da_).numpy(), orc.unary(op, a), 1e-5, 1e-6, f"{op} n={n}")


def test_unary_special_values(cb, orc):
    a = np.asarray([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-30, -1e-30, 88.0, -88.0, 1e4], np.float32)
    da_ = cb.to_device(a)
    with np.errstate(all="ignore"):
        for op in ("Neg", "ReLU", "Sigmoid", "Sin", "Cos"):
            got, ref = cb.ops.unary(op, da_).numpy(), orc.unary(op, a)
            assert_close(got, ref, 1e-5, 1e-6, op + " special values")


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
def test_tensor_op_float_bit_exact(cb, orc, kind):
    _, _, d, _ = _data(70001, 5)
    assert_exact(cb.ops.scalar(kind, cb.to_device(d), 1.7).numpy(), orc.scalar(kind, d, 1.7), f"scalar kind {kind}")


def test_fill_tile_accumulate_sgd_bit_exact(cb, orc):
    rng = np.random.default_rng(6)
    n = 40003
    p = rng.standard_normal(n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    d = cb.empty((n,))
    assert_exact(cb.ops.fill(d, 0.25).numpy(), np.full(n, 0.25, np.float32), "fill")
    row = rng.standard_normal(12).astype(np.float32)
    assert_exact(cb.ops.tile(cb.to_device(row), 12 * 11).numpy(), np.tile(row, 11), "tile")
    dp = cb.to_device(p)
    assert_exact(cb.ops.accumulate(dp, cb.to_device(g)).numpy(), p + g, "grad += val")
    dp = cb.to_device(p)
    expect = (p.astype(np.float64) - g.astype(np.float64) * np.float64(np.float32(0.01))).astype(np.float32)  # one rounding
    assert_exact(cb.ops.sgd_update(dp, cb.to_device(g), 0.01).numpy(), expect, "p -= g*lr (fused)")


@pytest.mark.parametrize("n", [1, 1031, (1 << 18) + 3])
def test_unary_backward(cb, orc, n):
    a, _, _, g = _data(n, 7)
    da_, dg = cb.to_device(a), cb.to_device(g)
    for op in EXACT_UN:
        assert_exact(cb.ops.unary_backward(op, da_, dg).numpy(), orc.grad_unary(op, a, g), op + " bwd")
    for op in TRANS_UN:
        assert_close(cb.ops.unary_backward(op, da_, dg).numpy(), orc.grad_unary(op, a, g), 1e-5, 1e-6, op + " bwd")


@pytest.mark.parametrize("n", [1, 1031, (1 << 18) + 3])
def test_binary_backward_bit_exact(cb, orc, n):
    a, b, d, g = _data(n, 8)
    for op, y in (("Add", b), ("Sub", b), ("Mul", b), ("Div", d)):
        da, db = cb.ops.binary_backward(op, cb.to_device(a), cb.to_device(y), cb.to_device(g))
        ra, rb = orc.grad_binary(op, a, y, g)
        assert_exact(da.numpy(), ra, op + " da")
        assert_exact(db.numpy(), rb, op + " db")


def test_bias_gradient_is_the_first_row(cb, orc):
    """[B,H] + [H]: the reference sends row 0 of the upstream gradient to the bias, not the column sums."""
    rng = np.random.default_rng(9)
    for B, H in ((64, 128), (5, 10), (3, 4096)):
        A = rng.standard_normal((B, H)).astype(np.float32)
        bias = rng.standard_normal(H).astype(np.float32)
        g = rng.standard_normal((B, H)).astype(np.float32)
        da, db = cb.ops.binary_backward("Add", cb.to_device(A), cb.to_device(bias), cb.to_device(g), cb.ops.B_ROW)
        ra, rb = orc.grad_binary("Add", A, bias, g, 2)
        assert_exact(da.numpy(), ra, "da")
        assert_exact(db.numpy(), rb, "db")
        assert_exact(db.numpy(), g[0], "db == g[0]")
    for op in ("Add", "Sub", "Mul"):
        A = rng.standard_normal(1000).astype(np.float32)
        s = np.asarray([1.5], np.float32)
        g = rng.standard_normal(1000).astype(np.float32)
        da, db = cb.ops.binary_backward(op, cb.to_device(A), cb.to_device(s), cb.to_device(g), cb.ops.B_SCALAR)
        ra, rb = orc.grad_binary(op, A, s, g, 1)
        assert_exact(da.numpy(), ra, op + " scalar da")
        assert_exact(db.numpy(), rb, op + " scalar db")


@pytest.mark.parametrize("n", [0, 1, 1031, (1 << 22) + 7])
def test_sum_mse_mae_dot(cb, orc, n):
    a, b, _, _ = _data(n, 10)
    da_, db_ = cb.to_device(a), cb.to_device(b)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    assert_sum_close(cb.ops.sum(da_).numpy(), orc.sum(a), a64.sum(), f"sum n={n}")
    if n == 0:
        return
    assert_sum_close(cb.ops.dot(da_, db_).numpy(), orc.dot(a, b), (a64 * b64).sum(), "dot")
    assert_sum_close(cb.ops.mse(da_, db_).numpy(), orc.mse(a, b), ((a64 - b64) ** 2).mean(), "mse")
    assert_sum_close(cb.ops.mae(da_, db_).numpy(), orc.mae(a, b), np.abs(a64 - b64).mean(), "mae")
    # rel 1e-5 directly against the reference's own value wherever its sequential sum is still accurate
    if n <= 1031:
        assert_close(cb.ops.mse(da_, db_).numpy(), orc.mse(a, b), 1e-5, 1e-7, "mse vs reference")
        assert_close(cb.ops.mae(da_, db_).numpy(), orc.mae(a, b), 1e-5, 1e-7, "mae vs reference")


def test_reduction_is_repeatable_and_scratch_is_reusable(cb, orc):
    a, b, _, _ = _data(300001, 11)
    da_ = cb.to_device(a)
    first = cb.ops.sum(da_).numpy()
    for _ in range(3):
        assert_exact(cb.ops.sum(da_).numpy(), first, "same bits every launch")
    mine = cb.empty((cb.lib.ctk_reduce_scratch_bytes() // 4 + 1,))
    mine.fill_bytes(0xFF)  # a dirty caller-supplied scratch must not matter
    assert_exact(cb.ops.sum(da_, scratch=mine).numpy(), first, "caller scratch")


def test_mean_loss_backward_bit_exact(cb, orc):
    a, b, _, _ = _data(50001, 12)
    g = cb.to_device(np.asarray(0.75, np.float32))
    assert_exact(cb.ops.mse_backward(cb.to_device(a), cb.to_device(b), g).numpy(), orc.grad_loss("MSE", a, b, 0.75), "mse bwd")
    assert_exact(cb.ops.mae_backward(cb.to_device(a), cb.to_device(b), g).numpy(), orc.grad_loss("MAE", a, b, 0.75), "mae bwd")


def test_against_golden_fixture(cb, golden):
    """The same kernels against numbers the unmodified reference produced."""
    G = golden
    a, b, d, g = (cb.to_device(G[k]) for k in ("ew.a", "ew.b", "ew.d", "ew.g"))
    for op in ("Add", "Sub", "Mul"):
        assert_exact(cb.ops.binary(op, a, b).numpy(), G[f"ew.{op}.same"], op)
    assert_exact(cb.ops.binary("Div", a, d).numpy(), G["ew.Div.same"], "Div")
    for op in ("Neg", "ReLU"):
        assert_exact(cb.ops.unary(op, a).numpy(), G[f"ew.{op}"], op)
    for op in TRANS_UN:
        assert_close(cb.ops.unary(op, a).numpy(), G[f"ew.{op}"], 1e-5, 1e-6, op)
        assert_close(cb.ops.unary_backward(op, a, g).numpy(), G[f"ew.{op}.dx"], 1e-5, 1e-6, op + " dx")
    da, db = cb.ops.binary_backward("Add", cb.to_device(G["row.a"]), cb.to_device(G["row.b"]), cb.to_device(G["row.g"]), cb.ops.B_ROW)
    assert_exact(db.numpy(), G["row.Add.db"], "golden bias gradient")
