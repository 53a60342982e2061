"""CPU tests: the oracle against the golden fixtures (produced by the unmodified reference) and,
where oracle/_ref has been built, against the reference library itself."""
import numpy as np
import pytest

import oracle
from oracle import B_ROW, B_SCALAR, A_SCALAR
from conftest import assert_exact, assert_close

TRANS = ("Sigmoid", "Tanh", "Sin", "Cos")  # libm-dependent: allow 1e-6 against another host's glibc


def _cmp(got, ref, what, libm=False):
    if libm:
        assert_close(got, ref, rel=1e-6, abs_=1e-7, what=what)
    else:
        assert_exact(got, ref, what)


def test_golden_elementwise(orc, golden):
    G = golden
    a, b, d, g = G["ew.a"], G["ew.b"], G["ew.d"], G["ew.g"]
    for op in ("Add", "Sub", "Mul"):
        _cmp(orc.binary(op, a, b), G[f"ew.{op}.same"], op)
        _cmp(orc.binary(op, a, d[:1], B_SCALAR), G[f"ew.{op}.bscalar"], op + " scalar")
        da, db = orc.grad_binary(op, a, b, g)
        _cmp(da, G[f"ew.{op}.da"], op + " da")
        _cmp(db, G[f"ew.{op}.db"], op + " db")
    for op in ("Sub", "Mul"):
        _cmp(orc.binary(op, d[:1], b, A_SCALAR), G[f"ew.{op}.ascalar"], op + " a-scalar")
    _cmp(orc.binary("Div", a, d), G["ew.Div.same"], "Div")
    da, db = orc.grad_binary("Div", a, d, g)
    _cmp(da, G["ew.Div.da"], "Div da")
    _cmp(db, G["ew.Div.db"], "Div db")
    for op in ("Neg", "ReLU", "Sigmoid", "Tanh", "Sin", "Cos"):
        _cmp(orc.unary(op, a), G[f"ew.{op}"], op, libm=op in TRANS)
        _cmp(orc.grad_unary(op, a, g), G[f"ew.{op}.dx"], op + " dx", libm=op in TRANS)
    for k in range(4):
        _cmp(orc.scalar(k, d, 1.7), G[f"ew.scalar{k}"], f"scalar kind {k}")


def test_golden_row_broadcast_first_row_gradient(orc, golden):
    G = golden
    _cmp(orc.binary("Add", G["row.a"], G["row.b"], B_ROW), G["row.Add"], "Add row")
    da, db = orc.grad_binary("Add", G["row.a"], G["row.b"], G["row.g"], B_ROW)
    _cmp(da, G["row.Add.da"], "Add row da")
    _cmp(db, G["row.Add.db"], "Add row db")
    assert_exact(db, G["row.g"][0], "bias gradient is the first row of the upstream gradient")


def test_golden_reductions(orc, golden):
    G = golden
    _cmp(orc.sum(G["sum.x"]), G["sum"], "sum")
    _cmp(orc.grad_unary("Sum", G["sum.x"][:9], np.asarray([0.5], np.float32)), G["sum.dx"], "sum dx")
    a, b = G["ew.a"], G["ew.b"]
    _cmp(orc.mse(a, b), G["mse"], "mse")
    _cmp(orc.mae(a, b), G["mae"], "mae")
    _cmp(orc.dot(a, b), G["dot"], "dot")
    _cmp(orc.grad_loss("MSE", a, b, 0.75), G["mse.dp"], "mse dp")
    _cmp(orc.grad_loss("MAE", a, b, 0.75), G["mae.dp"], "mae dp")


@pytest.mark.parametrize("C", [10, 130])
def test_golden_rowwise(orc, golden, C):
    G = golden
    L, oh, lab, g = G[f"rw{C}.logits"], G[f"rw{C}.onehot"], G[f"rw{C}.labels"], G[f"rw{C}.g"]
    _cmp(orc.softmax(L), G[f"rw{C}.softmax"], "softmax", libm=True)
    _cmp(orc.softmax(L), G[f"rw{C}.softmax_kernel"], "softmax kernel", libm=True)
    _cmp(orc.grad_unary("Softmax", L, g), G[f"rw{C}.softmax.dx"], "softmax dx", libm=True)
    _cmp(orc.ce(L, oh), G[f"rw{C}.ce_onehot"], "ce onehot", libm=True)
    _cmp(orc.ce(L, lab), G[f"rw{C}.ce_index"], "ce index", libm=True)
    _cmp(orc.grad_loss("CE", L, oh), G[f"rw{C}.ce.dlogits"], "ce dlogits", libm=True)


@pytest.mark.parametrize("tag", ["mm33x47x29", "mm64x100x16"])
def test_golden_matmul(orc, golden, tag):
    G = golden
    A, B, dC = G[tag + ".A"], G[tag + ".B"], G[tag + ".dC"]
    _cmp(orc.matmul(A, B), G[tag + ".C"], "C")
    _cmp(orc.matmul(dC, B, tb=True), G[tag + ".dA"], "dA = dC.B^T")   # B [k,n] read as (B^T)^T
    _cmp(orc.matmul(A, dC, ta=True), G[tag + ".dB"], "dB = A^T.dC")
    rows = np.asarray([0, A.shape[0] - 1])
    _cmp(orc.matmul_rows(A, B, rows), G[tag + ".C"][rows], "sampled rows")


def test_known_answers_from_reference_tests(orc, golden):
    G = golden
    z, t = G["ka.ce.z"], G["ka.ce.t"]
    sm = orc.softmax(z)
    # src/tests/test_activation_loss.cpp:156-170: CE == -log(softmax(z)[0]) within 1e-4
    assert abs(float(orc.ce(z, t)) - (-np.log(max(sm[0], 1e-10)))) < 1e-4
    assert_close(orc.ce(z, t), G["ka.ce"], rel=1e-6, what="ce known answer")
    # :172-189: CE grad == softmax - target within 1e-4
    assert np.abs(orc.grad_loss("CE", z, t) - (sm - t)).max() < 1e-4
    # :57-65, 94-112: softmax rows sum to 1 within 1e-5
    assert abs(float(orc.softmax(G["ka.sm.m"]).sum(axis=1)[0]) - 1.0) < 1e-5
    # :114-126: d sum(softmax(x)) / dx ~ 0 within 1e-4
    assert np.abs(orc.grad_unary("Softmax", G["ka.sm.m"], np.ones((2, 3), np.float32))).max() < 1e-4
    assert_close(orc.grad_unary("Softmax", G["ka.sm.m"], np.ones((2, 3), np.float32)), G["ka.sm.grad_of_sum"], rel=1e-6, abs_=1e-7)
    # src/tests/test_tensor_grad.cpp:76-149: [2,3] + [3], upstream ones -> grad_b == 1 (not 2)
    a23 = np.arange(6, dtype=np.float32).reshape(2, 3)
    da, db = orc.grad_binary("Add", a23, np.asarray([1, 2, 3], np.float32), np.ones((2, 3), np.float32), B_ROW)
    assert_exact(db, np.ones(3, np.float32), "bias grad == 1")
    assert_exact(db, G["ka.bias.db"])
    # src/tests/test.cpp:6-155: scalar gradients of a+b, a*b, a-b, -a, a/b at a=3, b=2... (a/b: 0.5, -0.75)
    a, b, g = np.asarray([3.0], np.float32), np.asarray([2.0], np.float32), np.asarray([1.0], np.float32)
    assert orc.grad_binary("Add", a, b, g)[0][0] == 1 and orc.grad_binary("Add", a, b, g)[1][0] == 1
    assert orc.grad_binary("Mul", a, b, g)[0][0] == 2 and orc.grad_binary("Mul", a, b, g)[1][0] == 3
    assert orc.grad_binary("Sub", a, b, g)[1][0] == -1
    assert orc.grad_unary("Neg", a, g)[0] == -1
    da, db = orc.grad_binary("Div", a, b, g)
    assert da[0] == 0.5 and db[0] == -0.75


@pytest.mark.parametrize("tag", ["mlp1", "mlp2"])
def test_golden_mlp_training(orc, golden, tag):
    G = golden
    dims = [int(v) for v in G[tag + ".dims"]]
    x = G[tag + ".x"].astype(np.float32) / np.float32(255.0)
    steps = int(G[tag + ".steps"])
    r = orc.mlp_train(dims, x, G[tag + ".labels"], G[tag + ".params0"], 0.01, steps, grad_steps=(0, 1, steps - 1))
    for k in ("losses", "grads", "params", "logits"):
        assert_close(r[k], G[tag + "." + k], rel=1e-6, abs_=1e-7, what=f"{tag} {k}")


def test_ce_index_rejects_bad_label(orc):
    L = np.zeros((2, 3), np.float32)
    with pytest.raises(ValueError):
        orc.ce(L, np.asarray([0, 3], np.float32))


def test_empty_inputs(orc):
    e = np.zeros(0, np.float32)
    assert orc.binary("Add", e, e).size == 0
    assert orc.unary("ReLU", e).size == 0
    assert float(orc.sum(e)) == 0.0


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_oracle_matches_reference_library_bit_for_bit(orc):
    R = oracle.Reference()
    rng = np.random.default_rng(7)
    n = 2051
    a = rng.uniform(-4, 4, n).astype(np.float32)
    b = rng.uniform(-4, 4, n).astype(np.float32)
    d = rng.uniform(0.5, 4, n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    for op in ("Add", "Sub", "Mul", "Div"):
        assert_exact(orc.binary(op, a, d), R.binary(op, a, d), op)
        x, y = orc.grad_binary(op, a, d, g), R.grad_binary(op, a, d, g)
        assert_exact(x[0], y[0], op + " da")
        assert_exact(x[1], y[1], op + " db")
    for op in ("Neg", "ReLU", "Sigmoid", "Tanh", "Sin", "Cos"):
        assert_exact(orc.unary(op, a), R.unary(op, a), op)
        assert_exact(orc.grad_unary(op, a, g), R.grad_unary(op, a, g), op + " dx")
    A = rng.standard_normal((37, 53)).astype(np.float32)
    B = rng.standard_normal((53, 41)).astype(np.float32)
    assert_exact(orc.matmul(A, B), R.matmul(A, B), "matmul")
    assert_exact(orc.matmul(A.T.copy(), B, ta=True), R.matmul(A.T.copy(), B, ta=True), "matmul ta")
    assert_exact(orc.matmul(A, B.T.copy(), tb=True), R.matmul(A, B.T.copy(), tb=True), "matmul tb")
    L = (2 * rng.standard_normal((19, 37))).astype(np.float32)
    lab = rng.integers(0, 37, 19)
    oh = np.zeros_like(L)
    oh[np.arange(19), lab] = 1
    assert_exact(orc.softmax(L), R.softmax(L), "softmax")
    assert_exact(orc.ce(L, oh), R.ce(L, oh), "ce onehot")
    assert_exact(orc.ce(L, lab.astype(np.float32)), R.ce(L, lab.astype(np.float32)), "ce index")
    assert_exact(orc.grad_loss("CE", L, oh), R.grad_loss("CE", L, oh), "ce bwd")
    assert_exact(orc.grad_unary("Softmax", L, rng.standard_normal(L.shape).astype(np.float32) * 0 + 1),
                 R.grad_unary("Softmax", L, np.ones_like(L)), "softmax bwd")
    assert_exact(orc.sum(a), R.sum(a), "sum")
    assert_exact(orc.mse(a, b), R.mse(a, b), "mse")
    assert_exact(orc.mae(a, b), R.mae(a, b), "mae")
    dims = [30, 12, 7]
    x = rng.integers(0, 256, (2, 2, 6, 30)).astype(np.float32) / np.float32(255)
    lab = rng.integers(0, 7, (2, 2, 6)).astype(np.float32)
    p = oracle.pack_params([rng.uniform(-.4, .4, (30, 12)).astype(np.float32), rng.uniform(-.4, .4, (12, 7)).astype(np.float32)],
                           [np.zeros(12, np.float32), np.zeros(7, np.float32)])
    o, r = orc.mlp_train(dims, x, lab, p, 0.01, 4, (0, 3)), R.mlp_train(dims, x, lab, p, 0.01, 4, (0, 3))
    for k in ("losses", "grads", "params", "logits"):
        assert_exact(o[k], r[k], "mlp " + k)


def test_softmax_down_the_columns_matches_reference_library(orc):
    """Tensor::softmax(0) and its backward rule: the restatement against the reference library."""
    if not oracle.Reference.available():
        pytest.skip("reference library not built here")
    R = oracle.Reference()
    rng = np.random.default_rng(77)
    for shape in ((37, 19), (1, 8), (64, 1), (5, 130)):
        x = (2 * rng.standard_normal(shape)).astype(np.float32)
        g = rng.standard_normal(shape).astype(np.float32)
        y, dx = R.softmax_dim(x, 0, g)
        y2, dx2 = orc.softmax_dim0(x, g)
        assert np.array_equal(y, y2) and np.array_equal(dx, dx2), shape
        assert np.array_equal(R.softmax_dim(x, 1), orc.softmax(x))


@pytest.mark.skipif(not oracle.Reference.available(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_sampled_matmul_functions_match_whole_products_of_the_reference(orc, ta, tb):
    """orc_matmul_entries and orc_matmul_rows (with its interchanged loops where B's rows are contiguous)
    are what the full-size GPU tests compare with: each sampled value equals, bit for bit, the entry of
    the whole product as the reference library computes it."""
    ref = oracle.Reference()
    rng = np.random.default_rng(40 + 2 * ta + tb)
    m, k, n = 70, 130, 90
    A = rng.standard_normal((m, k)).astype(np.float32)
    B = rng.standard_normal((k, n)).astype(np.float32)
    sa = A.T.copy() if ta else A
    sb = B.T.copy() if tb else B
    C = ref.matmul(sa, sb, ta, tb)
    rows = np.array([0, 5, m - 1])
    assert np.array_equal(orc.matmul_rows(sa, sb, rows, ta, tb), C[rows])
    ri, ci = rng.integers(0, m, 300), rng.integers(0, n, 300)
    assert np.array_equal(orc.matmul_entries(sa, sb, ri, ci, ta, tb), C[ri, ci])
    # columns as rows of the transposed product on materialised operands (how the full-size tests take them)
    cols = np.array([n - 1, 3])
    got = orc.matmul_rows(np.ascontiguousarray(B[:, cols].T), np.ascontiguousarray(A.T), np.arange(2))
    assert np.array_equal(got, C[:, cols].T)
