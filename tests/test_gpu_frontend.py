"""GPU parity of the C++ front end (Tensor / AutoDiff / Ctorch_Scheduler on kCUDA) against the oracle.

The first group re-runs the assertions of the reference's own test programs (src/tests/test.cpp,
test_tensor_grad.cpp, test_activation_loss.cpp) with tensors created on the CUDA device; the second
runs the MLP training step (mnist/mnist.cpp:44-92) and compares losses, gradients and weights.
Tolerances: bit-exact for Add/Sub/Mul/Div/Neg/ReLU results, rel 1e-5 for transcendental and
reduction results, normwise 1e-4 (3xTF32) for MatMul results and everything downstream of them."""
import numpy as np
import pytest

import oracle
from conftest import assert_close, assert_exact, assert_matmul_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def F(cb):
    from ctorch_b200 import frontend
    assert frontend.cuda_available(), "Ctorch_Scheduler::isDeviceAvailable(kCUDA) must be true on a GPU box"
    frontend.set_quiet(True)
    return frontend


def dev(F, a):
    return F.Tensor.from_numpy(np.asarray(a, np.float32))


# ---- src/tests/test.cpp: scalar autograd -------------------------------------------------------------
def test_scalar_gradients_like_StdTest(F):
    with F.AutoDiff():
        a, b = dev(F, [2.0]).requires_grad(), dev(F, [3.0]).requires_grad()
        c = a + b
        F.backward(c)
        assert F.grad(a).numpy()[0] == 1 and F.grad(b).numpy()[0] == 1            # test.cpp:6-34
    with F.AutoDiff():
        a, b = dev(F, [2.0]).requires_grad(), dev(F, [3.0]).requires_grad()
        F.backward(a * b)
        assert F.grad(a).numpy()[0] == 3 and F.grad(b).numpy()[0] == 2            # :36-65
    with F.AutoDiff():
        a, b = dev(F, [5.0]).requires_grad(), dev(F, [3.0]).requires_grad()
        F.backward(a - b)
        assert F.grad(a).numpy()[0] == 1 and F.grad(b).numpy()[0] == -1           # :67-96
    with F.AutoDiff():
        a = dev(F, [2.0]).requires_grad()
        F.backward(-a)
        assert F.grad(a).numpy()[0] == -1                                          # :98-124
    with F.AutoDiff():
        a, b = dev(F, [6.0]).requires_grad(), dev(F, [2.0]).requires_grad()
        F.backward(a / b)
        assert F.grad(a).numpy()[0] == 0.5 and F.grad(b).numpy()[0] == -1.5       # :126-155


# ---- src/tests/test_tensor_grad.cpp ---------------------------------------------------------------------
def test_tensor_gradients_like_TensorGradTest(F, orc):
    with F.AutoDiff():
        a, b = dev(F, [1, 2, 3]).requires_grad(), dev(F, [4, 5, 6]).requires_grad()
        d = (a + b) * 2.0
        F.backward(d)
        assert_exact(F.grad(a).numpy(), np.full(3, 2, np.float32))                 # :7-73
        assert_exact(F.grad(b).numpy(), np.full(3, 2, np.float32))
    with F.AutoDiff():
        a = dev(F, np.arange(6).reshape(2, 3)).requires_grad()
        b = dev(F, [10, 20, 30]).requires_grad()
        c = a + b
        assert_exact(c.numpy(), np.arange(6, dtype=np.float32).reshape(2, 3) + np.asarray([10, 20, 30], np.float32))
        F.backward(c)
        assert_exact(F.grad(a).numpy(), np.ones((2, 3), np.float32))
        assert_exact(F.grad(b).numpy(), np.ones(3, np.float32))                    # :132-138: 1, not 2
    with F.AutoDiff():
        x, y = dev(F, [1, 2, 3]).requires_grad(), dev(F, [4, 5, 6]).requires_grad()
        z = x * y + x
        F.backward(z)
        assert_exact(F.grad(x).numpy(), np.asarray([5, 6, 7], np.float32))         # :152-224: y + 1
        assert_exact(F.grad(y).numpy(), np.asarray([1, 2, 3], np.float32))


# ---- src/tests/test_activation_loss.cpp ---------------------------------------------------------------------
def test_activations_and_losses_like_ActivationLossTest(F, orc, golden):
    with F.AutoDiff():
        m = dev(F, [[1, 2, 3], [0, -1, 1]])
        p = m.softmax(1).numpy()
        assert abs(p[0].sum() - 1) < 1e-5 and abs(p[1].sum() - 1) < 1e-5          # :94-100
        x = dev(F, [[1, 2, 3], [0, -1, 1]]).requires_grad()
        L = x.softmax(1).sum()
        F.backward(L)
        assert np.abs(F.grad(x).numpy()).max() < 1e-4                              # :114-126
    with F.AutoDiff():
        z, t = dev(F, [2.0, 1.0, 0.1]), dev(F, [1.0, 0.0, 0.0])
        ce = z.cross_entropy(t)
        sm = z.softmax(0).numpy()
        assert abs(ce.item() - (-np.log(max(sm[0], 1e-10)))) < 1e-4                # :156-170
        assert_close(ce.item(), golden["ka.ce"], 1e-5, 1e-6, "CE known answer")
    with F.AutoDiff():
        z, t = dev(F, [2.0, 1.0, 0.1]).requires_grad(), dev(F, [1.0, 0.0, 0.0])
        F.backward(z.cross_entropy(t))
        g = F.grad(z).numpy()
        assert np.abs(g - (orc.softmax(np.asarray([2.0, 1.0, 0.1], np.float32)) - np.asarray([1, 0, 0], np.float32))).max() < 1e-4  # :172-189
        assert_close(g, golden["ka.ce.grad"], 1e-5, 1e-7, "CE grad known answer")
    with F.AutoDiff():
        y = dev(F, [-0.5, 0.5]).requires_grad()
        loss = y.sigmoid().sum() + y.tanh().sum()                                  # :68-86
        F.backward(loss)
        yy = np.asarray([-0.5, 0.5], np.float32)
        ref = orc.grad_unary("Sigmoid", yy, np.ones(2, np.float32)) + orc.grad_unary("Tanh", yy, np.ones(2, np.float32))
        assert_close(F.grad(y).numpy(), ref, 1e-5, 1e-6, "d(sum sigmoid + sum tanh)")


def test_every_operator_through_the_scheduler(F, orc):
    rng = np.random.default_rng(0)
    a = rng.uniform(-4, 4, (37, 64)).astype(np.float32)
    b = rng.uniform(0.5, 4, (37, 64)).astype(np.float32)
    row = rng.uniform(0.5, 4, 64).astype(np.float32)
    A, B, R = dev(F, a), dev(F, b), dev(F, row)
    for name, got in (("Add", A + B), ("Sub", A - B), ("Mul", A * B), ("Div", A / B)):
        assert_exact(got.numpy(), orc.binary(name, a, b), name)
    assert_exact((A + R).numpy(), orc.binary("Add", a, row, 2), "[N,H] + [H]")
    assert_exact((-A).numpy(), orc.unary("Neg", a), "Neg")
    assert_exact(A.relu().numpy(), orc.unary("ReLU", a), "ReLU")
    for name, got in (("Sigmoid", A.sigmoid()), ("Tanh", A.tanh()), ("Sin", A.sin()), ("Cos", A.cos())):
        assert_close(got.numpy(), orc.unary(name, a), 1e-5, 1e-6, name)
    for kind, got in ((0, A * 1.7), (1, A + 1.7), (2, A / 1.7), (3, 1.7 - A), (5, 1.7 * A), (6, 1.7 + A)):
        assert_exact(got.numpy(), orc.scalar(kind if kind < 5 else kind - 5, a, 1.7), f"scalar form {kind}")
    assert_exact((F.Tensor.scalar(2.0) * A).numpy(), orc.binary("Mul", np.asarray([2.0], np.float32), a, 3), "0-D host tensor * device tensor")
    assert_close(A.softmax(-1).numpy(), orc.softmax(a), 1e-5, 1e-9, "softmax")
    assert_close(A.sum().item(), a.astype(np.float64).sum(), 1e-5, 1e-4, "sum")
    assert_close(A.mse_loss(B).item(), orc.mse(a, b), 1e-5, 1e-7, "mse")
    assert_close(A.mae_loss(B).item(), orc.mae(a, b), 1e-5, 1e-7, "mae")
    w = rng.standard_normal((64, 48)).astype(np.float32)
    assert_matmul_close(A.matmul(dev(F, w)).numpy(), orc.matmul(a, w), 1e-4, "matmul")
    assert_matmul_close(A.t().numpy(), a.T, 0, "t() view reads back transposed")
    assert_matmul_close(A.t().matmul(A).numpy(), orc.matmul(a, a, ta=True), 1e-4, "A^T . A through a t() view")


def test_backward_rules_match_the_oracle(F, orc):
    rng = np.random.default_rng(1)
    x = rng.uniform(-3, 3, (9, 40)).astype(np.float32)
    g = rng.standard_normal((9, 40)).astype(np.float32)
    for name, fn in (("ReLU", lambda t: t.relu()), ("Sigmoid", lambda t: t.sigmoid()), ("Tanh", lambda t: t.tanh()),
                     ("Sin", lambda t: t.sin()), ("Cos", lambda t: t.cos()), ("Neg", lambda t: -t), ("Softmax", lambda t: t.softmax(1))):
        with F.AutoDiff():
            X = dev(F, x).requires_grad()
            F.backward(fn(X), dev(F, g))
            ref = orc.grad_unary(name, x, g)
            if name in ("ReLU", "Neg"):
                assert_exact(F.grad(X).numpy(), ref, name + " backward")
            else:
                assert np.abs(F.grad(X).numpy() - ref).max() <= 1e-5 * max(np.abs(ref).max(), np.abs(g).max()) + 1e-6, name
    d = rng.uniform(0.5, 3, (9, 40)).astype(np.float32)
    for name, fn in (("Add", lambda p, q: p + q), ("Sub", lambda p, q: p - q), ("Mul", lambda p, q: p * q), ("Div", lambda p, q: p / q)):
        with F.AutoDiff():
            P, Q = dev(F, x).requires_grad(), dev(F, d).requires_grad()
            F.backward(fn(P, Q), dev(F, g))
            ra, rb = orc.grad_binary(name, x, d, g)
            assert_exact(F.grad(P).numpy(), ra, name + " da")
            assert_exact(F.grad(Q).numpy(), rb, name + " db")
    t = rng.standard_normal((9, 40)).astype(np.float32)
    for name, fn in (("MSE", lambda p, q: p.mse_loss(q)), ("MAE", lambda p, q: p.mae_loss(q))):
        with F.AutoDiff():
            P = dev(F, x).requires_grad()
            F.backward(fn(P, dev(F, t)))
            assert_exact(F.grad(P).numpy(), orc.grad_loss(name, x, t, 1.0), name + " backward")
    oh = np.zeros((9, 40), np.float32)
    oh[np.arange(9), rng.integers(0, 40, 9)] = 1
    with F.AutoDiff():
        P = dev(F, x).requires_grad()
        F.backward(P.cross_entropy(dev(F, oh)))
        assert_close(F.grad(P).numpy(), orc.grad_loss("CE", x, oh), 1e-5, 1e-7, "CE backward")
    with F.AutoDiff():  # index labels: forward works, backward cannot (reference: the Sub broadcast throws)
        P = dev(F, x).requires_grad()
        loss = P.cross_entropy(dev(F, np.argmax(oh, 1).astype(np.float32)))
        assert_close(loss.item(), orc.ce(x, oh), 1e-5, 1e-6, "CE index forward")
        with pytest.raises(F.FrontendError):
            F.backward(loss)
    A = rng.standard_normal((33, 20)).astype(np.float32)
    Bm = rng.standard_normal((20, 28)).astype(np.float32)
    G = rng.standard_normal((33, 28)).astype(np.float32)
    with F.AutoDiff():
        TA, TB = dev(F, A).requires_grad(), dev(F, Bm).requires_grad()
        F.backward(TA.matmul(TB), dev(F, G))
        assert_matmul_close(F.grad(TA).numpy(), orc.matmul(G, Bm, tb=True), 1e-4, "dA = dC . B^T")
        assert_matmul_close(F.grad(TB).numpy(), orc.matmul(A, G, ta=True), 1e-4, "dB = A^T . dC")


def test_value_semantics_and_stale_snapshot(F, orc):
    """Copies are values (write after copy does not leak), and backward keeps multiplying by the
    weights as they were when first registered (src/AutoDiff.cpp:286-290 / :1651)."""
    a = dev(F, [1, 2, 3])
    c = a.copy()
    a.fill(9.0)
    assert_exact(c.numpy(), np.asarray([1, 2, 3], np.float32), "copy is unaffected by a later write")
    assert c.info()["id"] != a.info()["id"]
    x = np.asarray([[1.0, 2.0]], np.float32)
    w = np.asarray([[3.0], [7.0]], np.float32)
    ctx = F.AutoDiff()
    with ctx:
        W = dev(F, w)
        ctx.make_leaf(W, True)
        W.requires_grad(True)
        X = dev(F, x).requires_grad()
        F.backward(X.matmul(W))
        assert_exact(F.grad(X).numpy(), np.asarray([[3.0, 7.0]], np.float32))
        W.sgd_update_(dev(F, [[-27.0 / 0.5], [-63.0 / 0.5]]), 0.5)  # W <- 10 * W, in place
        assert_exact(W.numpy(), 10 * w)
        X2 = dev(F, x).requires_grad()
        Y2 = X2.matmul(W)
        assert_exact(Y2.numpy(), np.asarray([[170.0]], np.float32), "forward uses the live weights")
        F.backward(Y2)
        assert_exact(F.grad(X2).numpy(), np.asarray([[3.0, 7.0]], np.float32), "backward uses the first snapshot")


def test_no_kernel_on_the_host_device(F):
    a = F.Tensor.from_numpy([1.0, 2.0], device=F.CPU)
    with pytest.raises(F.FrontendError):
        a.relu()
    with pytest.raises(F.FrontendError):
        a + a


# ---- the training step -------------------------------------------------------------------------------------------
def _mlp_case(dims, batch, n_batches, seed_data=1234, seed_w=42):
    r = np.random.default_rng(seed_data)
    x = r.integers(0, 256, (1, n_batches, batch, dims[0])).astype(np.float32) / np.float32(255.0)
    lab = r.integers(0, dims[-1], (1, n_batches, batch)).astype(np.float32)
    rw = np.random.default_rng(seed_w)
    Ws, bs = [], []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        Ws.append(rw.uniform(-lim, lim, (i, j)).astype(np.float32))
        bs.append(np.zeros(j, np.float32))
    return x, lab, oracle.pack_params(Ws, bs)


def _run_gpu(F, dims, x, lab, p, lr, steps, grad_steps):
    tr = F.MlpTrainer(dims, p, lr)
    tr.keep_logits(True)
    losses, grads = [], {}
    for s in range(steps):
        bi = s % x.shape[1]
        losses.append(tr.step_host(x[0, bi], lab[0, bi]))
        if s in grad_steps:
            grads[s] = tr.grads()
    assert tr.node_count() == 2 * (len(dims) - 1), "only the parameter leaves stay on the tape between steps"
    return np.asarray(losses, np.float32), grads, tr.params(), tr.logits(x.shape[2])


@pytest.mark.parametrize("lr,tag", [(0.01, "config-1 as specified"), (0.01 / 64, "same, learning rate scaled to a mean loss")])
def test_mlp_784_128_10_hundred_steps(F, orc, lr, tag):
    """Config 1: 784-128-10, batch 64, pixels k/255, Kaiming-uniform weights (seed 42), data seed 1234,
    a fixed sequence of 100 batches, SGD lr 0.01, 100 steps of forward + backward + update."""
    dims = [784, 128, 10]
    x, lab, p = _mlp_case(dims, 64, 100)
    ref = orc.mlp_train(dims, x, lab, p, lr, 100, grad_steps=(0, 1, 99))
    losses, grads, params, logits = _run_gpu(F, dims, x, lab, p, lr, 100, (0, 1, 99))
    # With lr 0.01 on a loss SUMMED over 64 rows the specified run diverges within three steps (loss
    # 166 -> 1136, logits in the thousands, probabilities at the 1e-10 clamp), so a 1e-6 relative
    # difference in a logit moves a row's -log(p) by 1e-3 and more: the loss bound is 1e-3 there and
    # 1e-4 for the well-conditioned variant.  Gradients and weights keep the 1e-4 MatMul tolerance.
    loss_rel = 1e-3 if lr == 0.01 else 1e-4
    assert_close(losses, ref["losses"][:, 0], loss_rel, 1e-3, f"loss at every step ({tag})")
    assert np.median(np.abs(losses - ref["losses"][:, 0]) / np.abs(ref["losses"][:, 0])) < 1e-5
    for i, s in enumerate((0, 1, 99)):
        assert_matmul_close(grads[s], ref["grads"][i], 1e-4, f"gradients at step {s} ({tag})")
    assert_matmul_close(params, ref["params"], 1e-4, f"final weights ({tag})")
    flips = np.count_nonzero(np.argmax(logits, 1) != np.argmax(ref["logits"][0], 1))
    assert flips == 0, f"{flips} argmax flips in the last step's logits"


def test_mlp_deeper_network_with_ragged_widths(F, orc):
    dims = [100, 72, 40, 10]
    x, lab, p = _mlp_case(dims, 33, 7, 5, 6)
    ref = orc.mlp_train(dims, x, lab, p, 0.001, 12, grad_steps=(0, 5, 11))
    losses, grads, params, logits = _run_gpu(F, dims, x, lab, p, 0.001, 12, (0, 5, 11))
    assert_close(losses, ref["losses"][:, 0], 1e-4, 1e-3, "losses")
    for i, s in enumerate((0, 5, 11)):
        assert_matmul_close(grads[s], ref["grads"][i], 1e-4, f"gradients at step {s}")
    assert_matmul_close(params, ref["params"], 1e-4, "final weights")


def test_mlp_against_golden_fixture(F, golden):
    G = golden
    dims = [int(v) for v in G["mlp1.dims"]]
    x = G["mlp1.x"].astype(np.float32) / np.float32(255.0)
    steps = int(G["mlp1.steps"])
    losses, grads, params, logits = _run_gpu(F, dims, x, G["mlp1.labels"], G["mlp1.params0"], 0.01, steps, (0, 1, steps - 1))
    assert_close(losses, G["mlp1.losses"][:, 0], 1e-4, 1e-3, "golden losses")
    for i, s in enumerate((0, 1, steps - 1)):
        assert_matmul_close(grads[s], G["mlp1.grads"][i], 1e-4, f"golden gradients at step {s}")
    assert_matmul_close(params, G["mlp1.params"], 1e-4, "golden final weights")
    assert_matmul_close(logits, G["mlp1.logits"][0], 1e-4, "golden logits")


def test_step_on_device_resident_inputs_equals_step_from_host(F):
    dims = [64, 32, 10]
    x, lab, p = _mlp_case(dims, 16, 1, 9, 10)
    a, b = F.MlpTrainer(dims, p, 0.001), F.MlpTrainer(dims, p, 0.001)
    oh = np.zeros((16, 10), np.float32)
    oh[np.arange(16), lab[0, 0].astype(int)] = 1
    X, Y = dev(F, x[0, 0]), dev(F, oh)
    for _ in range(3):
        la, lb = a.step_host(x[0, 0], lab[0, 0]), b.step_device(X, Y)
        assert la == lb
    assert_exact(a.params(), b.params(), "same weights either way")


def test_staged_uploads_equal_steps_from_host(F, cb):
    """stage_host / step_staged (upload of the next batch overlapped with the current step) against
    step_host on the same sequence of batches: pageable and page-locked host buffers, two batches
    staged ahead, a third refused."""
    from ctorch_b200.device import PinnedArray
    dims = [64, 32, 10]
    rng = np.random.default_rng(21)
    _, _, p = _mlp_case(dims, 16, 1, 9, 10)
    batches = [(rng.uniform(0, 1, (16, 64)).astype(np.float32), rng.integers(0, 10, 16).astype(np.float32)) for _ in range(4)]
    a, b = F.MlpTrainer(dims, p, 0.01), F.MlpTrainer(dims, p, 0.01)
    ref = [a.step_host(x, l) for x, l in batches]
    pinned = []
    for x, l in batches[:2]:
        px, pl = PinnedArray(x.shape), PinnedArray(l.shape)
        px.array[...] = x
        pl.array[...] = l
        pinned.append((px, pl))
    b.stage_host(pinned[0][0].array, pinned[0][1].array)
    b.stage_host(pinned[1][0].array, pinned[1][1].array)
    with pytest.raises(F.FrontendError):
        b.stage_host(batches[2][0], batches[2][1])   # only two may wait
    got = [b.step_staged()]
    b.stage_host(batches[2][0], batches[2][1])       # pageable
    got.append(b.step_staged())
    b.stage_host(batches[3][0], batches[3][1])
    got.append(b.step_staged())
    got.append(b.step_staged())
    with pytest.raises(F.FrontendError):
        b.step_staged()                              # nothing staged
    assert got == ref
    assert_exact(a.params(), b.params(), "same weights either way")


def test_kept_operand_splits_follow_every_write(F, orc):
    """The 3xTF32 MatMul keeps the hi/lo split of an operand with the operand's buffer.  A write to
    the buffer (fill, in-place SGD, upload) must drop it, a copy made before the write must keep
    seeing the old values, and transposed views and both operands from one buffer must work."""
    rng = np.random.default_rng(31)
    x = rng.standard_normal((40, 24)).astype(np.float32)
    w = rng.standard_normal((24, 36)).astype(np.float32)
    X, W = dev(F, x), dev(F, w)
    y1 = X.matmul(W).numpy()
    y1_again = X.matmul(W).numpy()            # both splits reused
    assert_exact(y1, y1_again, "reusing kept splits changes nothing")
    assert_matmul_close(y1, orc.matmul(x, w), 1e-4, "first product")
    W_old = W.copy()                          # shares the buffer and its split
    W.sgd_update_(dev(F, np.ones_like(w)), 0.5)   # in place: W <- W - 0.5
    assert_matmul_close(X.matmul(W).numpy(), orc.matmul(x, w - 0.5), 1e-4, "product after the in-place update")
    assert_exact(X.matmul(W_old).numpy(), y1, "the copy made before the write still multiplies the old values")
    W.fill(2.0)
    assert_matmul_close(X.matmul(W).numpy(), orc.matmul(x, np.full_like(w, 2.0)), 1e-4, "product after fill")
    # the transposed view finds the split of the plain one and the other way round
    g = rng.standard_normal((40, 36)).astype(np.float32)
    G = dev(F, g)
    assert_matmul_close(X.t().matmul(G).numpy(), orc.matmul(x, g, ta=True), 1e-4, "X^T.G with X's kept split")
    assert_matmul_close(G.matmul(W_old.t()).numpy(), orc.matmul(g, w, tb=True), 1e-4, "G.W^T with W's kept split")
    assert_matmul_close(G.t().matmul(X).numpy(), orc.matmul(g, x, ta=True), 1e-4, "G^T.X")
    # both operands views of one buffer
    assert_matmul_close(X.matmul(X.t()).numpy(), orc.matmul(x, x, tb=True), 1e-4, "X.X^T")
    sq = rng.standard_normal((32, 32)).astype(np.float32)
    S = dev(F, sq)
    assert_matmul_close(S.matmul(S).numpy(), orc.matmul(sq, sq), 1e-4, "S.S")


def test_zero_grad_then_read_then_accumulate(F):
    """zero_grad (src/AutoDiff.cpp:502-510) followed by a read gives zeros; backward after zero_grad
    gives one contribution, backward twice without it gives the sum of both."""
    w = np.asarray([[1.0, -2.0], [3.0, 0.5]], np.float32)
    x = np.asarray([[2.0, 5.0]], np.float32)
    ctx = F.AutoDiff()
    with ctx:
        W = dev(F, w)
        ctx.make_leaf(W, True)
        W.requires_grad(True)
        F.backward(dev(F, x).matmul(W).sum())
        g1 = F.grad(W).numpy()
        assert_exact(g1, np.repeat(x.T, 2, axis=1), "dW = x^T . 1")
        F.backward((dev(F, 3 * x)).matmul(W).sum())
        assert_exact(F.grad(W).numpy(), 4 * g1, "a second backward adds to the first")
        ctx.zero_grad(W)
        assert_exact(F.grad(W).numpy(), np.zeros_like(w), "zeroed gradient reads as zeros")
        F.backward((dev(F, 3 * x)).matmul(W).sum())
        assert_exact(F.grad(W).numpy(), 3 * g1, "backward after zero_grad holds one contribution")
        ctx.zero_grad(W)
        F.backward(dev(F, x).matmul(W).sum())
        F.backward(dev(F, x).matmul(W).sum())
        assert_exact(F.grad(W).numpy(), 2 * g1, "zero, then two contributions")


def test_graph_replayed_steps_equal_eager_steps(F, cb):
    """cth_mlp_step_graph_host: two eager calls, the third records the step into a CUDA graph, later calls
    replay it.  Losses and weights must equal the eager trainer's bit for bit, across a change of batch
    size (new graph), an interleaved eager step (graph released, recorded again) and pageable as well
    as page-locked inputs."""
    from ctorch_b200.device import PinnedArray
    dims = [784, 128, 64, 10]
    rng = np.random.default_rng(41)
    _, _, p = _mlp_case(dims, 16, 1, 9, 10)

    def batch(n):
        return rng.integers(0, 256, (n, 784)).astype(np.float32) / np.float32(255.0), rng.integers(0, 10, n).astype(np.float32)

    a, b = F.MlpTrainer(dims, p, 0.001), F.MlpTrainer(dims, p, 0.001)
    seq = [batch(128) for _ in range(6)] + [batch(64) for _ in range(5)]
    for i, (x, l) in enumerate(seq):
        la = a.step_host(x, l)
        if i == 3:
            px, pl = PinnedArray(x.shape), PinnedArray(l.shape)
            px.array[...] = x
            pl.array[...] = l
            lb = b.step_graph_host(px.array, pl.array)
        else:
            lb = b.step_graph_host(x, l)
        assert la == lb, f"step {i}: eager {la} graph {lb}"
    assert_exact(a.params(), b.params(), "weights after graph-replayed steps")
    assert_exact(a.grads(), b.grads(), "gradients of the last step")
    # an eager step in between releases the graph; the next graph steps record a new one
    x, l = batch(64)
    assert a.step_host(x, l) == b.step_host(x, l)
    for _ in range(5):
        x, l = batch(64)
        assert a.step_host(x, l) == b.step_graph_host(x, l)
    assert_exact(a.params(), b.params(), "weights after eager and graph steps interleaved")
    assert cb.ops.matmul_status() == 0


def test_graph_epoch_equals_eager_epoch(F, cb, golden, tmp_path):
    import oracle as _o
    import os
    G = golden
    _o.idx_write_images(os.path.join(tmp_path, "train-images-idx3-ubyte"), G["mnist.pixels"])
    _o.idx_write_labels(os.path.join(tmp_path, "train-labels-idx1-ubyte"), G["mnist.labels_u8"])
    im, lb = F.mnist_load(tmp_path)
    dims = [int(v) for v in G["mnist.dims"]]
    a, b = F.MlpTrainer(dims, G["mnist.params0"], 0.002), F.MlpTrainer(dims, G["mnist.params0"], 0.002)
    for _ in range(3):
        assert a.train_epoch(im, lb, 32) == b.train_epoch_graph(im, lb, 32)
    assert_exact(a.params(), b.params(), "weights after three epochs")
    assert a.accuracy(im, lb) == b.accuracy(im, lb)


@pytest.mark.parametrize("relu", [True, False])
@pytest.mark.parametrize("m,k,n", [(256, 96, 320), (130, 64, 132), (384, 520, 600), (8192, 784, 128), (64, 40, 10)])
def test_fused_linear_equals_the_three_calls(F, cb, orc, m, k, n, relu):
    """Tensor::linear: MatMul + bias [+ ReLU] in the product's epilogue (with the result's hi/lo split)
    against x.matmul(w) + b [.relu()]: values, every gradient, and a following product that uses the
    split the epilogue wrote -- all bit for bit (with every tile computed whole: a fused epilogue needs
    the whole sum, so the unfused twin must not cut its last wave's K in two either).  n = 10 is not
    fusable (not a multiple of 4) and takes the three calls."""
    rng = np.random.default_rng(m + k + n)
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / np.sqrt(k)).astype(np.float32)
    b = rng.standard_normal(n).astype(np.float32)
    w2 = rng.standard_normal((n, 8)).astype(np.float32)
    out = {}
    for fused in (False, True):
        cb.ops.set_matmul_tail_split(0)
        with F.AutoDiff():
            X, W, B, W2 = (dev(F, a).requires_grad() for a in (x, w, b, w2))
            if fused:
                Y = X.linear(W, B, relu)
            else:
                Y = X.matmul(W) + B
                Y = Y.relu() if relu else Y
            Z = Y.matmul(W2)            # a product whose A operand split came from the epilogue
            F.backward(Z.sum())
            out[fused] = [Y.numpy(), Z.numpy(), F.grad(X).numpy(), F.grad(W).numpy(), F.grad(B).numpy(), F.grad(W2).numpy()]
        cb.ops.set_matmul_tail_split(1)
    for a, c, name in zip(out[False], out[True], ("y", "z", "dx", "dw", "db", "dw2")):
        assert_exact(c, a, f"{name}: fused == three calls")
    ref = orc.matmul(x, w) + b
    ref = np.maximum(ref, 0) if relu else ref
    assert_matmul_close(out[True][0], ref, 1e-4, "fused linear vs oracle")


def test_trainer_with_and_without_fused_linear_is_bit_identical(F, cb):
    """The trainer's forward uses linear(); CTORCH_FUSE_LINEAR=0 (read once per process) cannot be
    toggled here, so the unfused twin is the op-by-op front end driven from this test."""
    dims = [784, 128, 64, 12]
    rng = np.random.default_rng(5)
    parts = []
    Ws, bs = [], []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        Ws.append(rng.uniform(-lim, lim, (i, j)).astype(np.float32))
        bs.append(rng.uniform(-0.1, 0.1, j).astype(np.float32))
        parts += [Ws[-1].ravel(), bs[-1]]
    p = np.concatenate(parts)
    x = rng.integers(0, 256, (256, 784)).astype(np.float32) / np.float32(255.0)
    lab = rng.integers(0, 12, 256).astype(np.float32)
    oh = np.zeros((256, 12), np.float32)
    oh[np.arange(256), lab.astype(int)] = 1
    cb.ops.set_matmul_tail_split(0)   # the fused product computes whole tiles: so must its twin
    try:
        tr = F.MlpTrainer(dims, p, 0.001)
        loss = tr.step_host(x, lab)
        with F.AutoDiff() as ctx:
            W = [dev(F, a) for a in Ws]
            B = [dev(F, a) for a in bs]
            for t in W + B:
                ctx.make_leaf(t, True)
                t.requires_grad(True)
            h = dev(F, x)
            for l in range(3):
                h = h.matmul(W[l]) + B[l]
                if l < 2:
                    h = h.relu()
            L = h.cross_entropy(dev(F, oh))
            F.backward(L)
            grads = np.concatenate([np.concatenate([F.grad(W[l]).numpy().ravel(), F.grad(B[l]).numpy().ravel()]) for l in range(3)])
            assert float(L.numpy()) == loss
    finally:
        cb.ops.set_matmul_tail_split(1)
    assert_exact(tr.grads(), grads, "gradients: trainer (fused forward) == op-by-op front end")


@pytest.mark.parametrize("batch,dims", [(256, [96, 320, 256, 12]), (130, [64, 132, 260, 10]), (8192, [784, 256, 512, 10])])
def test_relu_backward_in_the_gradient_products_epilogue(F, cb, batch, dims):
    """set_fuse_relu_backward: the product g.W^T whose result only feeds a ReLU's backward rule applies
    the rule (and writes the hi/lo split the next two products read) in its epilogue.  Loss and every
    parameter gradient are bit for bit those of the unfused tape; the gradient stored for the hidden
    activation itself is the masked one."""
    rng = np.random.default_rng(batch + dims[1])
    Ws = [(rng.standard_normal((i, j)) / np.sqrt(i)).astype(np.float32) for i, j in zip(dims[:-1], dims[1:])]
    bs = [rng.uniform(-0.1, 0.1, j).astype(np.float32) for j in dims[1:]]
    x = rng.standard_normal((batch, dims[0])).astype(np.float32)
    oh = np.zeros((batch, dims[-1]), np.float32)
    oh[np.arange(batch), rng.integers(0, dims[-1], batch)] = 1
    out = {}
    cb.ops.set_matmul_tail_split(0)
    try:
        for fused in (False, True):
            with F.AutoDiff() as ctx:
                ctx.set_fuse_relu_backward(fused)
                W = [dev(F, a).requires_grad() for a in Ws]
                B = [dev(F, a).requires_grad() for a in bs]
                h = dev(F, x)
                hidden = []
                for l in range(len(Ws)):
                    h = h.linear(W[l], B[l], l + 1 < len(Ws))
                    hidden.append(h)
                L = h.cross_entropy(dev(F, oh))
                F.backward(L)
                out[fused] = [L.numpy()] + [F.grad(t).numpy() for t in W + B] + [F.grad(hidden[0]).numpy(), hidden[0].numpy()]
    finally:
        cb.ops.set_matmul_tail_split(1)
    for i, (a, c) in enumerate(zip(out[False][:-2], out[True][:-2])):
        assert_exact(c, a, f"loss / parameter gradient {i}: fused == unfused")
    g_plain, y = out[False][-2], out[False][-1]
    assert_exact(out[True][-2], g_plain * (y > 0).astype(np.float32), "stored gradient of the hidden activation: the masked one")


def test_relu_backward_fusion_is_skipped_when_the_activation_has_two_readers(F, cb):
    """A ReLU output read by two products keeps the plain rule: its gradient is a sum of two
    contributions and the mask applies to the sum."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((128, 64)).astype(np.float32)
    w, w2, w3 = (rng.standard_normal(s).astype(np.float32) / 8 for s in ((64, 64), (64, 32), (64, 32)))
    b = rng.standard_normal(64).astype(np.float32)
    out = {}
    for fused in (False, True):
        with F.AutoDiff() as ctx:
            ctx.set_fuse_relu_backward(fused)
            X, W, W2, W3, B = (dev(F, a).requires_grad() for a in (x, w, w2, w3, b))
            h = X.linear(W, B, True)
            L = (h.matmul(W2) * h.matmul(W3)).sum()
            F.backward(L)
            out[fused] = [F.grad(t).numpy() for t in (X, W, W2, W3, B)] + [F.grad(h).numpy()]
    for a, c in zip(out[False], out[True]):
        assert_exact(c, a, "two readers: nothing changes")


def test_gradient_of_a_shape_that_does_not_broadcast_is_folded(F):
    """check_and_adjust_grad_shape's fall-back (src/AutoDiff.cpp:910-1048): a gradient whose shape neither
    equals nor broadcasts to the tensor's is folded, result[i] = sum of grad[j] over j = i (mod n), added
    in ascending j in fp32.  Reached by backward(root, grad_output) with a grad_output of another shape."""
    rng = np.random.default_rng(17)
    for gshape, n in (((4, 5), 6), ((3, 7), 21), ((2, 3, 5), 4), ((5,), 8)):
        x = rng.standard_normal(n).astype(np.float32)
        g = rng.standard_normal(gshape).astype(np.float32)
        want = np.zeros(n, np.float32)
        for j, v in enumerate(g.ravel()):            # the reference's loop (:921-923)
            want[j % n] = np.float32(want[j % n] + v)
        with F.AutoDiff():
            X = dev(F, x).requires_grad()
            y = -X
            F.backward(y, dev(F, g))
            got = F.grad(X).numpy()
        assert_close(got, -want, 1e-5, 1e-6, f"fold {gshape} -> [{n}]")


def test_leaf_gradient_hook_fires_once_after_the_last_contribution(F):
    """AutoDiff::on_leaf_grad -- where a data-parallel driver starts a gradient's all-reduce -- is called
    once per leaf and pass, also for a leaf that enters several nodes (a shared weight): its gradient is
    complete only after the last of its contributions."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((32, 16)).astype(np.float32)
    w = rng.standard_normal((16, 16)).astype(np.float32) / 4
    v = rng.standard_normal((16, 8)).astype(np.float32) / 4
    with F.AutoDiff() as ctx:
        ctx.count_leaf_grads(True)
        X, W, V = dev(F, x), dev(F, w).requires_grad(), dev(F, v).requires_grad()
        h = X.matmul(W).relu().matmul(W)      # W enters two products
        L = h.matmul(V).sum()
        F.backward(L)
        assert ctx.leaf_grad_count(W) == 1, "a leaf with two consumers: one call, after the second contribution"
        assert ctx.leaf_grad_count(V) == 1
        assert ctx.leaf_grad_count(X) == 0, "no gradient was asked for"
        # and the gradient the hook saw complete is the sum of both contributions
        a1 = np.maximum(x.astype(np.float64) @ w, 0)
        g_h = np.ones((32, 8)) @ v.astype(np.float64).T
        want = a1.T @ g_h + x.astype(np.float64).T @ ((g_h @ w.astype(np.float64).T) * (a1 > 0))
        assert_matmul_close(F.grad(W).numpy(), want, 1e-4, "gradient of the shared weight")
        ctx.count_leaf_grads(False)


@pytest.mark.parametrize("rows,cols", [(8192, 4096), (130, 132), (257, 10), (1, 5), (3000, 1)])
def test_column_sum_kernel(cb, rows, cols):
    rng = np.random.default_rng(rows + cols)
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    d = cb.to_device(x)
    got = cb.ops.colsum(d).numpy()
    assert_close(got, x.astype(np.float64).sum(axis=0), 1e-5, 1e-4, "column sums")
    assert_exact(cb.ops.colsum(d).numpy(), got, "fixed order: the same bits again")


def _textbook_mlp_steps(Ws, bs, xs, labels, lr):
    """Plain SGD on a ReLU MLP with cross entropy SUMMED over the batch, in float64: bias gradients
    summed over the batch, backward against the current weights."""
    Ws, bs = [w.astype(np.float64) for w in Ws], [b.astype(np.float64) for b in bs]
    losses = []
    for x, lab in zip(xs, labels):
        hs = [x.astype(np.float64)]
        for l, (W, b) in enumerate(zip(Ws, bs)):
            z = hs[-1] @ W + b
            hs.append(np.maximum(z, 0) if l + 1 < len(Ws) else z)
        z = hs[-1]
        p = np.exp(z - z.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        idx = lab.astype(int)
        losses.append(-np.log(np.maximum(p[np.arange(len(idx)), idx], 1e-10)).sum())
        g = p.copy()
        g[np.arange(len(idx)), idx] -= 1
        for l in range(len(Ws) - 1, -1, -1):
            dW, db = hs[l].T @ g, g.sum(axis=0)
            if l > 0:
                g = (g @ Ws[l].T) * (hs[l] > 0)
            Ws[l] -= lr * dW
            bs[l] -= lr * db
    return np.asarray(losses), np.concatenate([np.concatenate([W.ravel(), b]) for W, b in zip(Ws, bs)])


def test_corrected_mode_is_textbook_sgd(F, cb):
    """set_corrected(exact_bias_grad, fresh_weights): an opt-in mode outside the reference's arithmetic.
    With both on the trainer follows plain SGD (float64 numpy) to 1e-4; with both off (the default, the
    reference's arithmetic) it does not: the first-row bias gradient and the stale backward weights are
    real differences."""
    dims, batch, steps, lr = [20, 64, 32, 8], 48, 5, 0.01 / 48
    rng = np.random.default_rng(8)
    Ws = [(rng.standard_normal((i, j)) / np.sqrt(i)).astype(np.float32) for i, j in zip(dims[:-1], dims[1:])]
    bs = [rng.uniform(-0.1, 0.1, j).astype(np.float32) for j in dims[1:]]
    p0 = np.concatenate([np.concatenate([W.ravel(), b]) for W, b in zip(Ws, bs)])
    xs = [rng.standard_normal((batch, dims[0])).astype(np.float32) for _ in range(steps)]
    labs = [rng.integers(0, dims[-1], batch).astype(np.float32) for _ in range(steps)]
    want_loss, want_p = _textbook_mlp_steps(Ws, bs, xs, labs, lr)
    tr = F.MlpTrainer(dims, p0, lr)
    tr.set_corrected(True, True)
    got = [tr.step_host(x, l) for x, l in zip(xs, labs)]
    assert_close(np.asarray(got, np.float64), want_loss, 1e-4, 0, "losses, corrected mode")
    assert_matmul_close(tr.params(), want_p, 1e-4, "weights, corrected mode")
    plain = F.MlpTrainer(dims, p0, lr)
    for x, l in zip(xs, labs):
        plain.step_host(x, l)
    dev_plain = np.abs(plain.params() - want_p).max()
    dev_corr = np.abs(tr.params() - want_p).max()
    assert dev_plain > 100 * max(dev_corr, 1e-9), "the default mode keeps the reference's arithmetic"
    # switching it off again returns to the reference's arithmetic from the current weights on
    tr.set_corrected(False, False)
    tr.step_host(xs[0], labs[0])


def test_deferred_losses_change_nothing_but_the_waiting(F, cb):
    """set_deferred_loss: the step calls return without waiting and report 0; sync_losses() hands out the
    same losses, and the weights end up bit for bit the same -- from device batches, from host batches
    and through the staged uploads (whose slots are then guarded by events, not by the host's wait)."""
    from ctorch_b200.device import PinnedArray
    dims, batch, steps = [64, 96, 12], 128, 6
    rng = np.random.default_rng(4)
    p0 = np.concatenate([np.concatenate([(rng.standard_normal((i, j)) / np.sqrt(i)).astype(np.float32).ravel(),
                                         rng.uniform(-0.1, 0.1, j).astype(np.float32)]) for i, j in zip(dims[:-1], dims[1:])])
    xs = [rng.standard_normal((batch, dims[0])).astype(np.float32) for _ in range(steps)]
    labs = [rng.integers(0, dims[-1], batch).astype(np.float32) for _ in range(steps)]
    a, b, c = (F.MlpTrainer(dims, p0, 0.001) for _ in range(3))
    want = [a.step_host(x, l) for x, l in zip(xs, labs)]
    b.set_deferred_loss(True)
    assert all(b.step_host(x, l) == 0.0 for x, l in zip(xs, labs))
    assert_exact(b.sync_losses(), np.asarray(want, np.float32), "deferred losses, host batches")
    b.set_deferred_loss(False)
    assert_exact(b.params(), a.params(), "weights, host batches")
    # staged uploads from page-locked buffers that stay unchanged until sync_losses()
    px = [PinnedArray(x.shape) for x in xs]
    pl = [PinnedArray(l.shape) for l in labs]
    for q, x in zip(px, xs):
        q.array[...] = x
    for q, l in zip(pl, labs):
        q.array[...] = l
    c.set_deferred_loss(True)
    c.stage_host(px[0].array, pl[0].array)
    for k in range(steps):
        if k + 1 < steps:
            c.stage_host(px[k + 1].array, pl[k + 1].array)
        assert c.step_staged() == 0.0
    assert_exact(c.sync_losses(), np.asarray(want, np.float32), "deferred losses, staged uploads")
    assert_exact(c.params(), a.params(), "weights, staged uploads")
    with pytest.raises(F.FrontendError, match="deferred"):
        c.train_epoch(F.Tensor.from_numpy(xs[0]), F.Tensor.from_numpy(labs[0]), 64)
