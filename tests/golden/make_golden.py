"""Regenerates golden.npz from the UNMODIFIED reference library (oracle/_ref/libctorch_ref.so).

Run where the reference checkout exists:  make -C oracle && python tests/golden/make_golden.py
Every record stores its inputs next to the reference's outputs, so the fixture does not depend on
any random-number generator being reproducible elsewhere.  Inputs follow the benchmark configs'
value distributions at sizes the CPU finishes instantly.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from oracle import B_ROW, B_SCALAR, A_SCALAR  # noqa: E402


def main():
    R = oracle.Reference()
    rng = np.random.default_rng(20261125)
    G = {}
    n = 1031  # odd on purpose: exercises vector tails
    a = rng.uniform(-4, 4, n).astype(np.float32)
    b = rng.uniform(-4, 4, n).astype(np.float32)
    d = rng.uniform(0.5, 4, n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    G["ew.a"], G["ew.b"], G["ew.d"], G["ew.g"] = a, b, d, g
    for op in ("Add", "Sub", "Mul"):
        G[f"ew.{op}.same"] = R.binary(op, a, b)
        G[f"ew.{op}.bscalar"] = R.binary(op, a, d[:1], B_SCALAR)
        da, db = R.grad_binary(op, a, b, g)
        G[f"ew.{op}.da"], G[f"ew.{op}.db"] = da, db
    for op in ("Sub", "Mul"):
        G[f"ew.{op}.ascalar"] = R.binary(op, d[:1], b, A_SCALAR)
    G["ew.Div.same"] = R.binary("Div", a, d)
    da, db = R.grad_binary("Div", a, d, g)
    G["ew.Div.da"], G["ew.Div.db"] = da, db
    A2 = rng.uniform(-4, 4, (5, 64)).astype(np.float32)
    row = rng.uniform(-4, 4, 64).astype(np.float32)
    g2 = rng.standard_normal((5, 64)).astype(np.float32)
    G["row.a"], G["row.b"], G["row.g"] = A2, row, g2
    G["row.Add"] = R.binary("Add", A2, row, B_ROW)
    G["row.Add.da"], G["row.Add.db"] = R.grad_binary("Add", A2, row, g2, B_ROW)
    for op in ("Neg", "ReLU", "Sigmoid", "Tanh", "Sin", "Cos"):
        G[f"ew.{op}"] = R.unary(op, a)
        G[f"ew.{op}.dx"] = R.grad_unary(op, a, g)
    for k in range(4):
        G[f"ew.scalar{k}"] = R.scalar(k, d, 1.7)
    G["sum.x"] = rng.uniform(-4, 4, 5000).astype(np.float32)
    G["sum"] = np.asarray(R.sum(G["sum.x"]))
    G["sum.dx"] = R.grad_unary("Sum", G["sum.x"][:9], np.asarray([0.5], np.float32))
    G["mse"], G["mae"], G["dot"] = np.asarray(R.mse(a, b)), np.asarray(R.mae(a, b)), np.asarray(R.dot(a, b))
    G["mse.dp"], G["mae.dp"] = R.grad_loss("MSE", a, b, 0.75), R.grad_loss("MAE", a, b, 0.75)
    for C in (10, 130):
        L = (2 * rng.standard_normal((7, C))).astype(np.float32)
        lab = rng.integers(0, C, 7)
        oh = np.zeros((7, C), np.float32)
        oh[np.arange(7), lab] = 1
        gg = rng.standard_normal((7, C)).astype(np.float32)
        G[f"rw{C}.logits"], G[f"rw{C}.labels"], G[f"rw{C}.onehot"], G[f"rw{C}.g"] = L, lab.astype(np.float32), oh, gg
        G[f"rw{C}.softmax"] = R.softmax(L)
        G[f"rw{C}.softmax_kernel"] = R.softmax_kernel(L)
        G[f"rw{C}.softmax.dx"] = R.grad_unary("Softmax", L, gg)
        G[f"rw{C}.ce_onehot"] = np.asarray(R.ce(L, oh))
        G[f"rw{C}.ce_index"] = np.asarray(R.ce(L, lab.astype(np.float32)))
        G[f"rw{C}.ce.dlogits"] = R.grad_loss("CE", L, oh, 1.0)
    for (m, k, nn) in ((33, 47, 29), (64, 100, 16)):
        A = rng.standard_normal((m, k)).astype(np.float32)
        B = rng.standard_normal((k, nn)).astype(np.float32)
        dC = rng.standard_normal((m, nn)).astype(np.float32)
        t = f"mm{m}x{k}x{nn}"
        G[t + ".A"], G[t + ".B"], G[t + ".dC"] = A, B, dC
        G[t + ".C"] = R.matmul(A, B)
        G[t + ".dA"], G[t + ".dB"] = R.grad_matmul(A, B, dC)
    # known answers held by the reference's own tests
    z = np.asarray([2.0, 1.0, 0.1], np.float32)      # src/tests/test_activation_loss.cpp:156-189
    t = np.asarray([1.0, 0.0, 0.0], np.float32)
    G["ka.ce.z"], G["ka.ce.t"] = z, t
    G["ka.ce"] = np.asarray(R.ce(z, t))
    G["ka.ce.grad"] = R.grad_loss("CE", z, t, 1.0)
    G["ka.softmax"] = R.softmax(z)
    m = np.asarray([[1, 2, 3], [0, -1, 1]], np.float32)  # test_activation_loss.cpp:94-126
    G["ka.sm.m"] = m
    G["ka.sm.grad_of_sum"] = R.grad_unary("Softmax", m, np.ones_like(m))
    a23 = np.arange(6, dtype=np.float32).reshape(2, 3)    # src/tests/test_tensor_grad.cpp:76-149
    G["ka.bias.da"], G["ka.bias.db"] = R.grad_binary("Add", a23, np.asarray([1, 2, 3], np.float32), np.ones((2, 3), np.float32), B_ROW)
    # the MLP training step: config-1 shape at a reduced width plus two summed-gradient replicas
    for tag, dims, batch, steps, reps, nb in (("mlp1", [784, 8, 10], 16, 6, 1, 1), ("mlp2", [40, 24, 16, 10], 8, 5, 2, 2)):
        x = rng.integers(0, 256, (reps, nb, batch, dims[0])).astype(np.float32) / np.float32(255.0)
        lab = rng.integers(0, dims[-1], (reps, nb, batch)).astype(np.float32)
        Ws, bs = [], []
        for i, j in zip(dims[:-1], dims[1:]):
            lim = np.sqrt(6.0 / i)
            Ws.append(rng.uniform(-lim, lim, (i, j)).astype(np.float32))
            bs.append(np.zeros(j, np.float32))
        p = oracle.pack_params(Ws, bs)
        r = R.mlp_train(dims, x, lab, p, 0.01, steps, grad_steps=(0, 1, steps - 1))
        G[tag + ".dims"] = np.asarray(dims, np.int64)
        G[tag + ".x"] = (x * 255).round().astype(np.uint8)  # pixels are k/255: store k
        G[tag + ".labels"], G[tag + ".params0"] = lab, p
        G[tag + ".steps"] = np.asarray(steps)
        for k in ("params", "losses", "grads", "logits"):
            G[tag + "." + k] = r[k]
    # the MNIST application path: an IDX image/label pair through the reference's own MNISTLoader, an
    # epoch loop over it (batches in file order), then prediction and accuracy on the whole set
    import tempfile
    n_img, bsz, dims = 96, 32, [784, 16, 12, 10]
    labels_u8 = rng.integers(0, 10, n_img).astype(np.uint8)
    pixels = rng.integers(0, 48, (n_img, 28, 28)).astype(np.uint8)   # dim noise ...
    pixels[0].reshape(-1)[-256:] = np.arange(256, dtype=np.uint8)     # (every byte value once)
    for i in range(n_img):                                            # ... and a bright mark per class
        pixels[i, labels_u8[i] * 2: labels_u8[i] * 2 + 2, :] = 255
    with tempfile.TemporaryDirectory() as d:
        oracle.idx_write_images(os.path.join(d, "train-images-idx3-ubyte"), pixels)
        oracle.idx_write_labels(os.path.join(d, "train-labels-idx1-ubyte"), labels_u8)
        im, lb = R.mnist_load(d)
    assert np.array_equal(im, oracle.idx_read_images_from_bytes(pixels)) and np.array_equal(lb, labels_u8.astype(np.float32))
    Ws, bs = [], []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        Ws.append(rng.uniform(-lim, lim, (i, j)).astype(np.float32))
        bs.append(np.zeros(j, np.float32))
    p0 = oracle.pack_params(Ws, bs)
    epochs, nb = 8, n_img // bsz
    lr = 0.002
    r = R.mlp_train(dims, im.reshape(1, nb, bsz, 784), lb.reshape(1, nb, bsz), p0, lr, epochs * nb)
    Wf, bf = oracle.unpack_params(r["params"], dims)
    h = im
    for l, (W, b) in enumerate(zip(Wf, bf)):
        h = R.binary("Add", R.matmul(h, W), b, B_ROW)
        if l + 1 < len(Wf):
            h = R.unary("ReLU", h)
    probs = R.softmax(h)
    G["mnist.pixels"], G["mnist.labels_u8"] = pixels, labels_u8
    G["mnist.images"], G["mnist.labels"] = im, lb
    G["mnist.dims"], G["mnist.batch"], G["mnist.epochs"] = np.asarray(dims, np.int64), np.asarray(bsz), np.asarray(epochs)
    G["mnist.lr"] = np.asarray(lr, np.float32)
    G["mnist.params0"], G["mnist.params"], G["mnist.losses"] = p0, r["params"], r["losses"]
    G["mnist.probs"] = probs
    G["mnist.pred"] = oracle.predicted_labels(probs)
    G["mnist.accuracy"] = np.asarray(oracle.accuracy(probs, lb), np.float32)
    # ---- comparisons, Tensor::to(DType), operator[], ones (src/Tensor.cpp:985-1309, 1462-1591, 199-243, 175-189, 422-450)
    rng = np.random.default_rng(77)
    ca = rng.integers(-3, 4, (37, 21)).astype(np.float32)
    cb_ = rng.integers(-3, 4, (37, 21)).astype(np.float32)
    ca[0, :4] = [np.nan, np.inf, -np.inf, -0.0]
    cb_[0, :4] = [1.0, np.inf, np.inf, 0.0]
    cb_[1, 0] = np.nan
    G["cmp.a"], G["cmp.b"], G["cmp.s"] = ca, cb_, np.asarray(1.0, np.float32)
    for c in oracle.CMP_NAMES:
        G[f"cmp.{c}.tt"] = R.compare(c, ca, cb_)
        G[f"cmp.{c}.ts"] = R.compare(c, ca, 1.0)
        G[f"cmp.{c}.st"] = R.compare(c, ca, 1.0, scalar_left=True)
    x = (rng.standard_normal(1003) * 1000).astype(np.float32)
    x[:8] = [0.0, -0.0, 0.5, -0.5, 0.99999994, -1.5, 16777216.0, -2147483648.0]
    G["cast.x"] = x
    for d in (1, 2, 3, 4):
        G[f"cast.{d}"] = R.cast_from_float(x, d)
    G["index.values"] = np.asarray([R.index_1d(x, i) for i in (0, 2, 1002)], np.float32)
    for d in range(5):
        G[f"ones.{d}"] = R.ones(d, 5)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(out, **G)
    print("wrote", out, os.path.getsize(out), "bytes,", len(G), "arrays")


if __name__ == "__main__":
    main()
