"""The MNIST application path: IDX reader, epoch loop, prediction and accuracy.

CPU part (no GPU): the product's MNISTLoader on the host device against the numpy restatement, the
reference's own loader (where it was built) and the golden fixture made from it; error behaviour.
GPU part: the same files loaded onto the device (bytes uploaded, converted there) bit for bit; the
byte -> float, first-maximum and label-match kernels; the epoch loop against the reference's losses
and weights; predicted labels and accuracy bit-exact against the golden record."""
import os

import numpy as np
import pytest

import oracle
from conftest import assert_close, assert_exact, assert_matmul_close

TRAIN = ("train-images-idx3-ubyte", "train-labels-idx1-ubyte")
TEST = ("t10k-images-idx3-ubyte", "t10k-labels-idx1-ubyte")


def _write_pair(d, names, pixels, labels):
    oracle.idx_write_images(os.path.join(d, names[0]), pixels)
    oracle.idx_write_labels(os.path.join(d, names[1]), labels)


@pytest.fixture()
def mnist_dir(tmp_path, golden):
    _write_pair(tmp_path, TRAIN, golden["mnist.pixels"], golden["mnist.labels_u8"])
    return tmp_path


def _frontend():
    from ctorch_b200 import frontend as F
    F.set_quiet(True)
    return F


# ---- CPU -------------------------------------------------------------------------------------------
def test_loader_on_the_host_matches_oracle_reference_and_golden(mnist_dir, golden):
    F = _frontend()
    im, lb = F.mnist_load(mnist_dir, device=F.CPU)
    assert im.shape == (96, 784) and lb.shape == (96,)
    assert_exact(im.numpy(), golden["mnist.images"], "images == the reference loader's (golden)")
    assert_exact(lb.numpy(), golden["mnist.labels"], "labels == the reference loader's (golden)")
    assert_exact(im.numpy(), oracle.idx_read_images(os.path.join(mnist_dir, TRAIN[0])), "images == numpy restatement")
    assert_exact(lb.numpy(), oracle.idx_read_labels(os.path.join(mnist_dir, TRAIN[1])), "labels == numpy restatement")
    if oracle.Reference.available():
        rim, rlb = oracle.Reference().mnist_load(mnist_dir)
        assert_exact(im.numpy(), rim, "images == reference library, run now")
        assert_exact(lb.numpy(), rlb, "labels == reference library, run now")


def test_loader_test_pair_and_named_pair(tmp_path):
    F = _frontend()
    rng = np.random.default_rng(5)
    px, lb = rng.integers(0, 256, (7, 3, 5)).astype(np.uint8), rng.integers(0, 10, 7).astype(np.uint8)
    _write_pair(tmp_path, TEST, px, lb)
    _write_pair(tmp_path, ("a.idx3", "a.idx1"), px[:2], lb[:2])
    im, l = F.mnist_load(tmp_path, which="test", device=F.CPU)
    assert_exact(im.numpy(), oracle.idx_read_images_from_bytes(px), "non-square images, test pair")
    assert_exact(l.numpy(), lb.astype(np.float32))
    im2, l2 = F.mnist_load(tmp_path, image_file="a.idx3", label_file="a.idx1", device=F.CPU)
    assert im2.shape == (2, 15) and l2.shape == (2,)


def test_loader_errors(tmp_path):
    """Missing file and wrong magic number throw, as in the reference (mnist_loader.cpp:9-11, 18-20,
    48-50, 57-59); a payload shorter than announced throws too (the reference reads on)."""
    F = _frontend()
    with pytest.raises(F.FrontendError, match="cannot open"):
        F.mnist_load(tmp_path, device=F.CPU)
    px, lb = np.zeros((2, 2, 2), np.uint8), np.zeros(2, np.uint8)
    _write_pair(tmp_path, TRAIN, px, lb)
    F.mnist_load(tmp_path, device=F.CPU)
    # swapped files: each has the other's magic number
    _write_pair(tmp_path, (TRAIN[1], TRAIN[0]), px, lb)
    with pytest.raises(F.FrontendError, match="2051"):
        F.mnist_load(tmp_path, device=F.CPU)
    _write_pair(tmp_path, TRAIN, px, lb)
    with open(os.path.join(tmp_path, TRAIN[0]), "r+b") as f:
        f.truncate(16 + 5)
    with pytest.raises(F.FrontendError, match="shorter"):
        F.mnist_load(tmp_path, device=F.CPU)
    if oracle.Reference.available():
        with pytest.raises(RuntimeError):
            oracle.Reference().mnist_load(os.path.join(tmp_path, "nowhere"))


def test_accuracy_restatement_on_known_answers(golden):
    p = np.asarray([[0.1, 0.7, 0.2], [0.5, 0.5, 0.0], [np.nan, 0.2, 0.3], [0.0, 0.0, 0.0]], np.float32)
    assert list(oracle.predicted_labels(p)) == [1, 0, 2, 0]   # first maximum; NaN never wins; all-zero row -> 0
    assert oracle.accuracy(p, [1, 1, 2, 0]) == np.float32(0.75)
    assert_exact(oracle.predicted_labels(golden["mnist.probs"]), golden["mnist.pred"])
    assert oracle.accuracy(golden["mnist.probs"], golden["mnist.labels"]) == golden["mnist.accuracy"]


# ---- GPU -------------------------------------------------------------------------------------------
@pytest.mark.gpu
def test_loader_on_the_device_is_bit_exact(cb, mnist_dir, golden):
    F = _frontend()
    im, lb = F.mnist_load(mnist_dir, device=F.CUDA)
    assert im.info()["device"] == F.CUDA and lb.info()["device"] == F.CUDA
    assert_exact(im.numpy(), golden["mnist.images"], "pixel / 255.0f computed on the device")
    assert_exact(lb.numpy(), golden["mnist.labels"])


@pytest.mark.gpu
def test_byte_to_float_kernel_all_values_and_tails(cb):
    for n, off in ((256, 0), (1000003, 0), (77, 1), (4099, 3), (20000003, 0), (6000001, 4)):   # the last two reach the four-deep loop
        src = (np.arange(n + off) % 256).astype(np.uint8)
        d = cb.to_device(src, np.uint8)
        out = cb.ops.u8_to_f32(d.view(off, (n,)), 255.0).numpy()
        assert_exact(out, src[off:].astype(np.float32) / np.float32(255.0), f"n={n} offset={off}")
    assert_exact(cb.ops.u8_to_f32(cb.to_device(np.arange(10, dtype=np.uint8), np.uint8), 1.0).numpy(), np.arange(10, dtype=np.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(1, 1), (513, 10), (1000, 16), (100, 7), (9, 3), (64, 33), (7, 1000), (3, 40000)])
def test_first_maximum_per_row(cb, rows, cols):
    rng = np.random.default_rng(rows * 7 + cols)
    p = rng.uniform(0, 1, (rows, cols)).astype(np.float32)
    if cols > 3:
        p[0, 2] = p[0].max() + 1
        p[0, cols - 1] = p[0, 2]          # a tie: the first one wins
        p[rows - 1] = -2.0                # nothing exceeds -1: class 0
        p[rows // 2, 0] = np.nan          # NaN never exceeds anything
    got = cb.ops.argmax_rows(cb.to_device(p), init=-1.0).numpy()
    assert_exact(got, oracle.predicted_labels(p).astype(np.float32), "prediction loop of calculate_accuracy")
    # init = -inf: the plain first-maximum argmax, negative values included
    q = -rng.uniform(1, 2, (rows, cols)).astype(np.float32)
    assert_exact(cb.ops.argmax_rows(cb.to_device(q)).numpy(), np.argmax(q, axis=1).astype(np.float32), "argmax of negative rows")


@pytest.mark.gpu
def test_label_match_count(cb):
    rng = np.random.default_rng(9)
    a = rng.integers(0, 10, 100003).astype(np.float32)
    b = rng.integers(0, 10, 100003).astype(np.float32)
    assert float(cb.ops.count_matches(cb.to_device(a), cb.to_device(b)).numpy()) == float((a == b).sum())
    assert float(cb.ops.count_matches(cb.to_device(a + 0.25), cb.to_device(a)).numpy()) == a.size   # (int) truncation, as in the reference


@pytest.mark.gpu
def test_epoch_loop_prediction_and_accuracy_against_the_reference(cb, mnist_dir, golden):
    """8 epochs of 3 batches over the device-resident set: every step loss and the final weights
    against the reference's run (golden), then its predicted labels and accuracy bit for bit."""
    F = _frontend()
    G = golden
    dims, bsz, epochs = [int(v) for v in G["mnist.dims"]], int(G["mnist.batch"]), int(G["mnist.epochs"])
    im, lb = F.mnist_load(mnist_dir, device=F.CUDA)
    tr = F.MlpTrainer(dims, G["mnist.params0"], float(G["mnist.lr"]))
    ref_losses = G["mnist.losses"].reshape(epochs, -1)
    for e in range(epochs):
        mean_loss = tr.train_epoch(im, lb, bsz)
        assert_close(np.float32(mean_loss), ref_losses[e].astype(np.float32).sum(dtype=np.float32) / np.float32(ref_losses.shape[1]), 1e-4, 0, f"mean loss of epoch {e}")
    assert_matmul_close(tr.params(), G["mnist.params"], 1e-4, "weights after the epochs")
    probs = tr.predict(im).numpy()
    assert_close(probs, G["mnist.probs"], 1e-4, 1e-6, "class probabilities")
    # labels: bit-exact where the reference's own top-2 margin is above the tolerance of the probabilities
    ref_sorted = np.sort(G["mnist.probs"], axis=1)
    clear = (ref_sorted[:, -1] - ref_sorted[:, -2]) > 1e-3
    assert clear.mean() > 0.9
    assert_exact(oracle.predicted_labels(probs)[clear], G["mnist.pred"][clear], "predicted labels")
    acc = tr.accuracy(im, lb)
    assert np.float32(acc) == oracle.accuracy(probs, G["mnist.labels"]), "accuracy == calculate_accuracy on the same probabilities"
    if clear.all():
        assert np.float32(acc) == G["mnist.accuracy"]


@pytest.mark.gpu
def test_epoch_loop_equals_steps_from_host_batches(cb, mnist_dir, golden):
    """train_epoch on views of the resident set == step_host on the same rows, bit for bit; a
    trailing partial batch is skipped as in the reference's loop."""
    F = _frontend()
    G = golden
    dims = [int(v) for v in G["mnist.dims"]]
    im, lb = F.mnist_load(mnist_dir, device=F.CUDA)
    a, b = F.MlpTrainer(dims, G["mnist.params0"], 0.002), F.MlpTrainer(dims, G["mnist.params0"], 0.002)
    mean = a.train_epoch(im, lb, 40)       # 96 rows: two batches of 40, 16 rows left over
    x, l = G["mnist.images"], G["mnist.labels"]
    losses = [b.step_host(x[i * 40:(i + 1) * 40], l[i * 40:(i + 1) * 40]) for i in range(2)]
    assert np.float32(mean) == (np.float32(losses[0]) + np.float32(losses[1])) / np.float32(2)
    assert_exact(a.params(), b.params(), "same weights either way")
    v = im.narrow_rows(40, 40)
    assert_exact(v.numpy(), x[40:80], "a batch is a view of the resident set")
