"""Parity at the FULL sizes of the benchmark configurations, where the CPU cannot evaluate the whole
result: the kernels run at full size on the GPU and are checked

  * against the oracle's exact recurrence on sampled entries, full rows and full columns
    (products), sampled rows (row-wise kernels) and slabs (elementwise), and against float64;
  * through properties that cover every output element at once (a random projection of a whole
    product, additivity of a summed loss over row slabs).

Sizes: 4096^3, 8192^3 and 65536 x 784 x 4096 products with both backward products, in both
tensor-core modes; one training step of 784-4096-4096-4096-10 at batch 8192; softmax / cross entropy
on [65536, 32000] (8.4 GB per array, byte offsets past 2^32); elementwise and Sum at 2^28.
Tolerances are the ones every parity test uses (conftest.py): bit-exact for exact elementwise ops,
rel 1e-5 for transcendentals and reductions, normwise 1e-4 (3xTF32) / 5e-3 (TF32) for products and
gradients.
"""
import ctypes
from concurrent.futures import ThreadPoolExecutor

import numpy as np
import pytest

from conftest import assert_close, assert_exact, assert_matmul_close, assert_sum_close

pytestmark = pytest.mark.gpu

TOL = {"3xtf32": 1e-4, "tf32": 5e-3}
N_ENTRIES = 4096
_pool = ThreadPoolExecutor(max_workers=8)


def _status_ok(cb):
    assert cb.ops.matmul_status() == 0, "a bounded wait in the tensor-core kernel ran out"


# ---- sampled oracle of one product ------------------------------------------------------------------
def _logical(stored, transposed):
    """The operand as the product sees it ([m,k] or [k,n]); a view, no copy."""
    return stored.T if transposed else stored


def _oracle_samples(orc, sa, sb, ta, tb, rng):
    """Sampled entries, two full rows and two full columns of A.B by the oracle's recurrence
    (bit-identical to the reference's loop) and in float64.  Returns (index arrays, ref32, ref64)."""
    A, B = _logical(sa, ta), _logical(sb, tb)          # [m,k], [k,n] views
    m, k = A.shape
    n = B.shape[1]
    ri = rng.integers(0, m, N_ENTRIES)
    ci = rng.integers(0, n, N_ENTRIES)
    rows = np.array([0, int(rng.integers(1, m))])
    cols = np.array([n - 1, int(rng.integers(0, n - 1))])
    # entries, in parallel chunks (ctypes releases the GIL)
    chunks = np.array_split(np.arange(N_ENTRIES), 8)
    parts = list(_pool.map(lambda c: orc.matmul_entries(sa, sb, ri[c], ci[c], ta, tb), chunks))
    e32 = np.concatenate(parts)
    r32 = orc.matmul_rows(sa, sb, rows, ta, tb)         # [2, n]
    # columns: row j of C^T = B^T.A^T on materialised operands (a*b == b*a bit for bit, same l order)
    bt_rows = np.ascontiguousarray(B[:, cols].T)        # [2, k]
    at = sa if ta else np.ascontiguousarray(A.T)        # [k, m] contiguous
    c32 = orc.matmul_rows(bt_rows, at, np.arange(len(cols)))   # [2, m]
    # float64 of the same samples
    e64 = np.empty(N_ENTRIES)
    for c in np.array_split(np.arange(N_ENTRIES), max(1, (N_ENTRIES * k * 8) // (256 << 20))):
        e64[c] = np.einsum("ek,ke->e", A[ri[c]].astype(np.float64), B[:, ci[c]].astype(np.float64))
    r64 = A[rows].astype(np.float64) @ B.astype(np.float64) if k * n <= (1 << 26) else np.stack(
        [sum(A[r, s:s + 4096].astype(np.float64) @ B[s:s + 4096].astype(np.float64) for s in range(0, k, 4096)) for r in rows])
    c64 = np.stack([sum(A[:, s:s + 4096].astype(np.float64) @ B[s:s + 4096, j].astype(np.float64) for s in range(0, k, 4096)) for j in cols])
    return (ri, ci, rows, cols), (e32, r32, c32), (e64, r64, c64)


def _normwise(got, ref):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def _product_errors(C, idx, ref32, ref64):
    """Normwise errors of the sampled entries, rows and columns: (vs the reference recurrence, vs float64)."""
    ri, ci, rows, cols = idx
    got = (C[ri, ci], C[rows], C[:, cols].T)
    return (max(_normwise(g, r) for g, r in zip(got, ref32)), max(_normwise(g, r) for g, r in zip(got, ref64)))


def _projection_check(C, sa, sb, ta, tb, tol, rng, what):
    """Every element of C at once: C.v against A.(B.v) in float64 for a random +-1 vector v."""
    A, B = _logical(sa, ta), _logical(sb, tb)
    n = B.shape[1]
    v = rng.integers(0, 2, n).astype(np.float64) * 2 - 1
    bv = np.zeros(B.shape[0])
    for s in range(0, B.shape[0], 2048):
        bv[s:s + 2048] = B[s:s + 2048].astype(np.float64) @ v
    want = np.empty(A.shape[0])
    got = np.empty(A.shape[0])
    for s in range(0, A.shape[0], 2048):
        want[s:s + 2048] = A[s:s + 2048].astype(np.float64) @ bv
        got[s:s + 2048] = C[s:s + 2048].astype(np.float64) @ v
    # |C.v| grows like sqrt(n) * |C|: the same normwise bound applies to the projected vector
    assert_matmul_close(got, want, tol, what + " projection of the whole product")


@pytest.mark.parametrize("m,k,n", [(4096, 4096, 4096), (8192, 8192, 8192), (65536, 784, 4096)])
def test_config3_products_at_full_size(cb, orc, m, k, n):
    """C = A.B, dA = dC.B^T and dB = A^T.dC (contractions of 784 to 65536 terms): the fp32-accurate mode with
    its correction terms on the bf16 path (the default) and on the TF32 path ("3xTF32"), and the TF32 mode."""
    rng = np.random.default_rng(1000 + m + k)
    A = rng.standard_normal((m, k), dtype=np.float32)
    B = rng.standard_normal((k, n), dtype=np.float32)
    dC = rng.standard_normal((m, n), dtype=np.float32)
    dA_, dB_, dG = cb.to_device(A), cb.to_device(B), cb.to_device(dC)
    products = (("C=A.B", A, B, False, False, dA_, dB_),
                ("dA=dC.B^T", dC, B, False, True, dG, dB_),
                ("dB=A^T.dC", A, dC, True, False, dA_, dG))
    report, bad = {}, []
    start = cb.lib.ctk_get_matmul_correction()
    for name, sa, sb, ta, tb, da, db in products:
        idx, ref32, ref64 = _oracle_samples(orc, sa, sb, ta, tb, rng)
        for mode, corr, label in (("3xtf32", 1, "tf32+2xbf16"), ("3xtf32", 0, "3xtf32"), ("tf32", 1, "tf32")):
            assert cb.ops.matmul_path(da, db, ta, tb, mode) == 0, "tensor-core path expected"
            cb.ops.set_matmul_correction(corr)
            try:
                out = cb.ops.matmul(da, db, ta, tb, mode)
            finally:
                cb.ops.set_matmul_correction(start)
            C = out.numpy()
            del out
            what = f"{name} {m}x{k}x{n} {label}"
            e32, e64 = _product_errors(C, idx, ref32, ref64)
            report[what] = f"{e32:.2e} vs the reference recurrence, {e64:.2e} vs float64"
            if max(e32, e64) > TOL[mode]:
                bad.append(what)
            _projection_check(C, sa, sb, ta, tb, TOL[mode], rng, what)
            del C
    _status_ok(cb)
    print("\nnormwise errors on 4096 entries + 2 rows + 2 columns:")
    for k_, v in report.items():
        print(f"  {k_}: {v}")
    assert not bad, f"above tolerance: {bad}; all: {report}"


# ---- config 5: one full-width training step -----------------------------------------------------------
def _fp64_step(dims, x, labels, Ws, bs, lr, masks, Ws_back=None):
    """The training step of mnist/mnist.cpp:44-92 in float64 with the reference's semantics: summed
    cross entropy with the 1e-10 clamp, bias gradient = row 0 of the upstream gradient
    (src/AutoDiff.cpp:690-757), backward through the weights as registered (equal to the live ones at
    the first step; Ws_back: those registered weights at a later step), p -= g*lr.
    masks[l]: which hidden units of layer l the DEVICE found active.  ReLU's
    derivative jumps at 0, so a pre-activation within rounding distance of 0 may fall on either side in
    float32 and float64; one such unit moves a whole column of a weight gradient by ~1 % of its size.
    Backward therefore uses the device's decisions (forward does not: it has no jump)."""
    h = [x.astype(np.float64)]
    for l, (W, b) in enumerate(zip(Ws, bs)):
        z = h[-1] @ W.astype(np.float64) + b.astype(np.float64)
        h.append(np.maximum(z, 0.0) if l + 1 < len(Ws) else z)
    logits = h[-1]
    zmax = logits.max(axis=1, keepdims=True)
    e = np.exp(logits - zmax)
    p = e / e.sum(axis=1, keepdims=True)
    onehot = np.zeros_like(p)
    onehot[np.arange(len(labels)), labels.astype(int)] = 1.0
    loss = -(onehot * np.log(np.maximum(p, 1e-10))).sum()
    g = p - onehot
    gW, gb = [None] * len(Ws), [None] * len(Ws)
    flips = 0
    for l in range(len(Ws) - 1, -1, -1):
        gb[l] = g[0].copy()
        gW[l] = h[l].T @ g
        if l > 0:
            flips += int(np.count_nonzero(masks[l - 1] != (h[l] > 0)))
            g = (g @ (Ws_back or Ws)[l].astype(np.float64).T) * masks[l - 1]
    newW = [W.astype(np.float64) - lr * gw for W, gw in zip(Ws, gW)]
    newb = [b.astype(np.float64) - lr * g_ for b, g_ in zip(bs, gb)]
    return logits, loss, gW, gb, newW, newb, flips


def test_config5_one_full_width_step(cb, orc):
    """784-4096-4096-4096-10, batch 8192, one step: logits of sampled rows against the oracle run on
    those rows (forward is row-independent), loss, every gradient and the updated weights against a
    float64 evaluation of the same step."""
    import oracle
    from ctorch_b200 import frontend as F
    F.set_quiet(True)
    dims, batch, lr = [784, 4096, 4096, 4096, 10], 8192, 0.01
    rng = np.random.default_rng(42)
    Ws, bs = [], []
    for i, j in zip(dims[:-1], dims[1:]):
        lim = np.sqrt(6.0 / i)
        Ws.append(rng.uniform(-lim, lim, (i, j)).astype(np.float32))
        bs.append((0.01 * rng.standard_normal(j)).astype(np.float32))   # non-zero, so the bias add is visible
    params = oracle.pack_params(Ws, bs)
    drng = np.random.default_rng(1234)
    x = drng.integers(0, 256, (batch, dims[0])).astype(np.float32) / np.float32(255.0)
    labels = drng.integers(0, dims[-1], batch).astype(np.float32)

    tr = F.MlpTrainer(dims, params, lr)
    tr.keep_logits(True)
    loss = tr.step_host(x, labels)
    logits = tr.logits(batch)
    grads, new_params = tr.grads(), tr.params()
    _status_ok(cb)

    # (1) sampled rows through the oracle (the reference's arithmetic, row by row)
    rows = np.array([0, 1, 4095, 4096, 8191, 777, 5000, 6001])
    ref = orc.mlp_train(dims, x[rows][None, None], labels[rows][None, None], params, lr, 1)
    assert_matmul_close(logits[rows], ref["logits"][0], 1e-4, "logits of sampled rows vs the oracle")

    # (2) the whole step in float64; the hidden units' on/off decisions come from the device (the same
    # fused product + bias + ReLU kernel the trainer's forward runs, outside any tape)
    h = F.Tensor.from_numpy(x)
    masks = []
    for l in range(len(Ws) - 1):
        h = h.linear(F.Tensor.from_numpy(Ws[l]), F.Tensor.from_numpy(bs[l]), True)
        masks.append(h.numpy() > 0)
    del h
    l64, loss64, gW, gb, newW, newb, flips = _fp64_step(dims, x, labels, Ws, bs, lr, masks)
    print(f"\nhidden units whose on/off decision differs between the device and float64: {flips} of {sum(m.size for m in masks)}")
    assert flips <= 1e-5 * sum(m.size for m in masks)
    report = {"logits": _normwise(logits, l64), "loss (rel)": abs(loss - loss64) / abs(loss64)}
    gW_gpu, gb_gpu = oracle.unpack_params(grads, dims)
    W_gpu, b_gpu = oracle.unpack_params(new_params, dims)
    for l in range(len(Ws)):
        report[f"dW{l}"] = _normwise(gW_gpu[l], gW[l])
        report[f"db{l} (row 0 of the upstream gradient)"] = _normwise(gb_gpu[l], gb[l])
        report[f"updated W{l}"] = _normwise(W_gpu[l], newW[l])
        report[f"updated b{l}"] = _normwise(b_gpu[l], newb[l])
        # the update really happened: the step is far above the resolution of the comparison
        assert np.abs(W_gpu[l].astype(np.float64) - Ws[l]).max() > 0
    print("normwise errors of one full-width step against float64:")
    for k_, v in report.items():
        print(f"  {k_}: {v:.2e}")
    bad = {k_: v for k_, v in report.items() if not v <= 1e-4}
    assert not bad, f"above 1e-4: {bad}"


# ---- config 4: [65536, 32000] row-wise kernels ----------------------------------------------------------
def _rows_of(dev, rows, cols):
    return np.stack([dev.view(int(r) * cols, (cols,)).numpy() for r in rows])


def _assert_rows_close_or_better(got, ref, exact, what, rel=1e-5, abs_=1e-12):
    """Rows that contain a sum of tens of thousands of terms: the reference adds them one by one in
    float32 and is itself ~1e-5 away from the exact value, so the device result passes if it is
    within rel of the float64 value, or at least as close to it as the reference is (per row)."""
    got, ref, exact = (np.asarray(v, np.float64) for v in (got, ref, exact))
    scale = np.abs(exact).max(axis=1, keepdims=True)
    eg = (np.abs(got - exact) / scale).max(axis=1)
    er = (np.abs(ref - exact) / scale).max(axis=1)
    bad = ~((eg <= rel + abs_) | (eg <= er))
    assert not bad.any(), f"{what}: {np.count_nonzero(bad)} rows; device error {eg.max():.2e}, reference error {er.max():.2e} (both against float64, per-row normwise)"
    return float(eg.max()), float(er.max())


def _softmax64(x):
    z = x.astype(np.float64)
    e = np.exp(z - z.max(axis=1, keepdims=True))
    return e / e.sum(axis=1, keepdims=True)


def test_config4_rowwise_at_65536_x_32000(cb, orc):
    """Softmax forward / backward, cross entropy (index labels) and the fused CE forward+backward on
    8.4 GB of logits: rows on both sides of the 2^32-byte offset, the first and last rows and random
    ones against the oracle; the summed loss against its own row slabs and one slab against the
    oracle."""
    R, C = 65536, 32000
    i64 = ctypes.c_int64
    x = cb.ops.rand_uniform((R, C), seed=7)                 # every element distinct: U[0,1)
    cb.ops.scalar(0, x, 12.0, out=x)                        # t*s
    cb.ops.scalar(1, x, -6.0, out=x)                        # t+s  -> U[-6, 6), the spread of N(0, 2^2) logits
    rng = np.random.default_rng(5)
    labels = rng.integers(0, C, R).astype(np.float32)
    dl = cb.to_device(labels)
    edge = (1 << 32) // (4 * C)                             # the row that contains byte offset 2^32
    rows = np.unique(np.concatenate([[0, 1, edge - 1, edge, edge + 1, R - 2, R - 1], rng.integers(0, R, 17)]))

    xs = _rows_of(x, rows, C)
    y = cb.ops.softmax(x)
    ys = _rows_of(y, rows, C)
    y64 = _softmax64(xs)
    print("\nsoftmax rows (device, reference) vs float64:", _assert_rows_close_or_better(ys, orc.softmax(xs), y64, "softmax rows"))
    # backward, with the logits themselves standing in for the upstream gradient: y * (g - sum(g * y))
    dx = cb.ops.softmax_backward(y, x)
    g64 = xs.astype(np.float64)
    dx64 = y64 * (g64 - (g64 * y64).sum(axis=1, keepdims=True))
    print("softmax backward rows:", _assert_rows_close_or_better(_rows_of(dx, rows, C), orc.grad_unary("Softmax", xs, xs), dx64, "softmax backward rows"))
    del dx, y
    assert cb.ops.rowwise_status() == 0

    total = float(cb.ops.cross_entropy(x, dl).numpy())
    slab = 4096
    parts = []
    for s in range(0, R, slab):
        parts.append(float(cb.ops.cross_entropy(x.view(s * C, (slab, C)), dl.view(s, (slab,))).numpy()))
    assert abs(total - sum(parts)) <= 1e-5 * abs(total), (total, sum(parts))
    s8 = (edge // slab) * slab                              # the slab that straddles byte offset 2^32
    xs8 = x.view(s8 * C, (slab, C)).numpy()
    ref8 = float(orc.ce(xs8, labels[s8:s8 + slab]))
    z8 = xs8.astype(np.float64)
    zmax = z8.max(axis=1)
    exact8 = float((zmax + np.log(np.exp(z8 - zmax[:, None]).sum(axis=1)) - z8[np.arange(slab), labels[s8:s8 + slab].astype(int)]).sum())
    assert_sum_close(parts[edge // slab], ref8, exact8, "summed cross entropy of the slab across byte offset 2^32")
    del xs8, z8

    loss_f, d = cb.ops.cross_entropy_fused(x, dl)
    assert abs(float(loss_f.numpy()) - total) <= 1e-5 * abs(total)
    onehot = np.zeros((len(rows), C), np.float32)
    onehot[np.arange(len(rows)), labels[rows].astype(int)] = 1
    print("fused CE gradient rows:", _assert_rows_close_or_better(_rows_of(d, rows, C), orc.grad_loss("CE", xs, onehot), y64 - onehot, "fused CE gradient rows"))
    assert cb.ops.rowwise_status() == 0


# ---- config 2: elementwise and Sum at 2^28 -------------------------------------------------------------
def test_config2_elementwise_and_sum_at_2_to_28(cb, orc):
    n = 1 << 28
    rng = np.random.default_rng(11)
    a = rng.random(n, dtype=np.float32) * np.float32(8) - np.float32(4)         # U(-4, 4)
    b = rng.random(n, dtype=np.float32) * np.float32(3.5) + np.float32(0.5)     # U(0.5, 4): no zero divisors
    da, db = cb.to_device(a), cb.to_device(b)
    slabs = [slice(0, 1 << 20), slice((n >> 1) - (1 << 19), (n >> 1) + (1 << 19)), slice(n - (1 << 20), n)]
    stride = np.arange(12345, n, 65521)
    out = cb.empty((n,))

    def sample(arr):
        return np.concatenate([arr[s] for s in slabs] + [arr[stride]])

    sa, sb = sample(a), sample(b)
    for op in ("Add", "Sub", "Mul", "Div"):
        got = cb.ops.binary(op, da, db, out=out).numpy()
        assert_exact(sample(got), orc.binary(op, sa, sb), f"{op} at 2^28")
    # the whole array for one exact op: nothing lost, nothing misplaced anywhere
    assert_exact(cb.ops.binary("Add", da, db, out=out).numpy(), a + b, "Add at 2^28, every element")
    for op in ("Neg", "ReLU"):
        assert_exact(sample(cb.ops.unary(op, da, out=out).numpy()), orc.unary(op, sa), f"{op} at 2^28")
    for op in ("Sigmoid", "Tanh", "Sin", "Cos"):
        assert_close(sample(cb.ops.unary(op, da, out=out).numpy()), orc.unary(op, sa), 1e-5, 1e-6, f"{op} at 2^28")
    # backward of Mul (the 20 B/element form) and of Tanh
    g = rng.standard_normal(n, dtype=np.float32)
    dg = cb.to_device(g)
    sg = sample(g)
    dA, dB = cb.ops.binary_backward("Mul", da, db, dg)
    rA, rB = orc.grad_binary("Mul", sa, sb, sg)
    assert_exact(sample(dA.numpy()), rA, "Mul backward da at 2^28")
    assert_exact(sample(dB.numpy()), rB, "Mul backward db at 2^28")
    del dA, dB
    # (1 - t^2) * g: the transcendental's 1e-6 absolute term scales with the upstream gradient (|g| up to ~6 here)
    assert_close(sample(cb.ops.unary_backward("Tanh", da, dg).numpy()), orc.grad_unary("Tanh", sa, sg), 1e-5, 1e-6 * float(np.abs(sg).max()), "Tanh backward at 2^28")
    # Sum: against float64, and at least as accurate as the reference's sequential fp32 sum
    s_gpu = float(cb.ops.sum(da).numpy())
    assert_sum_close(s_gpu, orc.sum(a), a.sum(dtype=np.float64), "Sum at 2^28")
