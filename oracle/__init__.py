"""TEST INFRASTRUCTURE ONLY: the parity oracle.

Two CPU implementations behind one numpy-facing interface:

* ``Oracle``    -- ``libctorch_oracle.so``, the plain-C restatement in ``ctorch_oracle.c``.
* ``Reference`` -- ``_ref/libctorch_ref.so``, the UNMODIFIED reference sources compiled where they
  lie plus ``ref_shim.cpp``.  Only exists where it has been built (``make -C oracle``).

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline leg may import this
package; the product package never does.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libctorch_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libctorch_ref.so")

OP = dict(Add=0, Sub=1, Neg=2, Mul=3, Div=4, MatMul=5, Dot=6, Cos=7, Sin=8, ReLU=11, Tanh=12,
          Sigmoid=13, Softmax=14, MSE=17, MAE=18, CE=19, Sum=21)
B_SAME, B_SCALAR, B_ROW, A_SCALAR = 0, 1, 2, 3

_f32p = ctypes.POINTER(ctypes.c_float)
_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int)


def _fp(a):
    return a.ctypes.data_as(_f32p) if a is not None else None


def _f32(a):
    # np.ascontiguousarray would promote a 0-D array to shape (1,); 0-D operands matter here.
    return np.require(a, dtype=np.float32, requirements="C")


def _shape(a):
    s = np.asarray(a.shape, dtype=np.int64)
    return s, s.ctypes.data_as(_i64p), a.ndim


def reference_root():
    """Where the reference checkout is looked for: $CTORCH_REFERENCE_ROOT, else a directory named
    `reference` beside this repository.  The path need not exist."""
    return os.environ.get("CTORCH_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def build(ref_root=None):
    """Compile the C restatement (always) and the reference library (if its sources are there)."""
    subprocess.run(["make", "-s", "-C", HERE, f"REF={ref_root or reference_root()}"], check=True)


def pack_params(Ws, bs):
    return np.concatenate([np.concatenate([_f32(W).ravel(), _f32(b).ravel()]) for W, b in zip(Ws, bs)])


def unpack_params(p, dims):
    Ws, bs, o = [], [], 0
    for i, j in zip(dims[:-1], dims[1:]):
        Ws.append(p[o:o + i * j].reshape(i, j)); o += i * j
        bs.append(p[o:o + j]); o += j
    return Ws, bs


# ---- the MNIST application path: IDX files, prediction, accuracy (byte / integer work: numpy) ----
def idx_write_images(path, pixels_u8):
    """Writes an IDX3 image file ([n, rows, cols] uint8): big-endian magic 2051 and extents, then bytes."""
    a = np.require(pixels_u8, dtype=np.uint8, requirements="C")
    with open(path, "wb") as f:
        f.write(np.asarray([2051, a.shape[0], a.shape[1], a.shape[2]], ">i4").tobytes())
        f.write(a.tobytes())


def idx_write_labels(path, labels_u8):
    a = np.require(labels_u8, dtype=np.uint8, requirements="C")
    with open(path, "wb") as f:
        f.write(np.asarray([2049, a.shape[0]], ">i4").tobytes())
        f.write(a.tobytes())


def idx_read_images(path):
    """MNISTLoader::read_images (mnist/mnist_loader.cpp:7-44): magic 2051, n, rows, cols as big-endian
    int32, then one byte per pixel, each stored as pixel / 255.0f.  Returns [n, rows*cols] float32."""
    raw = open(path, "rb").read()
    magic, n, rows, cols = (int(v) for v in np.frombuffer(raw[:16], ">i4"))
    if magic != 2051:
        raise ValueError("not an IDX image file")
    px = np.frombuffer(raw[16:16 + n * rows * cols], np.uint8)
    return (px.astype(np.float32) / np.float32(255.0)).reshape(n, rows * cols)


def idx_read_images_from_bytes(pixels_u8):
    """The same normalisation on an in-memory [n, rows, cols] uint8 array."""
    a = np.asarray(pixels_u8, np.uint8)
    return (a.astype(np.float32) / np.float32(255.0)).reshape(a.shape[0], -1)


def idx_read_labels(path):
    """MNISTLoader::read_labels (:46-73) + the float copy of load_training_data (:113-115)."""
    raw = open(path, "rb").read()
    magic, n = (int(v) for v in np.frombuffer(raw[:8], ">i4"))
    if magic != 2049:
        raise ValueError("not an IDX label file")
    return np.frombuffer(raw[8:8 + n], np.uint8).astype(np.float32)


# ---- comparisons, dtype conversion, operator[] (plain numpy: byte / integer work) -----------------------
CMP_NAMES = ("gt", "lt", "eq", "ge", "le", "ne")
_CMP_FUN = dict(gt=np.greater, lt=np.less, eq=np.equal, ge=np.greater_equal, le=np.less_equal, ne=np.not_equal)
NP_OF_DTYPE = {0: np.float32, 1: np.float64, 2: np.int32, 3: np.int64, 4: np.bool_}


def compare(cmp, a, other, scalar_left=False):
    """Tensor::operator>, <, ==, >=, <=, != (src/Tensor.cpp:985-1309) and the free operators with the
    scalar on the left (:1462-1591): element by element in memory order, IEEE comparisons, a kBool
    result of a's shape.  `other` is an array of a's shape or a float."""
    a = _f32(a)
    f = _CMP_FUN[cmp]
    if isinstance(other, np.ndarray):
        if other.shape != a.shape:
            raise ValueError("tensor shapes differ")        # :1124-1126 throws
        return f(a, _f32(other))
    s = np.float32(other)
    return f(s, a) if scalar_left else f(a, s)


def cast_from_float(a, dtype_code):
    """Tensor::to(DType) out of float (src/Tensor.cpp:199-243): static_cast per element -- exact to
    double, truncation toward zero to int32 / int64 (inside the target's range; outside it the
    reference's behaviour is undefined), != 0 to bool."""
    a = _f32(a)
    if dtype_code in (2, 3):
        return np.trunc(a).astype(NP_OF_DTYPE[dtype_code])
    if dtype_code == 4:
        return a != 0
    return a.astype(NP_OF_DTYPE[dtype_code])


def index_1d(a, i):
    """Tensor::operator[] (src/Tensor.cpp:175-189): 1-D only, range-checked, a view of one element."""
    a = _f32(a)
    if a.ndim != 1:
        raise ValueError("1-D tensors only")
    if not 0 <= i < a.shape[0]:
        raise IndexError("index out of range")
    return a[i:i + 1]


def predicted_labels(probs):
    """The prediction loop of calculate_accuracy (mnist/mnist.cpp:140-147): per row the first class whose
    probability exceeds -1 and every earlier one (NaN never does); 0 if none."""
    p = np.asarray(probs, np.float32)
    out = np.zeros(p.shape[0], np.int64)
    for i in range(p.shape[0]):
        best, lab = np.float32(-1.0), 0
        for j in range(p.shape[1]):
            if p[i, j] > best:
                best, lab = p[i, j], j
        out[i] = lab
    return out


def accuracy(probs, labels):
    """calculate_accuracy (:134-158): float(correct) / total with (int)label."""
    pred = predicted_labels(probs)
    correct = int((pred == np.asarray(labels, np.float32).astype(np.int64)).sum())
    return np.float32(correct) / np.float32(len(pred))


_ORACLE_LIB = None


def _oracle_lib():
    global _ORACLE_LIB
    if _ORACLE_LIB is None:
        if not os.path.exists(ORACLE_SO):
            build()
        _ORACLE_LIB = ctypes.CDLL(ORACLE_SO)
    return _ORACLE_LIB


class Oracle:
    """ctypes face of ctorch_oracle.c."""

    kind = "port"

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build()
        L = self.L = ctypes.CDLL(ORACLE_SO)
        for name in ("orc_sum", "orc_dot", "orc_mse", "orc_mae", "orc_ce_onehot"):
            getattr(L, name).restype = ctypes.c_float

    # ---- forward ----
    def binary(self, op, a, b, bmode=B_SAME):
        a, b = _f32(a), _f32(b)
        big = b if bmode == A_SCALAR else a
        out = np.empty_like(big)
        inner = b.size if bmode == B_ROW else 1
        self.L.orc_binary(OP[op], _fp(a), _fp(b), _fp(out), ctypes.c_int64(big.size), bmode, ctypes.c_int64(inner))
        return out

    def unary(self, op, a):
        a = _f32(a)
        out = np.empty_like(a)
        self.L.orc_unary(OP[op], _fp(a), _fp(out), ctypes.c_int64(a.size))
        return out

    def scalar(self, kind, a, s):
        a = _f32(a)
        out = np.empty_like(a)
        self.L.orc_scalar(kind, _fp(a), ctypes.c_int64(a.size), ctypes.c_float(s), _fp(out))
        return out

    def matmul(self, a, b, ta=False, tb=False):
        """a stored [m,k] (or [k,m] if ta), b stored [k,n] (or [n,k] if tb)."""
        a, b = _f32(a), _f32(b)
        m, k = (a.shape[1], a.shape[0]) if ta else a.shape
        n = b.shape[0] if tb else b.shape[1]
        sa = (1, m) if ta else (k, 1)
        sb = (1, k) if tb else (n, 1)
        c = np.empty((m, n), np.float32)
        i64 = ctypes.c_int64
        self.L.orc_matmul(_fp(a), _fp(b), _fp(c), i64(m), i64(k), i64(n), i64(sa[0]), i64(sa[1]), i64(sb[0]), i64(sb[1]))
        return c

    def matmul_rows(self, a, b, rows, ta=False, tb=False):
        a, b = _f32(a), _f32(b)
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        m, k = (a.shape[1], a.shape[0]) if ta else a.shape
        n = b.shape[0] if tb else b.shape[1]
        sa = (1, m) if ta else (k, 1)
        sb = (1, k) if tb else (n, 1)
        c = np.empty((rows.size, n), np.float32)
        i64 = ctypes.c_int64
        self.L.orc_matmul_rows(_fp(a), _fp(b), _fp(c), rows.ctypes.data_as(_i64p), i64(rows.size), i64(k), i64(n),
                               i64(sa[0]), i64(sa[1]), i64(sb[0]), i64(sb[1]))
        return c

    def matmul_entries(self, a, b, rows, cols, ta=False, tb=False):
        """(A.B)[rows[e], cols[e]] by the reference's recurrence, for products too large to evaluate in
        full.  Always the C restatement (the reference library can only compute whole products)."""
        a, b = _f32(a), _f32(b)
        rows = np.ascontiguousarray(rows, dtype=np.int64)
        cols = np.ascontiguousarray(cols, dtype=np.int64)
        m, k = (a.shape[1], a.shape[0]) if ta else a.shape
        n = b.shape[0] if tb else b.shape[1]
        sa = (1, m) if ta else (k, 1)
        sb = (1, k) if tb else (n, 1)
        out = np.empty(rows.size, np.float32)
        i64 = ctypes.c_int64
        _oracle_lib().orc_matmul_entries(_fp(a), _fp(b), _fp(out), rows.ctypes.data_as(_i64p), cols.ctypes.data_as(_i64p),
                                         i64(rows.size), i64(k), i64(sa[0]), i64(sa[1]), i64(sb[0]), i64(sb[1]))
        return out

    def sum(self, a):
        a = _f32(a)
        return np.float32(self.L.orc_sum(_fp(a), ctypes.c_int64(a.size)))

    def dot(self, a, b):
        a, b = _f32(a), _f32(b)
        return np.float32(self.L.orc_dot(_fp(a), _fp(b), ctypes.c_int64(a.size)))

    def mse(self, a, b):
        a, b = _f32(a), _f32(b)
        return np.float32(self.L.orc_mse(_fp(a), _fp(b), ctypes.c_int64(a.size)))

    def mae(self, a, b):
        a, b = _f32(a), _f32(b)
        return np.float32(self.L.orc_mae(_fp(a), _fp(b), ctypes.c_int64(a.size)))

    def softmax(self, x):
        x = _f32(x)
        x2 = x.reshape(1, -1) if x.ndim == 1 else x
        out = np.empty_like(x2)
        self.L.orc_softmax_rows(_fp(x2), _fp(out), ctypes.c_int64(x2.shape[0]), ctypes.c_int64(x2.shape[1]))
        return out.reshape(x.shape)

    def softmax_dim0(self, x, g=None):
        """Softmax down the columns of a 2-D array (src/Tensor.cpp:1728-1743): the same recurrence per
        column as the row form per row, so it is the row form of the transpose; with g also the backward
        rule of src/AutoDiff.cpp:1473-1484 (dot accumulated down the column in order)."""
        x = _f32(x)
        y = np.ascontiguousarray(self.softmax(np.ascontiguousarray(x.T)).T)
        if g is None:
            return y
        g = _f32(g)
        dot = np.zeros(x.shape[1], np.float32)
        for i in range(x.shape[0]):
            dot = (dot + g[i] * y[i]).astype(np.float32)
        return y, (y * (g - dot)).astype(np.float32)

    def ce(self, logits, target):
        """target: one-hot of logits' shape, or a [rows] vector of class indices stored as floats."""
        logits, target = _f32(logits), _f32(target)
        l2 = logits.reshape(1, -1) if logits.ndim == 1 else logits
        r, c = l2.shape
        if target.shape == logits.shape:
            return np.float32(self.L.orc_ce_onehot(_fp(l2), _fp(target), ctypes.c_int64(r), ctypes.c_int64(c)))
        loss = ctypes.c_float()
        rc = self.L.orc_ce_index(_fp(l2), _fp(target), ctypes.c_int64(r), ctypes.c_int64(c), ctypes.byref(loss))
        if rc:
            raise ValueError("label out of range")
        return np.float32(loss.value)

    # ---- backward ----
    def grad_unary(self, op, x, g):
        x, g = _f32(x), _f32(g)
        dx = np.empty_like(x)
        if op == "Softmax":
            y = self.softmax(x)
            y2 = y.reshape(1, -1) if y.ndim == 1 else y
            self.L.orc_softmax_backward_rows(_fp(y2), _fp(g), _fp(dx), ctypes.c_int64(y2.shape[0]), ctypes.c_int64(y2.shape[1]))
            return dx
        self.L.orc_grad_unary(OP[op], _fp(x), _fp(g), _fp(dx), ctypes.c_int64(x.size))
        return dx

    def grad_binary(self, op, a, b, g, bmode=B_SAME):
        a, b, g = _f32(a), _f32(b), _f32(g)
        da, db = np.empty_like(a), np.empty_like(b)
        inner = b.size if bmode == B_ROW else 1
        self.L.orc_grad_binary(OP[op], _fp(a), _fp(b), _fp(g), _fp(da), _fp(db), ctypes.c_int64(a.size), bmode, ctypes.c_int64(inner))
        return da, db

    def grad_loss(self, op, p, t, g=1.0):
        p, t = _f32(p), _f32(t)
        dp = np.empty_like(p)
        if op == "CE":
            p2 = p.reshape(1, -1) if p.ndim == 1 else p
            self.L.orc_ce_backward(_fp(p2), _fp(t), ctypes.c_float(g), _fp(dp), ctypes.c_int64(p2.shape[0]), ctypes.c_int64(p2.shape[1]))
        elif op == "MSE":
            self.L.orc_mse_backward(_fp(p), _fp(t), ctypes.c_float(g), _fp(dp), ctypes.c_int64(p.size))
        elif op == "MAE":
            self.L.orc_mae_backward(_fp(p), _fp(t), ctypes.c_float(g), _fp(dp), ctypes.c_int64(p.size))
        else:
            raise ValueError(op)
        return dp

    # ---- training step ----
    _mlp = "orc_mlp_train"

    def mlp_train(self, dims, x, labels, params, lr, steps, grad_steps=(), want_logits=True):
        """x [replicas, n_batches, batch, dims[0]], labels [replicas, n_batches, batch] (floats).
        Returns dict(params, losses [steps, replicas], grads [len(grad_steps), n_params], logits)."""
        x, labels = _f32(x), _f32(labels)
        replicas, n_batches, batch, _ = x.shape
        dims_a = np.asarray(dims, dtype=np.int64)
        p = _f32(params).copy()
        losses = np.zeros((steps, replicas), np.float32)
        gs = np.asarray(list(grad_steps), dtype=np.int32)
        grads = np.zeros((max(len(gs), 1), p.size), np.float32)
        logits = np.zeros((replicas, batch, dims[-1]), np.float32)
        rc = getattr(self.L, self._mlp)(
            len(dims) - 1, dims_a.ctypes.data_as(_i64p), ctypes.c_int64(batch), steps, replicas, _fp(x), _fp(labels),
            n_batches, _fp(p), ctypes.c_float(lr), _fp(losses), gs.ctypes.data_as(_i32p), len(gs), _fp(grads),
            _fp(logits) if want_logits else None)
        if rc:
            raise RuntimeError(self.last_error())
        return dict(params=p, losses=losses, grads=grads[:len(gs)], logits=logits)

    def last_error(self):
        return "oracle error"


class Reference(Oracle):
    """ctypes face of ref_shim.cpp: the reference's own CPU-BASIC results."""

    kind = "reference"
    _mlp = "ref_mlp_train"

    @staticmethod
    def available():
        return os.path.exists(REF_SO)

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO + " (build it with `make -C oracle` where the reference checkout exists)")
        L = self.L = ctypes.CDLL(REF_SO)
        L.ref_last_error.restype = ctypes.c_char_p
        self._chk(L.ref_init())

    def last_error(self):
        return self.L.ref_last_error().decode("utf-8", "replace")

    def softmax_dim(self, x, dim, g=None):
        """Tensor::softmax(dim) of the reference; with g also the gradient of sum(g * softmax(x, dim))."""
        x = _f32(x)
        s = _shape(x)
        out = np.empty_like(x)
        if g is None:
            self._chk(self.L.ref_softmax_dim(_fp(x), s[1], s[2], int(dim), _fp(out), None, None))
            return out
        g = _f32(g)
        dx = np.empty_like(x)
        self._chk(self.L.ref_softmax_dim(_fp(x), s[1], s[2], int(dim), _fp(out), _fp(g), _fp(dx)))
        return out, dx

    def compare(self, cmp, a, other, scalar_left=False):
        """The reference's comparison operators; bool array of a's shape."""
        a = _f32(a)
        s = _shape(a)
        out = np.empty(a.shape, np.uint8)
        c = CMP_NAMES.index(cmp)
        if isinstance(other, np.ndarray):
            b = _f32(other)
            self._chk(self.L.ref_compare(c, 0, _fp(a), _fp(b), ctypes.c_float(0), s[1], s[2], out.ctypes.data_as(ctypes.c_void_p)))
        else:
            self._chk(self.L.ref_compare(c, 2 if scalar_left else 1, _fp(a), None, ctypes.c_float(other), s[1], s[2], out.ctypes.data_as(ctypes.c_void_p)))
        return out.astype(np.bool_)

    def cast_from_float(self, a, dtype_code):
        """The reference's Tensor::to(DType) on a 1-D float tensor."""
        a = _f32(a).ravel()
        out = np.empty(a.size, np.uint8 if dtype_code == 4 else NP_OF_DTYPE[dtype_code])
        self._chk(self.L.ref_cast(int(dtype_code), _fp(a), ctypes.c_int64(a.size), out.ctypes.data_as(ctypes.c_void_p)))
        return out.astype(np.bool_) if dtype_code == 4 else out

    def index_1d(self, a, i):
        a = _f32(a)
        v = ctypes.c_float()
        self._chk(self.L.ref_index(_fp(a), ctypes.c_int64(a.size), ctypes.c_int64(i), ctypes.byref(v)))
        return np.float32(v.value)

    def ones(self, dtype_code, n):
        out = np.empty(n, np.float64)
        self._chk(self.L.ref_ones(int(dtype_code), ctypes.c_int64(n), out.ctypes.data_as(ctypes.c_void_p)))
        return out

    def mnist_load(self, directory, test=False):
        """The reference's own MNISTLoader on `directory`: (images [n, rows*cols], labels [n])."""
        n, sz, nl = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64()
        d = str(directory).encode()
        self._chk(self.L.ref_mnist_load(d, int(test), None, ctypes.c_int64(0), ctypes.byref(n), ctypes.byref(sz), None, ctypes.c_int64(0), ctypes.byref(nl)))
        im = np.empty((n.value, sz.value), np.float32)
        lb = np.empty(nl.value, np.float32)
        self._chk(self.L.ref_mnist_load(d, int(test), _fp(im), ctypes.c_int64(im.size), ctypes.byref(n), ctypes.byref(sz), _fp(lb), ctypes.c_int64(lb.size), ctypes.byref(nl)))
        return im, lb

    def _chk(self, rc):
        if rc:
            raise RuntimeError("reference threw: " + self.last_error())

    def _bin(self, op, a, b):
        a, b = _f32(a), _f32(b)
        _, ap, ar = _shape(a)
        _, bp, br = _shape(b)
        out = np.empty(max(a.size, b.size), np.float32)
        n = ctypes.c_int64()
        sa, sb = _shape(a), _shape(b)
        self._chk(self.L.ref_binary(OP[op], _fp(a), sa[1], ar, _fp(b), sb[1], br, _fp(out), ctypes.byref(n)))
        return out[:n.value]

    def binary(self, op, a, b, bmode=B_SAME):
        a, b = _f32(a), _f32(b)
        if bmode == B_SCALAR:
            b = b.reshape(())       # a 0-D operand is the only scalar form Sub/Mul accept
        if bmode == A_SCALAR:
            a = a.reshape(())
        big = b if bmode == A_SCALAR else a
        return self._bin(op, a, b).reshape(big.shape)

    def unary(self, op, a):
        a = _f32(a)
        s = _shape(a)
        out = np.empty(a.size, np.float32)
        n = ctypes.c_int64()
        self._chk(self.L.ref_unary(OP[op], _fp(a), s[1], s[2], _fp(out), ctypes.byref(n)))
        return out[:n.value].reshape(a.shape if n.value == a.size else ())

    def scalar(self, kind, a, s):
        a = _f32(a)
        out = np.empty_like(a)
        self._chk(self.L.ref_scalar(kind, _fp(a), ctypes.c_int64(a.size), ctypes.c_float(s), _fp(out)))
        return out

    def matmul(self, a, b, ta=False, tb=False):
        a, b = _f32(a), _f32(b)
        m, k = (a.shape[1], a.shape[0]) if ta else a.shape
        n = b.shape[0] if tb else b.shape[1]
        c = np.empty((m, n), np.float32)
        i64 = ctypes.c_int64
        self._chk(self.L.ref_matmul(_fp(a), _fp(b), i64(m), i64(k), i64(n), int(ta), int(tb), _fp(c)))
        return c

    def matmul_rows(self, a, b, rows, ta=False, tb=False):
        return self.matmul(a, b, ta, tb)[np.asarray(rows)]

    def sum(self, a):
        return np.float32(self.unary("Sum", a).reshape(-1)[0])

    def dot(self, a, b):
        return np.float32(self._bin("Dot", a, b)[0])

    def mse(self, a, b):
        return np.float32(self._bin("MSE", a, b)[0])

    def mae(self, a, b):
        return np.float32(self._bin("MAE", a, b)[0])

    def softmax(self, x):
        return self.unary("Softmax", x)

    def softmax_kernel(self, x):
        x = _f32(x)
        s = _shape(x)
        out = np.empty_like(x)
        self._chk(self.L.ref_softmax_kernel(_fp(x), s[1], s[2], _fp(out)))
        return out

    def ce(self, logits, target):
        r = self._bin("CE", logits, target)
        if r.size == 0:
            raise ValueError("label out of range")
        return np.float32(r[0])

    def grad_unary(self, op, x, g):
        x, g = _f32(x), _f32(g)
        s = _shape(x)
        dx = np.empty_like(x)
        self._chk(self.L.ref_grad_unary(OP[op], _fp(x), s[1], s[2], _fp(g), _fp(dx)))
        return dx

    def grad_binary(self, op, a, b, g, bmode=B_SAME):
        a, b, g = _f32(a), _f32(b), _f32(g)
        if bmode == B_SCALAR:
            b = b.reshape(())
        sa, sb = _shape(a), _shape(b)
        da, db = np.empty_like(a), np.empty_like(b)
        self._chk(self.L.ref_grad_binary(OP[op], _fp(a), sa[1], sa[2], _fp(b), sb[1], sb[2], _fp(g), _fp(da), _fp(db)))
        return da, db

    def grad_loss(self, op, p, t, g=1.0):
        p, t = _f32(p), _f32(t)
        sp, st = _shape(p), _shape(t)
        dp = np.empty_like(p)
        gg = np.asarray([g], np.float32)
        self._chk(self.L.ref_grad_binary(OP[op], _fp(p), sp[1], sp[2], _fp(t), st[1], st[2], _fp(gg), _fp(dp), None))
        return dp

    def grad_matmul(self, a, b, g):
        a, b, g = _f32(a), _f32(b), _f32(g)
        sa, sb = _shape(a), _shape(b)
        da, db = np.empty_like(a), np.empty_like(b)
        self._chk(self.L.ref_grad_binary(OP["MatMul"], _fp(a), sa[1], sa[2], _fp(b), sb[1], sb[2], _fp(g), _fp(da), _fp(db)))
        return da, db
