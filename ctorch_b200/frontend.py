"""Python face of the C++ front end (ctorch_b200_frontend.h): Tensor, AutoDiff context, MLP trainer.

Mirrors the reference's user-level API so tests read like the reference's own: operators, relu(),
matmul(), cross_entropy(), backward(loss), grad(t).  No compute happens in Python.
"""
import ctypes

import numpy as np

from ._lib import lib, CtkError

OP = dict(Add=0, Sub=1, Neg=2, Mul=3, Div=4, MatMul=5, Dot=6, Cos=7, Sin=8, ReLU=11, Tanh=12, Sigmoid=13,
          Softmax=14, MSE=17, MAE=18, CE=19, Sum=21)
CPU, CUDA = 0, 1
_vp = ctypes.c_void_p


class FrontendError(RuntimeError):
    pass


def _chk(rc):
    if rc:
        raise FrontendError(lib.cth_last_error().decode("utf-8", "replace"))


def cuda_available():
    return bool(lib.cth_cuda_available())


def set_quiet(q=True):
    lib.cth_set_quiet(1 if q else 0)


FLOAT, DOUBLE, INT, LONG, BOOL = 0, 1, 2, 3, 4          # enum class DType
NP_DTYPES = {0: np.float32, 1: np.float64, 2: np.int32, 3: np.int64, 4: np.bool_}


def manual_seed(seed):
    _chk(lib.cth_manual_seed(ctypes.c_uint64(seed)))


class Tensor:
    def __init__(self, handle):
        self.h = handle

    @staticmethod
    def from_numpy(a, device=CUDA):
        a = np.require(a, dtype=np.float32, requirements="C")
        shape = np.asarray(a.shape, dtype=np.int64)
        h = _vp()
        _chk(lib.cth_tensor_from_host(a.ctypes.data_as(_vp), shape.ctypes.data_as(_vp), a.ndim, device, ctypes.byref(h)))
        return Tensor(h)

    @staticmethod
    def zeros(shape, device=CUDA):
        s = np.asarray(shape, dtype=np.int64)
        h = _vp()
        _chk(lib.cth_tensor_from_host(None, s.ctypes.data_as(_vp), len(shape), device, ctypes.byref(h)))
        return Tensor(h)

    @staticmethod
    def scalar(v):
        h = _vp()
        _chk(lib.cth_tensor_scalar(ctypes.c_float(v), ctypes.byref(h)))
        return Tensor(h)

    def narrow_rows(self, start, count):
        """Rows [start, start+count) as a view of the same buffer."""
        h = _vp()
        _chk(lib.cth_tensor_narrow_rows(self.h, ctypes.c_int64(start), ctypes.c_int64(count), ctypes.byref(h)))
        return Tensor(h)

    def info(self):
        shape = (ctypes.c_int64 * 8)()
        rank, dev, rg = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        tid = ctypes.c_uint64()
        _chk(lib.cth_tensor_info(self.h, shape, ctypes.byref(rank), ctypes.byref(dev), ctypes.byref(rg), ctypes.byref(tid)))
        return dict(shape=tuple(shape[i] for i in range(rank.value)), device=dev.value, requires_grad=bool(rg.value), id=tid.value)

    @property
    def shape(self):
        return self.info()["shape"]

    @property
    def dtype(self):
        d = ctypes.c_int()
        _chk(lib.cth_tensor_dtype(self.h, ctypes.byref(d)))
        return d.value

    def numpy(self):
        dt = self.dtype
        if dt == FLOAT:
            out = np.empty(self.shape, np.float32)
            _chk(lib.cth_tensor_to_host(self.h, out.ctypes.data_as(_vp)))
            return out
        out = np.empty(self.shape, NP_DTYPES[dt])      # other dtypes: memory order
        _chk(lib.cth_tensor_read_raw(self.h, out.ctypes.data_as(_vp), ctypes.c_uint64(out.nbytes)))
        return out

    @staticmethod
    def empty(shape, dtype=0, device=CUDA):
        s = np.asarray(shape, dtype=np.int64)
        h = _vp()
        _chk(lib.cth_tensor_empty(s.ctypes.data_as(_vp), len(shape), dtype, device, ctypes.byref(h)))
        return Tensor(h)

    def _cmp(self, cmp, other, scalar_left=False):
        h = _vp()
        if isinstance(other, Tensor):
            _chk(lib.cth_tensor_compare(self.h, other.h, ctypes.c_float(0), cmp, 0, ctypes.byref(h)))
        else:
            _chk(lib.cth_tensor_compare(self.h, None, ctypes.c_float(other), cmp, 2 if scalar_left else 1, ctypes.byref(h)))
        return Tensor(h)

    def __gt__(self, o): return self._cmp(0, o)
    def __lt__(self, o): return self._cmp(1, o)
    def __eq__(self, o): return self._cmp(2, o)
    def __ge__(self, o): return self._cmp(3, o)
    def __le__(self, o): return self._cmp(4, o)
    def __ne__(self, o): return self._cmp(5, o)
    __hash__ = object.__hash__

    def scalar_cmp(self, cmp, s):
        """s cmp self: the free operators with the scalar on the left."""
        return self._cmp(cmp, s, scalar_left=True)

    def to_dtype(self, dtype):
        h = _vp()
        _chk(lib.cth_tensor_to_dtype(self.h, dtype, ctypes.byref(h)))
        return Tensor(h)

    def ones(self):
        _chk(lib.cth_tensor_ones(self.h))
        return self

    def rand(self):
        _chk(lib.cth_tensor_rand(self.h))
        return self

    def __getitem__(self, i):
        h = _vp()
        _chk(lib.cth_tensor_index(self.h, ctypes.c_uint64(i), ctypes.byref(h)))
        return Tensor(h)

    def item(self):
        v = ctypes.c_float()
        _chk(lib.cth_tensor_item(self.h, ctypes.byref(v)))
        return np.float32(v.value)

    def requires_grad(self, flag=True):
        _chk(lib.cth_tensor_requires_grad(self.h, 1 if flag else 0))
        return self

    def to(self, device):
        h = _vp()
        _chk(lib.cth_tensor_to_device(self.h, device, ctypes.byref(h)))
        return Tensor(h)

    def copy(self):
        h = _vp()
        _chk(lib.cth_tensor_copy(self.h, ctypes.byref(h)))
        return Tensor(h)

    def fill(self, v):
        _chk(lib.cth_tensor_fill(self.h, ctypes.c_float(v)))
        return self

    def t(self):
        h = _vp()
        _chk(lib.cth_transpose(self.h, ctypes.byref(h)))
        return Tensor(h)

    def _un(self, op, param=0):
        h = _vp()
        _chk(lib.cth_unary(self.h, OP[op], param, ctypes.byref(h)))
        return Tensor(h)

    def _bin(self, other, op):
        h = _vp()
        _chk(lib.cth_binary(self.h, other.h, OP[op], ctypes.byref(h)))
        return Tensor(h)

    def _sc(self, s, kind):
        h = _vp()
        _chk(lib.cth_scalar(self.h, ctypes.c_float(s), kind, ctypes.byref(h)))
        return Tensor(h)

    def relu(self): return self._un("ReLU")
    def sigmoid(self): return self._un("Sigmoid")
    def tanh(self): return self._un("Tanh")
    def sin(self): return self._un("Sin")
    def cos(self): return self._un("Cos")
    def softmax(self, dim=-1): return self._un("Softmax", dim)

    def linear(self, w, bias, relu=False):
        """(self.matmul(w) + bias)[.relu()] in one kernel where possible."""
        h = _vp()
        _chk(lib.cth_linear(self.h, w.h, bias.h, 1 if relu else 0, ctypes.byref(h)))
        return Tensor(h)

    def sum(self): return self._un("Sum")
    def __neg__(self): return self._un("Neg")
    def matmul(self, o): return self._bin(o, "MatMul")
    def dot(self, o): return self._bin(o, "Dot")
    def mse_loss(self, o): return self._bin(o, "MSE")
    def mae_loss(self, o): return self._bin(o, "MAE")
    def cross_entropy(self, o): return self._bin(o, "CE")
    def __add__(self, o): return self._bin(o, "Add") if isinstance(o, Tensor) else self._sc(o, 1)
    def __sub__(self, o): return self._bin(o, "Sub")
    def __mul__(self, o): return self._bin(o, "Mul") if isinstance(o, Tensor) else self._sc(o, 0)
    def __truediv__(self, o): return self._bin(o, "Div") if isinstance(o, Tensor) else self._sc(o, 2)
    def __radd__(self, s): return self._sc(s, 6)
    def __rmul__(self, s): return self._sc(s, 5)
    def __rsub__(self, s): return self._sc(s, 3)
    def __rtruediv__(self, s): return self._sc(s, 4)

    def sgd_update_(self, g, lr):
        _chk(lib.cth_sgd_update(self.h, g.h, ctypes.c_float(lr)))

    def __del__(self):
        try:
            if self.h:
                lib.cth_tensor_free(self.h)
        except Exception:
            pass


def mnist_load(directory, which="train", device=CUDA, image_file=None, label_file=None):
    """MNISTLoader: (images [n, rows*cols] of pixel/255, labels [n] as floats) from the IDX files of
    `directory`: the training pair, the test pair (which="test") or a named pair."""
    im, lb = _vp(), _vp()
    if image_file is not None and label_file is not None:
        a, b = image_file.encode(), label_file.encode()
    elif which == "test":
        a, b = b"test", None
    else:
        a, b = None, None
    _chk(lib.cth_mnist_load(str(directory).encode(), a, b, device, ctypes.byref(im), ctypes.byref(lb)))
    return Tensor(im), Tensor(lb)


class AutoDiff:
    """`AutoDiff ctx; AutoDiffContext::Guard guard(&ctx);` as a Python context manager."""

    def __init__(self):
        h = _vp()
        _chk(lib.cth_ctx_create(ctypes.byref(h)))
        self.h = h

    def __enter__(self):
        _chk(lib.cth_ctx_set_current(self.h))
        return self

    def __exit__(self, *a):
        _chk(lib.cth_ctx_set_current(None))

    def make_leaf(self, t, requires_grad=True): _chk(lib.cth_ctx_make_leaf(self.h, t.h, 1 if requires_grad else 0))
    def zero_grad(self, t): _chk(lib.cth_ctx_zero_grad(self.h, t.h))
    def clear_graph(self): _chk(lib.cth_ctx_clear(self.h))
    def release_step_nodes(self): _chk(lib.cth_ctx_release_step_nodes(self.h))
    def set_fuse_relu_backward(self, on): _chk(lib.cth_ctx_set_fuse_relu_backward(self.h, 1 if on else 0))
    def count_leaf_grads(self, on=True): _chk(lib.cth_ctx_count_leaf_grads(self.h, 1 if on else 0))

    def leaf_grad_count(self, t):
        """How often the leaf-gradient hook fired for tensor t since count_leaf_grads()."""
        n = ctypes.c_uint64()
        _chk(lib.cth_ctx_leaf_grad_count(self.h, t.h, ctypes.byref(n)))
        return n.value

    def node_count(self):
        n = ctypes.c_uint64()
        _chk(lib.cth_ctx_node_count(self.h, ctypes.byref(n)))
        return n.value

    def __del__(self):
        try:
            lib.cth_ctx_destroy(self.h)
        except Exception:
            pass


def backward(root, grad_output=None):
    _chk(lib.cth_backward(root.h, grad_output.h if grad_output is not None else None))


def grad(t):
    h = _vp()
    _chk(lib.cth_grad(t.h, ctypes.byref(h)))
    return Tensor(h)


class MlpTrainer:
    """The training step of mnist/mnist.cpp for any layer list (see ctorch_b200_frontend.h)."""

    def __init__(self, dims, params, lr):
        self.dims = [int(d) for d in dims]
        d = np.asarray(self.dims, dtype=np.int64)
        p = np.require(params, dtype=np.float32, requirements="C")
        h = _vp()
        _chk(lib.cth_mlp_create(len(self.dims) - 1, d.ctypes.data_as(_vp), p.ctypes.data_as(_vp), ctypes.c_float(lr), ctypes.byref(h)))
        self.h = h
        n = ctypes.c_int64()
        _chk(lib.cth_mlp_n_params(self.h, ctypes.byref(n)))
        self.n_params = n.value

    def set_comm(self, comm_handle):
        _chk(lib.cth_mlp_set_comm(self.h, comm_handle))

    DP_MODES = {"inplace": 0, "arena": 1, "serial": 2, "sharded": 3}

    def set_dp_mode(self, mode):
        """How gradients cross the ranks (before set_comm): 'inplace' (default), 'arena', 'serial', 'sharded'."""
        _chk(lib.cth_mlp_set_dp_mode(self.h, self.DP_MODES.get(mode, mode)))

    def set_comm_timeout_ms(self, ms):
        _chk(lib.cth_mlp_set_comm_timeout_ms(self.h, int(ms)))

    def set_corrected(self, exact_bias_grad=True, fresh_weights=True):
        """Opt-in: true bias gradients and backward against the current weights (not the reference's arithmetic)."""
        _chk(lib.cth_mlp_set_corrected(self.h, 1 if exact_bias_grad else 0, 1 if fresh_weights else 0))

    def set_deferred_loss(self, on=True):
        """Steps return without waiting for the device (and report 0); sync_losses() reads the losses."""
        _chk(lib.cth_mlp_set_deferred_loss(self.h, 1 if on else 0))

    def sync_losses(self):
        out = (ctypes.c_float * 16)()
        n = ctypes.c_int()
        _chk(lib.cth_mlp_sync_losses(self.h, out, 16, ctypes.byref(n)))
        return np.asarray(out[:n.value], np.float32)

    def keep_logits(self, keep=True):
        _chk(lib.cth_mlp_keep_logits(self.h, 1 if keep else 0))

    def step_host(self, x, labels):
        """x, labels: numpy arrays or raw host pointers (ints) with an explicit batch via x.shape[0]."""
        loss = ctypes.c_float()
        _chk(lib.cth_mlp_step_host(self.h, x.ctypes.data_as(_vp), labels.ctypes.data_as(_vp), ctypes.c_int64(x.shape[0]), ctypes.byref(loss)))
        return loss.value

    def stage_host(self, x, labels):
        """Starts the upload of a batch; returns at once for page-locked arrays."""
        _chk(lib.cth_mlp_stage_host(self.h, x.ctypes.data_as(_vp), labels.ctypes.data_as(_vp), ctypes.c_int64(x.shape[0])))

    def step_staged(self):
        """The step on the oldest staged batch."""
        loss = ctypes.c_float()
        _chk(lib.cth_mlp_step_staged(self.h, ctypes.byref(loss)))
        return loss.value

    def predict(self, x):
        """Class probabilities of a device batch (NeuralNetwork::predict)."""
        h = _vp()
        _chk(lib.cth_mlp_predict(self.h, x.h, ctypes.byref(h)))
        return Tensor(h)

    def accuracy(self, x, labels):
        """calculate_accuracy on the device: fraction of rows whose first-maximum class equals the label."""
        a = ctypes.c_float()
        _chk(lib.cth_mlp_accuracy(self.h, x.h, labels.h, ctypes.byref(a)))
        return a.value

    def train_epoch(self, images, labels, batch_size):
        """One pass over a device-resident data set in consecutive batches; returns the mean step loss."""
        loss = ctypes.c_float()
        _chk(lib.cth_mlp_train_epoch(self.h, images.h, labels.h, ctypes.c_int64(batch_size), ctypes.byref(loss)))
        return loss.value

    def step_graph_host(self, x, labels):
        """The step replayed as a CUDA graph (recorded on the second call of a batch size)."""
        loss = ctypes.c_float()
        _chk(lib.cth_mlp_step_graph_host(self.h, x.ctypes.data_as(_vp), labels.ctypes.data_as(_vp), ctypes.c_int64(x.shape[0]), ctypes.byref(loss)))
        return loss.value

    def train_epoch_graph(self, images, labels, batch_size):
        loss = ctypes.c_float()
        _chk(lib.cth_mlp_train_epoch_graph(self.h, images.h, labels.h, ctypes.c_int64(batch_size), ctypes.byref(loss)))
        return loss.value

    def step_device(self, x, onehot):
        loss = ctypes.c_float()
        _chk(lib.cth_mlp_step_device(self.h, x.h, onehot.h, ctypes.byref(loss)))
        return loss.value

    def params(self):
        out = np.empty(self.n_params, np.float32)
        _chk(lib.cth_mlp_get_params(self.h, out.ctypes.data_as(_vp)))
        return out

    def grads(self):
        out = np.empty(self.n_params, np.float32)
        _chk(lib.cth_mlp_get_grads(self.h, out.ctypes.data_as(_vp)))
        return out

    def logits(self, batch):
        out = np.empty((batch, self.dims[-1]), np.float32)
        _chk(lib.cth_mlp_get_logits(self.h, out.ctypes.data_as(_vp)))
        return out

    def node_count(self):
        n = ctypes.c_uint64()
        _chk(lib.cth_mlp_node_count(self.h, ctypes.byref(n)))
        return n.value

    def __del__(self):
        try:
            lib.cth_mlp_destroy(self.h)
        except Exception:
            pass
