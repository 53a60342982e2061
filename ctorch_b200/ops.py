"""One Python function per C-ABI compute entry point, on DeviceArray operands.

Names follow the reference's operators.  Nothing here computes: each function allocates the result
buffer and forwards to libctorch_b200.so.
"""
import ctypes

import numpy as np

from ._lib import lib, check
from .device import DeviceArray, _sh

OP = dict(Add=0, Sub=1, Neg=2, Mul=3, Div=4, MatMul=5, Dot=6, Cos=7, Sin=8, ReLU=11, Tanh=12, Sigmoid=13,
          Softmax=14, MSE=17, MAE=18, CE=19, Sum=21)
B_SAME, B_SCALAR, B_ROW, A_SCALAR = 0, 1, 2, 3
MODE_3XTF32, MODE_TF32, MODE_FP32_SIMT = 0, 1, 2
MODES = {"3xtf32": 0, "tf32": 1, "fp32_simt": 2}

_i64 = ctypes.c_int64
_f = ctypes.c_float


def binary(op, a, b, layout=B_SAME, out=None, stream=None):
    big = b if layout == A_SCALAR else a
    out = out or DeviceArray(big.shape)
    inner = b.size if layout == B_ROW else 1
    check(lib.ctk_binary_f32(OP[op], a.p, b.p, out.p, _i64(big.size), layout, _i64(inner), _sh(stream)))
    return out


def unary(op, a, out=None, stream=None):
    out = out or DeviceArray(a.shape)
    check(lib.ctk_unary_f32(OP[op], a.p, out.p, _i64(a.size), _sh(stream)))
    return out


def scalar(kind, a, s, out=None, stream=None):
    out = out or DeviceArray(a.shape)
    check(lib.ctk_scalar_f32(kind, a.p, _f(s), out.p, _i64(a.size), _sh(stream)))
    return out


def fill(a, value, stream=None):
    check(lib.ctk_fill_f32(a.p, _f(value), None, _i64(a.size), _sh(stream)))
    return a


def tile(src, n, stream=None):
    out = DeviceArray((n,))
    check(lib.ctk_tile_f32(src.p, _i64(src.size), out.p, _i64(n), _sh(stream)))
    return out


def unary_backward(op, x, g, stream=None):
    dx = DeviceArray(g.shape)
    check(lib.ctk_unary_backward_f32(OP[op], x.p if x is not None else None, g.p, dx.p, _i64(g.size), _sh(stream)))
    return dx


def binary_backward(op, a, b, g, layout=B_SAME, want_da=True, want_db=True, stream=None):
    da = DeviceArray(a.shape) if want_da else None
    db = DeviceArray(b.shape) if want_db else None
    inner = b.size if layout == B_ROW else 1
    check(lib.ctk_binary_backward_f32(OP[op], a.p, b.p, g.p, da.p if da else None, db.p if db else None, _i64(g.size),
                                      layout, _i64(inner), _sh(stream)))
    return da, db


def accumulate(dst, src, stream=None):
    check(lib.ctk_accumulate_f32(dst.p, src.p, _i64(dst.size), _sh(stream)))
    return dst


def sgd_update(p, g, lr, stream=None):
    check(lib.ctk_sgd_update_f32(p.p, g.p, _f(lr), _i64(p.size), _sh(stream)))
    return p


def _scalar_out():
    return DeviceArray(())


def sum(a, scratch=None, stream=None):  # noqa: A001 (mirrors Tensor::sum)
    out = _scalar_out()
    check(lib.ctk_sum_f32(a.p, _i64(a.size), out.p, scratch.p if scratch else None, _sh(stream)))
    return out


def dot(a, b, stream=None):
    out = _scalar_out()
    check(lib.ctk_dot_f32(a.p, b.p, _i64(a.size), out.p, None, _sh(stream)))
    return out


def mse(a, b, stream=None):
    out = _scalar_out()
    check(lib.ctk_mse_f32(a.p, b.p, _i64(a.size), out.p, None, _sh(stream)))
    return out


def mae(a, b, stream=None):
    out = _scalar_out()
    check(lib.ctk_mae_f32(a.p, b.p, _i64(a.size), out.p, None, _sh(stream)))
    return out


def mse_backward(p, t, g=None, stream=None):
    dp = DeviceArray(p.shape)
    check(lib.ctk_mse_backward_f32(p.p, t.p, g.p if g else None, dp.p, _i64(p.size), _sh(stream)))
    return dp


def mae_backward(p, t, g=None, stream=None):
    dp = DeviceArray(p.shape)
    check(lib.ctk_mae_backward_f32(p.p, t.p, g.p if g else None, dp.p, _i64(p.size), _sh(stream)))
    return dp


def _rc(a):
    return (1, a.shape[0]) if len(a.shape) == 1 else (a.shape[0], a.shape[1])


def softmax(x, out=None, stream=None):
    r, c = _rc(x)
    out = out or DeviceArray(x.shape)
    check(lib.ctk_softmax_rows_f32(x.p, out.p, _i64(r), _i64(c), _sh(stream)))
    return out


def softmax_backward(y, g, stream=None):
    r, c = _rc(y)
    dx = DeviceArray(y.shape)
    check(lib.ctk_softmax_backward_rows_f32(y.p, g.p, dx.p, _i64(r), _i64(c), _sh(stream)))
    return dx


def cross_entropy(logits, target, stream=None, bad_flag=None):
    """target: one-hot of logits' shape, or [rows] class indices stored as floats."""
    r, c = _rc(logits)
    out = _scalar_out()
    if target.shape == logits.shape:
        check(lib.ctk_ce_onehot_f32(logits.p, target.p, _i64(r), _i64(c), out.p, None, _sh(stream)))
    else:
        check(lib.ctk_ce_index_f32(logits.p, target.p, _i64(r), _i64(c), out.p, bad_flag.p if bad_flag else None, None, _sh(stream)))
    return out


def cross_entropy_backward(logits, onehot, g=None, stream=None):
    r, c = _rc(logits)
    d = DeviceArray(logits.shape)
    check(lib.ctk_ce_backward_f32(logits.p, onehot.p, g.p if g else None, d.p, _i64(r), _i64(c), _sh(stream)))
    return d


def cross_entropy_fused(logits, labels, stream=None, bad_flag=None):
    r, c = _rc(logits)
    out = _scalar_out()
    d = DeviceArray(logits.shape)
    check(lib.ctk_ce_fused_index_f32(logits.p, labels.p, _i64(r), _i64(c), out.p, d.p, bad_flag.p if bad_flag else None, None, _sh(stream)))
    return out, d


def matmul(a, b, ta=False, tb=False, mode=-1, out=None, workspace=None, stream=None):
    """a stored [m,k] (or [k,m] viewed through t() if ta); b stored [k,n] (or [n,k] if tb)."""
    mode = MODES.get(mode, mode)
    m, k = (a.shape[1], a.shape[0]) if ta else a.shape
    n = b.shape[0] if tb else b.shape[1]
    sa = (1, m) if ta else (k, 1)
    sb = (1, k) if tb else (n, 1)
    out = out or DeviceArray((m, n))
    check(lib.ctk_matmul_f32(a.p, b.p, out.p, _i64(m), _i64(n), _i64(k), _i64(sa[0]), _i64(sa[1]), _i64(sb[0]),
                             _i64(sb[1]), mode, workspace.p if workspace else None, _sh(stream)))
    return out


_fused_cache = {}


def matmul_fused(a, b, bias=None, relu=False, mask=None, want_split=False, ta=False, tb=False, stream=None, keep_split=False):
    """[relu](a.b + bias) * (mask > 0), the epilogue forms of the 3xTF32 product in one launch.
    Returns (c, hi, rest) when want_split (the split the epilogue wrote, decoded by _decode_split), else c.
    keep_split: write the split too, into buffers (and c) reused from call to call, and do not read it back."""
    m, k = (a.shape[1], a.shape[0]) if ta else a.shape
    n = b.shape[0] if tb else b.shape[1]
    sa = (1, m) if ta else (k, 1)
    sb = (1, k) if tb else (n, 1)
    split = None
    if keep_split:
        if (m, n) not in _fused_cache:
            _fused_cache[(m, n)] = (DeviceArray((m, n)), DeviceArray((int(lib.ctk_matmul_split_bytes(m, n)) // 4,)))
        out, split = _fused_cache[(m, n)]
    else:
        out = DeviceArray((m, n))
        if want_split:
            split = DeviceArray((int(lib.ctk_matmul_split_bytes(m, n)) // 4,))
    check(lib.ctk_matmul_3xtf32_fused_f32(a.p, b.p, out.p, _i64(m), _i64(n), _i64(k), _i64(sa[0]), _i64(sa[1]), _i64(sb[0]), _i64(sb[1]),
                                          None, None, None, None, bias.p if bias else None, int(bool(relu)), mask.p if mask else None,
                                          split.p if split else None, None, _sh(stream)))
    if not want_split:
        return out
    hi, rest = _decode_split(split, m, n, out)
    return out, hi, rest


def _decode_split(split, outer, inner, source):
    """The arrays of a split buffer as numpy: (hi, lo) as float32 [outer, inner] when the correction terms
    run on the TF32 path, (hi, bits) with bits a uint16 [2, outer, inner] array holding the bf16 patterns
    of h16 and l16 when they run on the bf16 path (see ctk_set_matmul_correction).  source: the contiguous
    [outer, inner] device array the split belongs to; where it serves as the split's hi part itself (see
    ctk_matmul_split_tag_for) hi is returned as the tensor core reads it: the low 13 mantissa bits cleared."""
    pitch = (inner + 7) // 8 * 8
    pad = (-split.ptr) % 256 // 4          # the library aligns the buffer to 256 bytes
    flat = split.numpy()
    if lib.ctk_matmul_split_tag_for(source.p, _i64(inner), _i64(inner)) >= 3:
        hi = (np.ascontiguousarray(source.numpy(), np.float32).reshape(outer, inner).view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    else:
        hi = flat[pad:pad + outer * pitch].reshape(outer, pitch)[:, :inner]
    if lib.ctk_get_matmul_correction() == 0:
        return hi, flat[pad + outer * pitch:pad + 2 * outer * pitch].reshape(outer, pitch)[:, :inner]
    u16 = flat.view(np.uint16)
    o = 2 * (pad + outer * pitch)
    h16 = u16[o:o + outer * pitch].reshape(outer, pitch)[:, :inner]
    l16 = u16[o + outer * pitch:o + 2 * outer * pitch].reshape(outer, pitch)[:, :inner]
    return hi, np.stack([h16, l16])


def sgd_update_split(p, g, lr, stream=None):
    """p -= g*lr on a 2-D array and the split of the new p in the same pass; returns it as _decode_split does."""
    outer, inner = p.shape
    split = DeviceArray((int(lib.ctk_matmul_split_bytes(inner, outer)) // 4,))
    check(lib.ctk_sgd_update_split_f32(p.p, g.p, _f(lr), _i64(outer), _i64(inner), _i64(inner), split.p, _sh(stream)))
    return _decode_split(split, outer, inner, p)


CMP = {"gt": 0, "lt": 1, "eq": 2, "ge": 3, "le": 4, "ne": 5}
CMP_TENSOR, CMP_SCALAR_RIGHT, CMP_SCALAR_LEFT = 0, 1, 2
DTYPES = {0: np.float32, 1: np.float64, 2: np.int32, 3: np.int64, 4: np.uint8}   # DType values; bool as bytes


def compare(cmp, a, other, scalar_left=False, stream=None):
    """a cmp other (other a DeviceArray or a float), or other cmp a when scalar_left; bytes 0/1."""
    out = DeviceArray(a.shape, np.uint8)
    if isinstance(other, DeviceArray):
        check(lib.ctk_compare_f32(CMP[cmp], CMP_TENSOR, a.p, other.p, _f(0.0), out.p, _i64(a.size), _sh(stream)))
    else:
        form = CMP_SCALAR_LEFT if scalar_left else CMP_SCALAR_RIGHT
        check(lib.ctk_compare_f32(CMP[cmp], form, a.p, None, _f(other), out.p, _i64(a.size), _sh(stream)))
    return out


def cast(a, dtype_code, stream=None):
    out = DeviceArray(a.shape, DTYPES[dtype_code])
    check(lib.ctk_cast_f32(int(dtype_code), a.p, out.p, _i64(a.size), _sh(stream)))
    return out


def fill_dtype(out, dtype_code, value, stream=None):
    check(lib.ctk_fill_dtype(int(dtype_code), out.p, ctypes.c_double(value), _i64(out.size), _sh(stream)))
    return out


def rand_uniform(shape, seed, offset=0, out=None, stream=None):
    out = out or DeviceArray(shape)
    check(lib.ctk_rand_uniform_f32(out.p, _i64(out.size), ctypes.c_uint64(seed), ctypes.c_uint64(offset), _sh(stream)))
    return out


def matmul_path(a, b, ta=False, tb=False, mode=-1):
    mode = MODES.get(mode, mode)
    m, k = (a.shape[1], a.shape[0]) if ta else a.shape
    n = b.shape[0] if tb else b.shape[1]
    sa = (1, m) if ta else (k, 1)
    sb = (1, k) if tb else (n, 1)
    return lib.ctk_matmul_path(a.p, b.p, _i64(m), _i64(n), _i64(k), _i64(sa[0]), _i64(sa[1]), _i64(sb[0]), _i64(sb[1]), mode)


def u8_to_f32(src_u8, divisor, out=None):
    """src_u8: a DeviceArray of dtype uint8; returns float(src) / divisor."""
    out = out or DeviceArray(src_u8.shape)
    check(lib.ctk_u8_to_f32(src_u8.p, _i64(src_u8.size), ctypes.c_float(divisor), out.p, None))
    return out


def argmax_rows(x, init=float("-inf")):
    r, c = _rc(x)
    out = DeviceArray((r,))
    check(lib.ctk_argmax_rows_f32(x.p, _i64(r), _i64(c), ctypes.c_float(init), out.p, None))
    return out


def colsum(x):
    r, c = _rc(x)
    out = DeviceArray((c,))
    check(lib.ctk_colsum_f32(x.p, _i64(r), _i64(c), out.p, None))
    return out


def count_matches(a, b):
    out = _scalar_out()
    check(lib.ctk_count_matches_f32(a.p, b.p, _i64(a.size), out.p, None, None))
    return out


def rowwise_status():
    s = ctypes.c_int()
    check(lib.ctk_rowwise_status(ctypes.byref(s)))
    return s.value


def set_matmul_pairing(pairing):
    """0: 256 x 256 tiles on CTA pairs where the shape allows (default); 1: single-CTA kernel only."""
    check(lib.ctk_set_matmul_pairing(int(pairing)))


def set_matmul_correction(bf16):
    """Correction terms of the fp32-accurate mode: 0 on the TF32 path (3xTF32), 1 on the bf16 path."""
    check(lib.ctk_set_matmul_correction(int(bf16)))


def set_matmul_tail_split(on):
    check(lib.ctk_set_matmul_tail_split(int(on)))


def matmul_status():
    s = ctypes.c_int()
    check(lib.ctk_matmul_status(ctypes.byref(s)))
    return s.value
