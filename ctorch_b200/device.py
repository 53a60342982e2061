"""Device buffers, streams and events on top of the C ABI (no torch, no numpy compute)."""
import ctypes

import numpy as np

from ._lib import lib, check

_vp = ctypes.c_void_p


class Stream:
    def __init__(self):
        h = _vp()
        check(lib.ctk_stream_create(ctypes.byref(h)))
        self.handle = h

    def sync(self):
        check(lib.ctk_stream_sync(self.handle))

    def wait(self, event):
        check(lib.ctk_stream_wait_event(self.handle, event.handle))

    def __del__(self):
        try:
            lib.ctk_stream_destroy(self.handle)
        except Exception:
            pass


def _sh(stream):
    return stream.handle if isinstance(stream, Stream) else _vp(stream) if stream else None


class Event:
    def __init__(self):
        h = _vp()
        check(lib.ctk_event_create(ctypes.byref(h)))
        self.handle = h

    def record(self, stream=None):
        check(lib.ctk_event_record(self.handle, _sh(stream)))
        return self

    def sync(self):
        check(lib.ctk_event_sync(self.handle))

    def elapsed_ms(self, later):
        ms = ctypes.c_float()
        check(lib.ctk_event_elapsed_ms(self.handle, later.handle, ctypes.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            lib.ctk_event_destroy(self.handle)
        except Exception:
            pass


class DeviceArray:
    """An fp32 (or raw byte) buffer in device memory, owned unless it is a view."""

    def __init__(self, shape, dtype=np.float32, _ptr=None, _owner=None):
        self.shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        self.dtype = np.dtype(dtype)
        self.size = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        self.nbytes = self.size * self.dtype.itemsize
        self._owner = _owner
        if _ptr is None:
            p = _vp()
            check(lib.ctk_malloc(ctypes.byref(p), ctypes.c_size_t(self.nbytes)))
            self.ptr = p.value or 0
            self._owned = True
        else:
            self.ptr = _ptr
            self._owned = False

    @property
    def p(self):
        return _vp(self.ptr)

    def view(self, offset_elems, shape):
        """A window into this buffer (used to build unaligned / offset operands in tests)."""
        return DeviceArray(shape, self.dtype, _ptr=self.ptr + offset_elems * self.dtype.itemsize, _owner=self)

    def reshape(self, *shape):
        shape = shape[0] if len(shape) == 1 and isinstance(shape[0], (tuple, list)) else shape
        return DeviceArray(shape, self.dtype, _ptr=self.ptr, _owner=self)

    def copy_from_host(self, arr, stream=None):
        arr = np.require(arr, dtype=self.dtype, requirements="C")
        assert arr.size == self.size, (arr.shape, self.shape)
        check(lib.ctk_memcpy_h2d(self.p, arr.ctypes.data_as(_vp), ctypes.c_size_t(self.nbytes), _sh(stream)))
        if stream is None:
            synchronize()
        return self

    def numpy(self, stream=None):
        out = np.empty(self.shape, self.dtype)
        check(lib.ctk_memcpy_d2h(out.ctypes.data_as(_vp), self.p, ctypes.c_size_t(self.nbytes), _sh(stream)))
        if stream is None:
            synchronize()
        else:
            stream.sync()
        return out

    def fill_bytes(self, byte=0, stream=None):
        check(lib.ctk_memset(self.p, byte, ctypes.c_size_t(self.nbytes), _sh(stream)))
        return self

    def free(self):
        if self._owned and self.ptr:
            lib.ctk_free(self.p)
            self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def to_device(arr, dtype=np.float32):
    arr = np.require(arr, dtype=dtype, requirements="C")
    return DeviceArray(arr.shape, dtype).copy_from_host(arr)


def empty(shape, dtype=np.float32):
    return DeviceArray(shape, dtype)


def zeros(shape, dtype=np.float32):
    d = DeviceArray(shape, dtype)
    d.fill_bytes(0)
    return d


def synchronize():
    check(lib.ctk_device_sync())


def launch_count():
    return int(lib.ctk_launch_count())


class PinnedArray:
    """Page-locked host memory exposed as a numpy array (H2D/D2H staging)."""

    def __init__(self, shape, dtype=np.float32):
        self.shape = tuple(shape) if isinstance(shape, (tuple, list)) else (shape,)
        self.dtype = np.dtype(dtype)
        n = int(np.prod(self.shape, dtype=np.int64))
        self.nbytes = n * self.dtype.itemsize
        p = _vp()
        check(lib.ctk_malloc_host(ctypes.byref(p), ctypes.c_size_t(self.nbytes)))
        self.ptr = p.value
        buf = (ctypes.c_char * self.nbytes).from_address(self.ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype).reshape(self.shape)

    def free(self):
        if self.ptr:
            self.array = None
            lib.ctk_free_host(_vp(self.ptr))
            self.ptr = 0
