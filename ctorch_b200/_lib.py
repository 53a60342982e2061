"""ctypes loader for libctorch_b200.so.  No fallback of any kind."""
import ctypes
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libctorch_b200.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
HEADERS = [os.path.join(INCLUDE, "ctorch_b200.h"), os.path.join(INCLUDE, "ctorch_b200_frontend.h")]

_lib = None


class CtkError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"ctk status {code}: {msg}")
        self.code = code


def declared_symbols(headers=None):
    """Names of every function the public headers declare."""
    names = set()
    for header in headers or HEADERS:
        text = open(header).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names.update(re.findall(r"\b(ct[kh]_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def load():
    """Loads the library; raises if it is missing (build it with `python -m ctorch_b200.build`)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: the CUDA extension is not built. Run `python -m ctorch_b200.build` "
            "(needs nvcc). There is no CPU fallback.")
    L = ctypes.CDLL(LIB_PATH, mode=ctypes.RTLD_GLOBAL)
    L.ctk_last_error.restype = ctypes.c_char_p
    L.ctk_launch_count.restype = ctypes.c_uint64
    L.ctk_reduce_scratch_bytes.restype = ctypes.c_size_t
    L.ctk_matmul_workspace_bytes.restype = ctypes.c_size_t
    L.ctk_matmul_workspace_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
    L.ctk_matmul_split_bytes.restype = ctypes.c_size_t
    L.ctk_matmul_split_bytes.argtypes = [ctypes.c_int64, ctypes.c_int64]
    L.cth_last_error.restype = ctypes.c_char_p
    L.cth_error_count.restype = ctypes.c_uint64
    _lib = L
    return L


class _Lazy:
    def __getattr__(self, name):
        return getattr(load(), name)


lib = _Lazy()


def check(status):
    if status != 0:
        raise CtkError(status, load().ctk_last_error().decode("utf-8", "replace"))
