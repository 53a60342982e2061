"""ctorch_b200: B200-native CUDA backend for CTorch's reserved DeviceType::kCUDA slot.

The product is the C-ABI shared library ``lib/libctorch_b200.so`` (hand-written sm_100a kernels,
see ``include/ctorch_b200.h``) and the C++ front end compiled into it.  This Python package is a
thin ctypes face used by the tests and the benchmark; it has no compute of its own and no CPU
fallback: loading fails loudly if the library has not been built.
"""
from ._lib import lib, load, LIB_PATH, CtkError, check  # noqa: F401
from .device import DeviceArray, Stream, Event, to_device, empty, zeros, synchronize, launch_count  # noqa: F401
from . import ops  # noqa: F401
from . import frontend  # noqa: F401

__all__ = ["lib", "load", "LIB_PATH", "CtkError", "check", "DeviceArray", "Stream", "Event", "to_device", "empty",
           "zeros", "synchronize", "launch_count", "ops", "frontend"]
