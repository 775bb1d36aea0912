"""The few CUDA runtime calls the host side needs, through ctypes on libcudart:
device memory for workspaces and for host-array callers, copies, and stream
synchronisation.  Nothing here computes anything; the kernels live in the C-ABI
library (`_native`).  Importing this module does not load the runtime; the
first call does, and raises if no CUDA runtime or device is there (there is no
CPU path).
"""

from __future__ import annotations

import ctypes
import ctypes.util
import glob
import os
import sys

_RT = None

MEMCPY_H2D, MEMCPY_D2H, MEMCPY_D2D = 1, 2, 3


def _candidates():
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"
    yield from sorted(glob.glob(os.path.join(home, "lib64", "libcudart.so*")), reverse=True)
    for entry in sys.path:  # the runtime that ships as a Python wheel
        yield from sorted(glob.glob(os.path.join(entry, "nvidia", "cuda_runtime", "lib", "libcudart.so*")))
    found = ctypes.util.find_library("cudart")
    if found:
        yield found


def runtime() -> ctypes.CDLL:
    """libcudart, loaded once."""
    global _RT
    if _RT is None:
        errors = []
        for path in _candidates():
            try:
                lib = ctypes.CDLL(path)
            except OSError as exc:
                errors.append(f"{path}: {exc}")
                continue
            lib.cudaGetErrorString.restype = ctypes.c_char_p
            _RT = lib
            break
        else:
            raise RuntimeError(
                "flywheel_tpu (B200 build) needs the CUDA runtime (libcudart); none"
                " could be loaded. " + "; ".join(errors))
    return _RT


def check(code: int, what: str) -> None:
    if code != 0:
        text = runtime().cudaGetErrorString(code).decode("utf-8", "replace")
        raise RuntimeError(f"{what}: {text} (CUDA error {code})")


def device_count() -> int:
    count = ctypes.c_int(0)
    code = runtime().cudaGetDeviceCount(ctypes.byref(count))
    return count.value if code == 0 else 0


def current_device() -> int:
    index = ctypes.c_int(0)
    check(runtime().cudaGetDevice(ctypes.byref(index)), "cudaGetDevice")
    return index.value


def set_device(index: int) -> None:
    check(runtime().cudaSetDevice(ctypes.c_int(index)), "cudaSetDevice")


def malloc(nbytes: int) -> int:
    ptr = ctypes.c_void_p()
    check(runtime().cudaMalloc(ctypes.byref(ptr), ctypes.c_size_t(max(int(nbytes), 1))), "cudaMalloc")
    return ptr.value


def free(ptr: int) -> None:
    if ptr and _RT is not None:
        _RT.cudaFree(ctypes.c_void_p(ptr))   # best effort: also called from __del__ at shutdown


def memset(ptr: int, value: int, nbytes: int, stream: int = 0) -> None:
    check(runtime().cudaMemsetAsync(ctypes.c_void_p(ptr), ctypes.c_int(value), ctypes.c_size_t(nbytes),
                                    ctypes.c_void_p(stream)), "cudaMemsetAsync")


def memcpy(dst: int, src: int, nbytes: int, kind: int, stream: int = 0) -> None:
    if nbytes:
        check(runtime().cudaMemcpyAsync(ctypes.c_void_p(dst), ctypes.c_void_p(src), ctypes.c_size_t(nbytes),
                                        ctypes.c_int(kind), ctypes.c_void_p(stream)), "cudaMemcpyAsync")


def synchronize(stream: int = 0) -> None:
    check(runtime().cudaStreamSynchronize(ctypes.c_void_p(stream)), "cudaStreamSynchronize")

