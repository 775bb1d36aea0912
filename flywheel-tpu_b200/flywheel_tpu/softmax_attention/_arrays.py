"""Array plumbing between callers and the C ABI.

The reference takes and returns JAX arrays.  The kernels only need device
pointers, so the entry points accept whatever array kind the caller has and
answer in kind.  Two back-ends share one code path in the entry points:

* torch - any operand that is a torch tensor selects it: CUDA tensors are used
  in place (nothing copied), CPU tensors are copied in and the results copied
  back, outputs are torch tensors on torch's current stream.  torch is imported
  only when such an operand shows up.
* raw - everything else: host NumPy arrays (with ml_dtypes for bf16 / fp8) are
  copied into `DeviceArray`s (cudaMalloc through ctypes on libcudart, see
  `_cuda`) and the results copied back to NumPy; objects that expose
  `__cuda_array_interface__` are used in place.  No torch anywhere.

Neither back-end computes any part of the attention: they move bytes and keep
metadata (lengths, cumulative offsets) in int32 arrays.
"""

from __future__ import annotations

import sys

import numpy as np

from flywheel_tpu.softmax_attention import _cuda

try:  # ml_dtypes gives NumPy its bf16 / fp8 types
    import ml_dtypes
    NP_BY_NAME = {
        "bfloat16": np.dtype(ml_dtypes.bfloat16),
        "float8_e4m3fn": np.dtype(ml_dtypes.float8_e4m3fn),
        "float8_e5m2": np.dtype(ml_dtypes.float8_e5m2),
    }
except ImportError:  # pragma: no cover
    NP_BY_NAME = {}

ITEMSIZE = {"bfloat16": 2, "float16": 2, "float8_e4m3fn": 1, "float8_e5m2": 1, "float32": 4,
            "float64": 8, "int32": 4, "int64": 8, "uint8": 1, "int16": 2, "int8": 1, "uint16": 2,
            "uint32": 4, "uint64": 8, "bool": 1}
# NumPy carriers for the bit patterns of the types torch.from_numpy rejects.
CARRIER = {"bfloat16": np.int16, "float8_e4m3fn": np.uint8, "float8_e5m2": np.uint8}
_TYPESTR = {"float32": "<f4", "float64": "<f8", "float16": "<f2", "int32": "<i4", "int64": "<i8",
            "uint8": "|u1", "int8": "|i1", "int16": "<i2", "bfloat16": "<V2", "float8_e4m3fn": "|V1",
            "float8_e5m2": "|V1"}


# ---------------------------------------------------------------- torch, on demand
def _torch():
    import torch
    return torch


def is_torch_tensor(x) -> bool:
    """True for torch tensors, without importing torch for callers that do not use it."""
    module = sys.modules.get("torch")
    return module is not None and isinstance(x, module.Tensor)


def _torch_dtype(name):
    torch = _torch()
    return {"bfloat16": torch.bfloat16, "float8_e4m3fn": torch.float8_e4m3fn,
            "float8_e5m2": torch.float8_e5m2, "float32": torch.float32, "float16": torch.float16,
            "float64": torch.float64, "int32": torch.int32, "int64": torch.int64,
            "uint8": torch.uint8, "int16": torch.int16}[name]


# ---------------------------------------------------------------- the raw back-end
class DType:
    """Element type of a DeviceArray: a name and a size."""

    def __init__(self, name):
        self.name, self.itemsize = name, ITEMSIZE[name]

    def __eq__(self, other):
        return dtype_name(other) == self.name

    def __hash__(self):
        return hash(self.name)

    def __repr__(self):
        return f"DType({self.name})"


class RawDevice:
    """A CUDA device of the raw back-end."""

    type = "cuda"

    def __init__(self, index):
        self.index = int(index)

    def __eq__(self, other):
        return isinstance(other, RawDevice) and other.index == self.index

    def __hash__(self):
        return hash(("raw", self.index))

    def __repr__(self):
        return f"RawDevice({self.index})"


class DeviceArray:
    """A contiguous array in device memory: pointer, shape, element type.  Owns
    its memory (freed with the last view) unless it wraps someone else's
    (`__cuda_array_interface__`).  `host` is the NumPy array it was uploaded
    from, when there is one: index arithmetic on metadata then needs no
    device-to-host copy."""

    is_cuda = True

    def __init__(self, ptr, shape, dtype, device_index, owner=None, host=None):
        self._ptr, self.shape = int(ptr), tuple(int(n) for n in shape)
        self.dtype = dtype if isinstance(dtype, DType) else DType(dtype)
        self.device = RawDevice(device_index)
        self._owner = owner       # the object that keeps the memory alive: a _Block or a foreign array
        self.host = host

    # -- what the entry points use of a tensor
    def data_ptr(self):
        return self._ptr

    @property
    def ndim(self):
        return len(self.shape)

    def numel(self):
        return int(np.prod(self.shape, dtype=np.int64))

    @property
    def nbytes(self):
        return self.numel() * self.dtype.itemsize

    def contiguous(self):
        return self

    def is_contiguous(self):
        return True

    def reshape(self, *shape):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        known = int(np.prod([n for n in shape if n != -1], dtype=np.int64))
        shape = tuple(self.numel() // max(known, 1) if n == -1 else int(n) for n in shape)
        if int(np.prod(shape, dtype=np.int64)) != self.numel():
            raise ValueError(f"cannot reshape {self.shape} to {shape}")
        host = None if self.host is None else self.host.reshape(shape)
        return DeviceArray(self._ptr, shape, self.dtype, self.device.index, self._owner, host)

    view = reshape

    def __getitem__(self, key):
        """x[first:] and x[first:last] along the leading axis: views."""
        if not isinstance(key, slice) or key.step not in (None, 1):
            raise TypeError("a DeviceArray is sliced along its leading axis only")
        first, last, _ = key.indices(self.shape[0])
        row = self.numel() // max(self.shape[0], 1) * self.dtype.itemsize
        host = None if self.host is None else self.host[first:last]
        return DeviceArray(self._ptr + first * row, (max(last - first, 0), *self.shape[1:]), self.dtype,
                           self.device.index, self._owner, host)

    def numpy(self):
        """A host copy (synchronises the default stream)."""
        name = self.dtype.name
        out = np.empty(self.shape, NP_BY_NAME.get(name) or np.dtype(name))
        _cuda.set_device(self.device.index)
        _cuda.memcpy(out.ctypes.data, self._ptr, self.nbytes, _cuda.MEMCPY_D2H)
        _cuda.synchronize()
        return out

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": _TYPESTR[self.dtype.name], "data": (self._ptr, False),
                "version": 3, "strides": None}


class _Block:
    """cudaMalloc'ed memory, freed when the last DeviceArray over it goes."""

    def __init__(self, nbytes, device_index):
        _cuda.set_device(device_index)
        self.ptr = _cuda.malloc(nbytes)

    def __del__(self):
        _cuda.free(self.ptr)


def _raw_empty(shape, name, device_index, host=None):
    nbytes = int(np.prod(shape, dtype=np.int64)) * ITEMSIZE[name]
    block = _Block(nbytes, device_index)
    return DeviceArray(block.ptr, shape, name, device_index, block, host)


def _raw_upload(array, device_index, name=None):
    array = np.ascontiguousarray(array)
    if name is not None and dtype_name(array.dtype) != name:
        array = array.astype(NP_BY_NAME.get(name) or np.dtype(name))
    out = _raw_empty(array.shape, dtype_name(array.dtype), device_index, host=array)
    _cuda.memcpy(out.data_ptr(), array.ctypes.data, array.nbytes, _cuda.MEMCPY_H2D)
    return out


def _from_cuda_array_interface(x):
    info = x.__cuda_array_interface__
    if info.get("strides") not in (None,):
        expected, stride = [], 1
        for n in reversed(info["shape"]):
            expected.insert(0, stride * np.dtype(info["typestr"]).itemsize)
            stride *= n
        if tuple(info["strides"]) != tuple(expected):
            raise ValueError("device arrays must be contiguous.")
    name = dtype_name(x.dtype) if hasattr(x, "dtype") else np.dtype(info["typestr"]).name
    return DeviceArray(info["data"][0], info["shape"], name, _cuda.current_device(), owner=x)


# ---------------------------------------------------------------- queries
def dtype(x):
    return x.dtype


def shape(x):
    return tuple(x.shape)


def dtype_name(dt) -> str:
    if isinstance(dt, DType):
        return dt.name
    if type(dt).__module__.split(".")[0] == "torch":
        return str(dt).replace("torch.", "")
    return np.dtype(dt).name if not hasattr(dt, "name") else str(dt.name)


def itemsize(dt) -> int:
    name = dtype_name(dt)
    return ITEMSIZE[name] if name in ITEMSIZE else np.dtype(dt).itemsize


def is_floating(x) -> bool:
    name = dtype_name(x.dtype)
    return name.startswith("float") or name == "bfloat16"


def is_integer(x) -> bool:
    name = dtype_name(x.dtype)
    return name.startswith("int") or name.startswith("uint")


def is_host(x) -> bool:
    if is_torch_tensor(x):
        return not x.is_cuda
    return isinstance(x, (np.ndarray, np.generic, int, float))


def is_device_resident(x) -> bool:
    """The caller's own device memory: results that alias it are returned as is."""
    if is_torch_tensor(x):
        return x.is_cuda
    return isinstance(x, DeviceArray) or hasattr(x, "__cuda_array_interface__")


# ---------------------------------------------------------------- devices and streams
def pick_device(*operands):
    """The device the call runs on, which also picks the back-end: the CUDA
    device of the first device-resident torch operand (else torch's current one)
    when any operand is a torch tensor, otherwise a RawDevice.  Raises where no
    CUDA device exists: there is no CPU path."""
    if any(is_torch_tensor(x) for x in operands):
        torch = _torch()
        if not torch.cuda.is_available():
            raise RuntimeError("flywheel_tpu (B200 build) needs a CUDA device; there is no CPU path.")
        for x in operands:
            if is_torch_tensor(x) and x.is_cuda:
                return x.device
        return torch.device("cuda", torch.cuda.current_device())
    if _cuda.device_count() == 0:
        raise RuntimeError("flywheel_tpu (B200 build) needs a CUDA device; there is no CPU path.")
    for x in operands:
        if isinstance(x, DeviceArray):
            return x.device
    return RawDevice(_cuda.current_device())


def is_raw(device) -> bool:
    return isinstance(device, RawDevice)


def current_stream(device) -> int:
    """The stream launches go to: torch's current stream, or the default stream."""
    if is_raw(device):
        _cuda.set_device(device.index)
        return 0
    return _torch().cuda.current_stream(device).cuda_stream


# ---------------------------------------------------------------- moving data
def to_device(x, device, dtype=None):
    """x as a device array of the call's back-end; dtype (a name) casts integer /
    float metadata (never the cache or q)."""
    if is_raw(device):
        if isinstance(x, DeviceArray):
            if dtype is not None and x.dtype.name != dtype:
                return _raw_upload(x.numpy() if x.host is None else x.host, device.index, dtype)
            return x
        if hasattr(x, "__cuda_array_interface__"):
            wrapped = _from_cuda_array_interface(x)
            if dtype is not None and wrapped.dtype.name != dtype:
                return _raw_upload(wrapped.numpy(), device.index, dtype)
            return wrapped
        if isinstance(x, (np.ndarray, np.generic, int, float, list, tuple)):
            return _raw_upload(np.asarray(x), device.index, dtype)
        raise TypeError(f"cannot take a {type(x).__name__} without torch; pass NumPy arrays or arrays "
                        "with __cuda_array_interface__.")
    torch = _torch()
    if isinstance(x, torch.Tensor):
        tensor = x
    elif isinstance(x, (np.ndarray, np.generic)):
        arr = np.asarray(x)
        name = dtype_name(arr.dtype)
        if name in CARRIER:
            carrier = np.ascontiguousarray(arr).view(CARRIER[name])
            tensor = torch.from_numpy(carrier).view(_torch_dtype(name))
        else:
            tensor = torch.from_numpy(np.ascontiguousarray(arr))
    elif isinstance(x, (int, float)):
        tensor = torch.tensor(x)
    elif isinstance(x, DeviceArray):
        tensor = torch.from_numpy(x.numpy().view(CARRIER.get(x.dtype.name, x.numpy().dtype)))
        if x.dtype.name in CARRIER:
            tensor = tensor.view(_torch_dtype(x.dtype.name))
    elif hasattr(x, "__dlpack__"):
        tensor = torch.from_dlpack(x)
    else:
        tensor = torch.as_tensor(x)
    if dtype is not None and tensor.dtype != _torch_dtype(dtype):
        tensor = tensor.to(_torch_dtype(dtype))
    if not tensor.is_cuda or tensor.device != device:
        if not tensor.is_cuda and not tensor.is_pinned() and tensor.numel() > 0:
            tensor = tensor.contiguous()
        tensor = tensor.to(device, non_blocking=True)
    return tensor


def to_host_numpy(array) -> np.ndarray:
    if isinstance(array, DeviceArray):
        return array.numpy()
    name = dtype_name(array.dtype)
    host = array.detach().cpu()
    if name in CARRIER:
        torch = _torch()
        carrier_torch = torch.int16 if name == "bfloat16" else torch.uint8
        return host.view(carrier_torch).numpy().view(NP_BY_NAME[name])
    return host.numpy()


def like(result, template):
    """`result` (a device array of the call's back-end) in the array kind of `template`."""
    if isinstance(result, DeviceArray):
        if isinstance(template, (np.ndarray, np.generic)):
            return result.numpy()
        return result
    if is_torch_tensor(template):
        if template.is_cuda:
            return result
        torch = _torch()
        if template.is_pinned():
            # a pinned caller gets a pinned result: one DMA, no staging copy
            host = torch.empty(result.shape, dtype=result.dtype, pin_memory=True)
            host.copy_(result, non_blocking=True)
            torch.cuda.current_stream(result.device).synchronize()
            return host
        return result.cpu()
    if isinstance(template, (np.ndarray, np.generic)):
        return to_host_numpy(result)
    if hasattr(template, "__dlpack__"):
        try:  # a JAX caller gets JAX arrays back
            import jax.dlpack  # type: ignore
            return jax.dlpack.from_dlpack(result)
        except ImportError:
            return result
    return result


def data_ptr(array) -> int:
    return 0 if array is None else array.data_ptr()


# ---------------------------------------------------------------- allocation and metadata arithmetic
def empty(shape, name, device):
    if is_raw(device):
        return _raw_empty(tuple(shape), name, device.index)
    return _torch().empty(tuple(shape), dtype=_torch_dtype(name), device=device)


def empty_like(array):
    if isinstance(array, DeviceArray):
        return _raw_empty(array.shape, array.dtype.name, array.device.index)
    return _torch().empty_like(array)


def _host_ints(array) -> np.ndarray:
    """int metadata of the raw back-end on the host: its upload source when there
    is one, else a device-to-host copy (synchronises)."""
    return np.asarray(array.host if array.host is not None else array.numpy())


def int32_array(values, device):
    """A small int32 device array from host values."""
    if is_raw(device):
        return _raw_upload(np.asarray(values, np.int32), device.index)
    return _torch().tensor(list(values), dtype=_torch().int32, device=device)


def arange_scaled(count, scale, device, first=0):
    """int32 [first, first + 1, ...) * scale, `count` entries."""
    if is_raw(device):
        return _raw_upload((np.arange(first, first + count, dtype=np.int32) * scale).astype(np.int32), device.index)
    torch = _torch()
    return torch.arange(first, first + count, dtype=torch.int32, device=device) * scale


def broadcast_scalar(array, count, device):
    """A 0-d / 1-element int array repeated `count` times."""
    if is_raw(device):
        return _raw_upload(np.broadcast_to(_host_ints(array).reshape(-1)[:1], (count,)).astype(np.int32), device.index)
    return array.reshape(1).expand(count).contiguous()


def add_token_counts(lengths, cu):
    """lengths + diff(cu): each request's KV length after its new tokens."""
    if isinstance(lengths, DeviceArray):
        counts = np.diff(_host_ints(cu)).astype(np.int32)
        return _raw_upload(_host_ints(lengths).astype(np.int32) + counts, lengths.device.index)
    return (lengths + (cu[1:] - cu[:-1])).contiguous()


def rebase_count(active, first, rows):
    """clamp(active - first, 0, rows) as a one-element int32 device array."""
    if isinstance(active, DeviceArray):
        value = int(np.clip(int(_host_ints(active).reshape(-1)[0]) - first, 0, rows))
        return _raw_upload(np.asarray([value], np.int32), active.device.index)
    return (active - first).clamp_(0, rows)


def heads_first_to_batch_first(lse, nheads, batch, seqlen_q):
    """(nheads, batch * seqlen_q) f32 -> (batch, nheads, seqlen_q)."""
    if isinstance(lse, DeviceArray):
        host = lse.numpy().reshape(nheads, batch, seqlen_q).transpose(1, 0, 2)
        return _raw_upload(np.ascontiguousarray(host), lse.device.index)
    return lse.reshape(nheads, batch, seqlen_q).permute(1, 0, 2).contiguous()
