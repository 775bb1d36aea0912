"""Array plumbing between callers and the C ABI.

The reference takes and returns JAX arrays.  Here the device memory and the
streams come from PyTorch, so the entry points accept
  * CUDA torch tensors (used in place, nothing copied),
  * host arrays: NumPy (with ml_dtypes for bf16 / fp8) or CPU torch tensors,
    copied to the device for the call and the results copied back,
  * anything that speaks DLPack on a CUDA device (a JAX array, for one),
and return results of the same kind as ``q``.  Torch is plumbing only: no torch
operator computes any part of the attention.
"""

from __future__ import annotations

import numpy as np
import torch

try:  # ml_dtypes gives NumPy its bf16 / fp8 types
    import ml_dtypes
    NP_BY_NAME = {
        "bfloat16": np.dtype(ml_dtypes.bfloat16),
        "float8_e4m3fn": np.dtype(ml_dtypes.float8_e4m3fn),
        "float8_e5m2": np.dtype(ml_dtypes.float8_e5m2),
    }
except ImportError:  # pragma: no cover
    NP_BY_NAME = {}

TORCH_BY_NAME = {
    "bfloat16": torch.bfloat16,
    "float8_e4m3fn": torch.float8_e4m3fn,
    "float8_e5m2": torch.float8_e5m2,
    "float32": torch.float32,
    "float16": torch.float16,
    "float64": torch.float64,
    "int32": torch.int32,
    "int64": torch.int64,
}
NAME_BY_TORCH = {v: k for k, v in TORCH_BY_NAME.items()}
# NumPy carriers for the bit patterns of the types torch.from_numpy rejects.
CARRIER = {"bfloat16": np.int16, "float8_e4m3fn": np.uint8, "float8_e5m2": np.uint8}


def dtype(x):
    return x.dtype


def shape(x):
    return tuple(x.shape)


def dtype_name(dt) -> str:
    if isinstance(dt, torch.dtype):
        return NAME_BY_TORCH.get(dt, str(dt).replace("torch.", ""))
    return np.dtype(dt).name if not hasattr(dt, "name") else str(dt.name)


def itemsize(dt) -> int:
    if isinstance(dt, torch.dtype):
        return torch.empty((), dtype=dt).element_size()
    return np.dtype(dt).itemsize


def is_floating(x) -> bool:
    name = dtype_name(x.dtype)
    return name.startswith("float") or name == "bfloat16"


def is_integer(x) -> bool:
    name = dtype_name(x.dtype)
    return name.startswith("int") or name.startswith("uint")


def is_host(x) -> bool:
    if isinstance(x, torch.Tensor):
        return not x.is_cuda
    if isinstance(x, (np.ndarray, np.generic, int, float)):
        return True
    return False


def pick_device(*operands) -> torch.device:
    """The CUDA device of the first device-resident operand, else the current
    one.  Raises where no CUDA device exists: there is no CPU path."""
    if not torch.cuda.is_available():
        raise RuntimeError(
            "flywheel_tpu (B200 build) needs a CUDA device; there is no CPU"
            " path.")
    for x in operands:
        if isinstance(x, torch.Tensor) and x.is_cuda:
            return x.device
    return torch.device("cuda", torch.cuda.current_device())


def to_device(x, device, dtype=None) -> torch.Tensor:
    """x as a torch tensor on `device`; dtype (a name) casts integer / float
    metadata (never the cache or q)."""
    if isinstance(x, torch.Tensor):
        tensor = x
    elif isinstance(x, np.ndarray) or isinstance(x, np.generic):
        arr = np.asarray(x)
        name = dtype_name(arr.dtype)
        if name in CARRIER:
            carrier = np.ascontiguousarray(arr).view(CARRIER[name])
            tensor = torch.from_numpy(carrier).view(TORCH_BY_NAME[name])
        else:
            tensor = torch.from_numpy(np.ascontiguousarray(arr))
    elif isinstance(x, (int, float)):
        tensor = torch.tensor(x)
    elif hasattr(x, "__dlpack__"):
        tensor = torch.from_dlpack(x)
    else:
        tensor = torch.as_tensor(x)
    if dtype is not None and tensor.dtype != TORCH_BY_NAME[dtype]:
        tensor = tensor.to(TORCH_BY_NAME[dtype])
    if not tensor.is_cuda or tensor.device != device:
        if not tensor.is_cuda and not tensor.is_pinned() and tensor.numel() > 0:
            tensor = tensor.contiguous()
        tensor = tensor.to(device, non_blocking=True)
    return tensor


def to_host_numpy(tensor: torch.Tensor) -> np.ndarray:
    name = dtype_name(tensor.dtype)
    host = tensor.detach().cpu()
    if name in CARRIER:
        carrier_torch = torch.int16 if name == "bfloat16" else torch.uint8
        return host.view(carrier_torch).numpy().view(NP_BY_NAME[name])
    return host.numpy()


def like(result: torch.Tensor, template):
    """`result` (a CUDA tensor) in the array kind of `template`."""
    if isinstance(template, torch.Tensor):
        if template.is_cuda:
            return result
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


def data_ptr(tensor) -> int:
    return 0 if tensor is None else tensor.data_ptr()
