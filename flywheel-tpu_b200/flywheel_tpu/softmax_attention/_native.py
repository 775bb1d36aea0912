"""ctypes binding of the C ABI in include/flywheel_b200.h.

The shared library is built in-tree (build.py) and must be present: importing
the entry points without it raises, there is no fallback.
"""

from __future__ import annotations

import ctypes
import os
import pathlib

from flywheel_tpu.softmax_attention import _cuda

PACKAGE_ROOT = pathlib.Path(__file__).resolve().parents[2]
LIBRARY_PATH = PACKAGE_ROOT / "lib" / "libflywheel_b200.so"

FW_OK = 0
ERRORS = {
    -1: ValueError,            # FW_ERR_BAD_SHAPE
    -2: NotImplementedError,   # FW_ERR_BAD_DTYPE
    -3: NotImplementedError,   # FW_ERR_UNSUPPORTED
    -4: RuntimeError,          # FW_ERR_LAUNCH
    -5: TimeoutError,          # FW_ERR_TIMEOUT
    -6: ValueError,            # FW_ERR_WORKSPACE
}
DTYPE_CODE = {"bfloat16": 0, "float8_e4m3fn": 1, "float8_e5m2": 2}
ROUTE_CODE = {"auto": 0, "tcgen05": 1, "splitkv": 2}   # FwPrefillArgs.route

c_ptr = ctypes.c_void_p
i32, i64, u64, f32 = ctypes.c_int32, ctypes.c_int64, ctypes.c_uint64, ctypes.c_float


class FwDecodeArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_ptr), ("out", c_ptr), ("lse", c_ptr), ("kv_cache", c_ptr),
        ("v_cache", c_ptr), ("k_new", c_ptr), ("v_new", c_ptr),
        ("cache_seqlens", c_ptr), ("block_table", c_ptr),
        ("cache_batch_idx", c_ptr), ("num_active", c_ptr),
        ("k_descale", c_ptr), ("v_descale", c_ptr), ("sinks", c_ptr),
        ("partial_out", c_ptr), ("partial_lse", c_ptr), ("workspace", c_ptr),
        ("workspace_bytes", u64), ("num_pages", i64), ("page_size", i32),
        ("pages_per_seq", i32), ("batch", i32), ("seqlen_q", i32),
        ("nheads", i32), ("nheads_k", i32), ("head_dim", i32),
        ("kv_dtype", i32), ("causal", i32), ("window_left", i32),
        ("softmax_scale", f32), ("softcap", f32), ("num_ctas", i32),
        ("append_enable", c_ptr),
    ]


class FwAppendArgs(ctypes.Structure):
    _fields_ = [
        ("kv_cache", c_ptr), ("k_new", c_ptr), ("v_new", c_ptr),
        ("cu_seqlens_q", c_ptr), ("cache_seqlens", c_ptr),
        ("block_table", c_ptr), ("num_active", c_ptr), ("num_pages", i64),
        ("page_size", i32), ("pages_per_seq", i32), ("batch", i32),
        ("total_tokens", i32), ("nheads_k", i32), ("head_dim", i32),
        ("kv_dtype", i32),
    ]


class FwWritePagesArgs(ctypes.Structure):
    _fields_ = [
        ("kv_cache", c_ptr), ("k_new", c_ptr), ("v_new", c_ptr), ("slices", c_ptr),
        ("num_slices", c_ptr), ("num_pages", i64), ("page_size", i32),
        ("num_columns", i32), ("total_tokens", i32), ("nheads_k", i32),
        ("head_dim", i32), ("kv_dtype", i32),
    ]


class FwPrefillArgs(ctypes.Structure):
    _fields_ = [
        ("q", c_ptr), ("out", c_ptr), ("lse", c_ptr), ("kv_cache", c_ptr),
        ("cu_seqlens_q", c_ptr), ("seqused_k", c_ptr), ("block_table", c_ptr),
        ("num_active", c_ptr), ("k_descale", c_ptr), ("v_descale", c_ptr),
        ("sinks", c_ptr), ("workspace", c_ptr), ("workspace_bytes", u64),
        ("num_pages", i64), ("page_size", i32), ("pages_per_seq", i32),
        ("batch", i32), ("total_q", i32), ("max_seqlen_q", i32),
        ("nheads", i32), ("nheads_k", i32), ("head_dim", i32),
        ("kv_dtype", i32), ("causal", i32), ("window_left", i32),
        ("softmax_scale", f32), ("softcap", f32), ("token_major", i32),
        ("rotary_cos", c_ptr), ("rotary_sin", c_ptr), ("rotary_len", i32),
        ("rotary_interleaved", i32), ("rotary_bf16", i32),
        ("v_packed", c_ptr), ("cu_seqlens_k", c_ptr), ("total_k", i32),
        ("kv_token_major", i32), ("rotary_k", i32), ("sink_period", i32),
        ("window_right", i32), ("kv_request_stride", i32), ("route", i32),
        ("first_request", c_ptr),
    ]


class FwExtendArgs(ctypes.Structure):
    _fields_ = [
        ("attn", FwPrefillArgs), ("num_decode", c_ptr), ("k_new", c_ptr),
        ("v_new", c_ptr), ("slices", c_ptr), ("num_slices", c_ptr),
        ("num_columns", i32), ("total_tokens", i32),
    ]


class FwCombineArgs(ctypes.Structure):
    _fields_ = [
        ("partial_out", c_ptr), ("partial_lse", c_ptr), ("sinks", c_ptr),
        ("out", c_ptr), ("lse", c_ptr), ("parts", i32), ("rows", i32),
        ("nheads", i32), ("head_dim", i32), ("lse_head_stride", i32),
        ("lse_token_stride", i32), ("part_stride_out", i64),
        ("part_stride_lse", i64),
    ]


class FwExchangeArgs(ctypes.Structure):
    _fields_ = [
        ("peer_buffers", c_ptr), ("state_out", c_ptr), ("state_lse", c_ptr),
        ("sinks", c_ptr), ("out", c_ptr), ("lse", c_ptr), ("status", c_ptr),
        ("world", i32), ("rank", i32), ("rows", i32), ("nheads", i32),
        ("head_dim", i32), ("lse_head_stride", i32), ("lse_token_stride", i32),
        ("global_len", c_ptr), ("local_len", c_ptr), ("append_enable", c_ptr),
        ("page_size", i32), ("advance", i32),
    ]


class FwShardStepArgs(ctypes.Structure):
    _fields_ = [
        ("global_len", c_ptr), ("local_len", c_ptr), ("append_enable", c_ptr),
        ("page_size", i32), ("world", i32), ("rank", i32), ("advance", i32),
    ]


class FwShardedDecodeArgs(ctypes.Structure):
    _fields_ = [
        ("decode", FwDecodeArgs), ("peer_buffers", c_ptr), ("world", i32), ("rank", i32),
        ("global_len", c_ptr), ("local_len", c_ptr), ("append_enable", c_ptr),
        ("advance", i32), ("deliver_only", i32),
    ]


EXPORTS = {
    "fw_decode_workspace_bytes": (u64, [ctypes.POINTER(FwDecodeArgs)]),
    "fw_decode_kvcache": (ctypes.c_int, [ctypes.POINTER(FwDecodeArgs), c_ptr]),
    "fw_decode_kvcache_static": (ctypes.c_int, [ctypes.POINTER(FwDecodeArgs), c_ptr]),
    "fw_append_ragged": (ctypes.c_int, [ctypes.POINTER(FwAppendArgs), c_ptr]),
    "fw_write_kv_pages": (ctypes.c_int, [ctypes.POINTER(FwWritePagesArgs), c_ptr]),
    "fw_prefill_workspace_bytes": (u64, [ctypes.POINTER(FwPrefillArgs)]),
    "fw_prefill_paged": (ctypes.c_int, [ctypes.POINTER(FwPrefillArgs), c_ptr]),
    "fw_extend_workspace_bytes": (u64, [ctypes.POINTER(FwExtendArgs)]),
    "fw_extend_mixed": (ctypes.c_int, [ctypes.POINTER(FwExtendArgs), c_ptr]),
    "fw_attention_packed_workspace_bytes": (u64, [ctypes.POINTER(FwPrefillArgs)]),
    "fw_attention_packed": (ctypes.c_int, [ctypes.POINTER(FwPrefillArgs), c_ptr]),
    "fw_lse_combine": (ctypes.c_int, [ctypes.POINTER(FwCombineArgs), c_ptr]),
    "fw_exchange_buffer_bytes": (u64, [i32, i32, i32]),
    "fw_peer_alloc": (ctypes.c_int, [u64, ctypes.POINTER(c_ptr), c_ptr]),
    "fw_peer_open": (ctypes.c_int, [c_ptr, ctypes.POINTER(c_ptr)]),
    "fw_peer_close": (ctypes.c_int, [c_ptr]),
    "fw_peer_free": (ctypes.c_int, [c_ptr]),
    "fw_state_exchange_merge": (ctypes.c_int, [ctypes.POINTER(FwExchangeArgs), c_ptr]),
    "fw_shard_step": (ctypes.c_int, [ctypes.POINTER(FwShardStepArgs), c_ptr]),
    "fw_sharded_decode_step": (ctypes.c_int, [ctypes.POINTER(FwShardedDecodeArgs), c_ptr]),
    "fw_selftest_wait_timeout": (ctypes.c_int, [c_ptr, ctypes.c_uint32, c_ptr]),
    "fw_read_status": (ctypes.c_int, [c_ptr, c_ptr, ctypes.POINTER(i32)]),
    "fw_read_status_static": (ctypes.c_int, [c_ptr, ctypes.POINTER(i32)]),
    "fw_last_error": (ctypes.c_char_p, []),
    "fw_version": (ctypes.c_int, []),
}

_LIB = None


def library() -> ctypes.CDLL:
    """The loaded shared library; raises if it has not been built."""
    global _LIB
    if _LIB is None:
        path = pathlib.Path(os.environ.get("FLYWHEEL_B200_LIBRARY", LIBRARY_PATH))
        if not path.exists():
            raise ImportError(
                f"{path} is missing: build the CUDA library first"
                " (python flywheel-tpu_b200/build.py). There is no fallback"
                " path.")
        lib = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _LIB = lib
    return _LIB


def last_error() -> str:
    return library().fw_last_error().decode("utf-8", "replace")


def check(code: int) -> None:
    if code != FW_OK:
        raise ERRORS.get(code, RuntimeError)(last_error())


def current_stream(device) -> int:
    from flywheel_tpu.softmax_attention import _arrays
    return _arrays.current_stream(device)


class Workspace:
    """Scratch memory for the kernels: cudaMalloc'ed through libcudart, zeroed
    once, 256-byte aligned (cudaMalloc aligns to at least that).  It looks
    enough like a tensor (data_ptr / numel) for the callers that pass one."""

    def __init__(self, nbytes, device_index, stream):
        _cuda.set_device(device_index)
        self.nbytes, self.device_index = int(nbytes), device_index
        self.ptr = _cuda.malloc(self.nbytes)
        _cuda.memset(self.ptr, 0, self.nbytes, stream)

    def data_ptr(self):
        return self.ptr

    def numel(self):
        return self.nbytes

    def __del__(self):
        _cuda.free(self.ptr)


_WORKSPACES: dict = {}


def workspace(device, nbytes: int) -> Workspace:
    """A zero-initialised scratch buffer on `device`, grown on demand and reused
    by later calls on the same device and stream."""
    stream = current_stream(device)
    key = (device.index, stream)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _cuda.synchronize(stream)   # the old buffer may still be in use on this stream
        buf = Workspace(max(nbytes, 1 << 20), device.index, stream)
        _WORKSPACES[key] = buf
    return buf


def read_status(buf, device) -> int:
    """The device status word at the head of workspace `buf` (the OR of the
    FW_STATUS_* bits reported since the last read), cleared once read.
    Synchronises the current stream."""
    status = i32(0)
    check(library().fw_read_status(buf.data_ptr(), current_stream(device),
                                   ctypes.byref(status)))
    return status.value


STATUS_TEXT = {
    1: "a bounded device-side wait gave up (FW_STATUS_WAIT_TIMEOUT): the results"
       " of that launch are void",
    2: "a block-table entry outside the pool, or a position past the table row /"
       " the cache capacity, was met (FW_STATUS_BAD_PAGE): reads were clamped to"
       " page 0 and an append there stored nothing",
}


def status_check_enabled() -> bool:
    """FLYWHEEL_CHECK_STATUS=1 makes every entry point read the device status
    word after its launch and raise on a non-zero one.  Off by default: the read
    synchronises the stream, which a serving step cannot afford; the reference
    has no runtime error channel at all."""
    return os.environ.get("FLYWHEEL_CHECK_STATUS", "0") not in ("", "0")


def raise_on_status(buf, device) -> None:
    """Reads the status word of `buf` when the check is enabled and raises
    TimeoutError (a wait gave up) or RuntimeError (bad page) if it is set."""
    if not status_check_enabled():
        return
    status = read_status(buf, device)
    if status == 0:
        return
    text = "; ".join(msg for bit, msg in STATUS_TEXT.items() if status & bit)
    raise (TimeoutError if status & 1 else RuntimeError)(
        f"device status {status}: {text}")
