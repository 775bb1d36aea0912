"""write_kv_cache_pages: new K/V rows into the merged interleaved paged KV
cache, for callers that keep the cache themselves (a serving engine's prefill
cache fill).  Mirrors flywheel_tpu/softmax_attention/page.py:35-73 of the
reference project."""

from __future__ import annotations

import ctypes

from flywheel_tpu.softmax_attention import _arrays, _native
from flywheel_tpu.softmax_attention.kv_layout import (
    check_merged_kv_dtype,
    merged_cache_heads,
)


def write_kv_cache_pages(k, v, kv_cache, slices, num_slices, *, interpret=False):
    """Copy new K/V rows into the merged interleaved cache; returns the cache,
    updated in place when it lives on the device.

    k and v are (T, H, D) and kv_cache is (P, S, merged_cache_heads(H), D), all
    of one dtype: bf16, or fp8 already quantized by the caller. slices is
    i32[3, n] and num_slices i32[1]: column j < num_slices[0] of slices is
    (cache_row_start, new_row_start, length) in rows of the flat (P * S) cache
    view and of k / v, each piece inside one page; later columns are ignored.
    `interpret` is accepted and ignored.
    """
    del interpret
    _, num_kv_heads, head_dim = k.shape
    _, _, cache_heads, cache_head_dim = kv_cache.shape
    check_merged_kv_dtype(kv_cache.dtype)
    names = [_arrays.dtype_name(x.dtype) for x in (k, v, kv_cache)]
    if names[0] != names[2] or names[1] != names[2]:
        raise NotImplementedError(
            f"k, v and the cache must share one dtype; got {names[0]},"
            f" {names[1]}, {names[2]}.")
    if tuple(v.shape) != tuple(k.shape) or (cache_heads, cache_head_dim) != (
            merged_cache_heads(num_kv_heads, kv_cache.dtype), head_dim):
        raise ValueError(
            "k and v must be (T, H, D) of a (P, S, merged_cache_heads(H), D)"
            f" cache; got {tuple(k.shape)=}, {tuple(v.shape)=}, {tuple(kv_cache.shape)=}.")
    if head_dim % 128:
        raise ValueError(f"head_dim must be a multiple of 128; got {head_dim}.")
    if len(_arrays.shape(slices)) != 2 or _arrays.shape(slices)[0] != 3:
        raise ValueError(f"slices must be i32[3, n]; got {_arrays.shape(slices)}.")
    device = _arrays.pick_device(kv_cache, k)
    cache = _arrays.to_device(kv_cache, device)
    if not cache.is_contiguous():
        raise ValueError("the KV cache must be contiguous.")
    k_dev = _arrays.to_device(k, device).contiguous()
    v_dev = _arrays.to_device(v, device).contiguous()
    table = _arrays.to_device(slices, device, dtype="int32").contiguous()
    count = _arrays.to_device(num_slices, device, dtype="int32").reshape(-1)[:1].contiguous()
    args = _native.FwWritePagesArgs(
        kv_cache=cache.data_ptr(), k_new=k_dev.data_ptr(), v_new=v_dev.data_ptr(),
        slices=table.data_ptr(), num_slices=count.data_ptr(), num_pages=cache.shape[0],
        page_size=cache.shape[1], num_columns=table.shape[1], total_tokens=k_dev.shape[0],
        nheads_k=num_kv_heads, head_dim=head_dim,
        kv_dtype=_native.DTYPE_CODE[names[2]])
    _native.check(_native.library().fw_write_kv_pages(
        ctypes.byref(args), _native.current_stream(device)))
    if _arrays.is_device_resident(kv_cache):
        return kv_cache
    return _arrays.like(cache, kv_cache)
