"""A mixed serving step - decode rows and prefill chunks of one batch - as one
launch sequence.

The reference library has no entry point for this; its serving backend composes
one from three calls (``flywheel_tpu_extend``, patches/tpu-inference.patch:
8219-8320 of the reference project): write the scheduled tokens' K/V through the
slice table, run the decode kernel over the leading one-token requests, run the
paged varlen kernel over the remaining requests with every per-request array
slid past the decode rows, and stitch the two outputs.  ``paged_extend`` keeps
that routine's arguments and result; underneath it is one C-ABI call
(fw_extend_mixed) in which the counts stay on the device, nothing is slid or
stitched on the host, and a one-token row never occupies a tensor-core query
tile.
"""

from __future__ import annotations

import ctypes
import math

from flywheel_tpu.softmax_attention import _arrays, _native
from flywheel_tpu.softmax_attention.config import SUPPORTED_HEAD_DIMS
from flywheel_tpu.softmax_attention.inputs import descale_operand, sinks_operand
from flywheel_tpu.softmax_attention.kv_layout import resolve_merged_kv_heads

__all__ = ["paged_extend"]


def _count_operand(value, name, device):
    tensor = _arrays.to_device(value, device, dtype="int32")
    if tensor.numel() != 1:
        raise ValueError(f"{name} must be one integer; got {tuple(tensor.shape)}.")
    return tensor.reshape(1)


def paged_extend(q, k, v, kv_cache, kv_lens, page_indices, cu_q_lens,
                 kv_write_slices, kv_write_num_slices, num_decode, num_active, *,
                 sm_scale=None, nheads_k=None, window_left=None, softcap=0.0,
                 k_descale=None, v_descale=None, learnable_sink=None):
    """Appends the scheduled tokens, then attends every request to its cache.

    q: (T, nheads, head_dim) bf16, the step's scheduled tokens packed request by
    request; k, v: (T, nheads_k, head_dim) in the cache dtype, or None when the
    pool already holds them.  kv_cache: the merged (num_pages, page_size,
    cache_heads, head_dim) pool.  kv_lens: (max_num_seqs,) KV length of each
    request with this step's tokens included.  page_indices: the block table,
    (max_num_seqs, pages_per_seq) or flat.  cu_q_lens: (max_num_seqs + 1,)
    cumulative query lengths; the first num_decode requests have one token each.
    kv_write_slices / kv_write_num_slices: the (3, columns) slice table of
    write_kv_cache_pages.  num_decode, num_active: ints or device scalars.
    Causal, bottom-right aligned; window_left / softcap / sinks / descales as in
    flash_attn_with_kvcache.

    Returns (output (T, nheads, head_dim), kv_cache); rows past
    cu_q_lens[num_active] are zero.  A device-resident pool is updated in place.
    """
    if q.ndim != 3:
        raise ValueError(f"q must be (tokens, nheads, head_dim); got {tuple(q.shape)}.")
    if (k is None) != (v is None):
        raise ValueError("k and v must be passed together, or both left out.")
    total_q, nheads, head_dim = q.shape
    if kv_cache.ndim != 4:
        raise ValueError(
            "kv_cache must be the merged (num_pages, page_size, cache_heads,"
            f" head_dim) pool; got {tuple(kv_cache.shape)}.")
    if nheads_k is None and k is not None:
        nheads_k = k.shape[-2]
    num_kv_heads = resolve_merged_kv_heads(kv_cache.shape[2], kv_cache.dtype, nheads_k)
    cache_dtype = _arrays.dtype_name(kv_cache.dtype)
    if _arrays.dtype_name(q.dtype) != "bfloat16":
        raise NotImplementedError(f"q must be bfloat16; got {_arrays.dtype_name(q.dtype)}.")
    if kv_cache.shape[3] != head_dim or head_dim not in SUPPORTED_HEAD_DIMS:
        raise ValueError(
            f"head_dim must be one of {SUPPORTED_HEAD_DIMS} and match the cache's;"
            f" got q {head_dim}, cache {kv_cache.shape[3]}.")
    if nheads % num_kv_heads:
        raise ValueError(f"{nheads=} must be a multiple of nheads_k={num_kv_heads}.")
    if k is not None:
        want = (total_q, num_kv_heads, head_dim)
        if tuple(k.shape) != want or tuple(v.shape) != want:
            raise ValueError(f"k and v must be {want}; got {tuple(k.shape)}, {tuple(v.shape)}.")
        if any(_arrays.dtype_name(x.dtype) != cache_dtype for x in (k, v)):
            raise NotImplementedError("k and v must have the cache's dtype; the kernels never quantise.")
        if kv_write_slices is None or kv_write_num_slices is None:
            raise ValueError("k and v need kv_write_slices and kv_write_num_slices.")
    batch = _arrays.shape(kv_lens)[0]
    if _arrays.shape(cu_q_lens) != (batch + 1,):
        raise ValueError(f"cu_q_lens must be ({batch + 1},); got {_arrays.shape(cu_q_lens)}.")

    device = _arrays.pick_device(kv_cache, q)
    pool = _arrays.to_device(kv_cache, device)
    if not pool.is_contiguous():
        raise ValueError("the KV cache must be contiguous.")
    table = _arrays.to_device(page_indices, device, dtype="int32").contiguous().reshape(batch, -1)
    q_dev = _arrays.to_device(q, device).contiguous()
    out = _arrays.empty_like(q_dev)
    lens = _arrays.to_device(kv_lens, device, dtype="int32").contiguous()
    cu = _arrays.to_device(cu_q_lens, device, dtype="int32").contiguous()
    decode_count = _count_operand(num_decode, "num_decode", device)
    active_count = _count_operand(num_active, "num_active", device)
    sinks = sinks_operand(learnable_sink, nheads, device)
    k_scale = descale_operand(k_descale, "k_descale", device)
    v_scale = descale_operand(v_descale, "v_descale", device)
    scale = 1.0 / math.sqrt(head_dim) if sm_scale is None else float(sm_scale)

    args = _native.FwExtendArgs()
    args.attn = _native.FwPrefillArgs(
        q=q_dev.data_ptr(), out=out.data_ptr(), kv_cache=pool.data_ptr(),
        cu_seqlens_q=cu.data_ptr(), seqused_k=lens.data_ptr(), block_table=table.data_ptr(),
        num_active=active_count.data_ptr(), k_descale=_arrays.data_ptr(k_scale),
        v_descale=_arrays.data_ptr(v_scale), sinks=_arrays.data_ptr(sinks),
        num_pages=pool.shape[0], page_size=pool.shape[1], pages_per_seq=table.shape[1],
        batch=batch, total_q=total_q, max_seqlen_q=total_q, nheads=nheads,
        nheads_k=num_kv_heads, head_dim=head_dim, kv_dtype=_native.DTYPE_CODE[cache_dtype],
        causal=1, window_left=-1 if window_left is None else int(window_left),
        softmax_scale=scale, softcap=float(softcap), token_major=1)
    args.num_decode = decode_count.data_ptr()
    keep = []
    if k is not None:
        k_dev = _arrays.to_device(k, device).contiguous()
        v_dev = _arrays.to_device(v, device).contiguous()
        slices = _arrays.to_device(kv_write_slices, device, dtype="int32").contiguous()
        if slices.ndim != 2 or slices.shape[0] != 3:
            raise ValueError(f"kv_write_slices must be (3, columns); got {tuple(slices.shape)}.")
        count = _count_operand(kv_write_num_slices, "kv_write_num_slices", device)
        args.k_new, args.v_new = k_dev.data_ptr(), v_dev.data_ptr()
        args.slices, args.num_slices = slices.data_ptr(), count.data_ptr()
        args.num_columns, args.total_tokens = slices.shape[1], total_q
        keep += [k_dev, v_dev, slices, count]
    lib = _native.library()
    stream = _native.current_stream(device)
    nbytes = lib.fw_extend_workspace_bytes(ctypes.byref(args))
    if nbytes == 0:
        _native.check(lib.fw_extend_mixed(ctypes.byref(args), stream))
        raise RuntimeError(_native.last_error())
    scratch = _native.workspace(device, nbytes)
    args.attn.workspace, args.attn.workspace_bytes = scratch.data_ptr(), scratch.numel()
    _native.check(lib.fw_extend_mixed(ctypes.byref(args), stream))
    _native.raise_on_status(scratch, device)
    cache_out = kv_cache if _arrays.is_device_resident(kv_cache) else _arrays.like(pool, kv_cache)
    return _arrays.like(out, q), cache_out
