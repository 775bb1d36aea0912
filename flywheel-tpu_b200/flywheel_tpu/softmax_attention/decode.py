"""flash_attn_with_kvcache on B200: attention against a contiguous or paged KV
cache with the new tokens' K/V append fused into the launch.

Mirrors flywheel_tpu/softmax_attention/decode.py:189-625 of the reference
project: same name, arguments, layouts, return tuples and error behaviour.
Differences, all widening: page_size may be any multiple of 16 (the reference
needs 128), a (batch, seqlen_q, ...) verify window runs on the decode kernel
also with a left window, and the arrays are torch / NumPy / DLPack arrays
instead of JAX arrays (see _arrays; torch is not needed for NumPy callers).
"""

from __future__ import annotations

import ctypes
import math

from flywheel_tpu.softmax_attention import _arrays, _native
from flywheel_tpu.softmax_attention.config import (
    DECODE_HEAD_DIMS,
    MAX_DECODE_BATCH,
    max_folded_query_rows,
    PAGE_SIZE_MULTIPLE,
    SUPPORTED_HEAD_DIMS,
)
from flywheel_tpu.softmax_attention.inputs import (
    check_common_kwargs,
    check_paged_window,
    descale_operand,
    resolve_window,
    sinks_operand,
)
from flywheel_tpu.softmax_attention.kv_layout import resolve_merged_kv_heads


def _num_active_operand(num_active, batch, device):
    if num_active is None:
        return None
    if isinstance(num_active, int):
        if not 0 <= num_active <= batch:
            raise ValueError(
                f"num_active must be in [0, {batch}]; got {num_active}.")
    tensor = _arrays.to_device(num_active, device, dtype="int32")
    if tensor.numel() != 1:
        raise ValueError(
            f"num_active must be one integer; got {tuple(tensor.shape)}.")
    return tensor.reshape(1)


def append_ragged(kv_cache, k, v, cu_seqlens_q, cache_seqlens, block_table,
                  num_active, *, nheads_k):
    """Packed new K/V rows (total, nheads_k, d) -> merged pages, in place
    (kernels/kv_append.py:116-184 of the reference).  All operands are CUDA
    tensors."""
    device = kv_cache.device
    args = _native.FwAppendArgs(
        kv_cache=kv_cache.data_ptr(), k_new=k.data_ptr(), v_new=v.data_ptr(),
        cu_seqlens_q=cu_seqlens_q.data_ptr(),
        cache_seqlens=cache_seqlens.data_ptr(),
        block_table=block_table.data_ptr(),
        num_active=_arrays.data_ptr(num_active),
        num_pages=kv_cache.shape[0], page_size=kv_cache.shape[1],
        pages_per_seq=block_table.shape[1], batch=cache_seqlens.shape[0],
        total_tokens=k.shape[0], nheads_k=nheads_k, head_dim=k.shape[-1],
        kv_dtype=_native.DTYPE_CODE[_arrays.dtype_name(kv_cache.dtype)])
    _native.check(_native.library().fw_append_ragged(
        ctypes.byref(args), _native.current_stream(device)))
    return kv_cache


def flash_attn_with_kvcache(
    q,
    k_cache,
    v_cache,
    k=None,
    v=None,
    *,
    cache_seqlens,
    cache_batch_idx=None,
    block_table=None,
    num_active=None,
    cu_seqlens_q=None,
    max_seqlen_q=None,
    softmax_scale=None,
    causal=False,
    window_size=(-1, -1),
    softcap=0.0,
    return_softmax_lse=False,
    interpret=False,
    k_descale=None,
    v_descale=None,
    nheads_k=None,
    learnable_sink=None,
):
    """Attention against a contiguous or paged KV cache, with optional append.

    block_table picks one of two cache layouts:

    - block_table=None, contiguous pair: k_cache and v_cache are separate
      (batch_cache, capacity, nheads_k, head_dim) bf16 arrays, capacity a
      multiple of 16; cache_batch_idx: optional (batch,) cache row per query
      row.  Single-token decode only.
    - block_table given, paged merged: k_cache is one (num_pages, page_size,
      cache_heads, head_dim) pool whose token rows hold [k0, v0, k1, v1, ...],
      page_size a multiple of 16, v_cache None; bf16, or float8_e4m3fn /
      float8_e5m2 with per-tensor k_descale / v_descale (an odd fp8 nheads_k is
      padded by one zero head and needs nheads_k).

    q: (batch, seqlen_q, nheads, head_dim) bf16, or packed (total_q, nheads,
    head_dim) with cu_seqlens_q and a static max_seqlen_q.  k / v: new tokens in
    q's token layout with nheads_k heads in the cache dtype, appended after
    each row's cache_seqlens and then attended.  causal and window_size are
    bottom-right aligned; multi-token and packed calls take a window right
    bound of -1 or 0 only.  softcap > 0 applies softcap * tanh(s / softcap).
    learnable_sink: (nheads,) logits that join the softmax denominator with no
    value row.  num_active: leading rows that are real requests.

    Returns (out, k_cache, v_cache) for the contiguous pair and (out,
    kv_cache) for the paged merged cache, with lse after out when
    return_softmax_lse: (batch, nheads, seqlen_q), or (nheads, total_q) when
    packed.  Device-resident caches are updated in place and returned.
    `interpret` is accepted and ignored: there is no CPU path.
    """
    del interpret
    window_size = check_common_kwargs(window_size, softcap=softcap)
    is_ragged = cu_seqlens_q is not None
    if is_ragged:
        cu_shape = _arrays.shape(cu_seqlens_q)
        if (len(cu_shape) != 1 or cu_shape[0] < 2
                or not _arrays.is_integer(cu_seqlens_q)):
            raise ValueError(
                "cu_seqlens_q must be a 1-D integer array of batch + 1"
                " boundaries.")
        if q.ndim != 3:
            raise ValueError(
                "With cu_seqlens_q, q must be (total_q, nheads, head_dim).")
        if type(max_seqlen_q) is not int or max_seqlen_q <= 0:
            raise ValueError(
                "With cu_seqlens_q, max_seqlen_q must be a positive static"
                " python int, the longest request's query length; got"
                f" {max_seqlen_q!r}.")
        batch = cu_shape[0] - 1
        nheads, head_dim = q.shape[-2:]
        seqlen_q = None
    elif max_seqlen_q is not None:
        raise ValueError(
            "max_seqlen_q is only for a packed q with cu_seqlens_q; a (batch,"
            " seqlen_q, nheads, head_dim) q takes seqlen_q from its shape; got"
            f" {max_seqlen_q=}.")
    elif q.ndim != 4:
        raise ValueError(
            f"q must be (batch, seqlen_q, nheads, head_dim); got {tuple(q.shape)=}.")
    else:
        batch, seqlen_q, nheads, head_dim = q.shape
        if batch <= 0 or seqlen_q <= 0:
            raise ValueError("batch and seqlen_q must be positive.")
    is_extend = is_ragged or seqlen_q != 1
    is_paged = block_table is not None
    if is_extend and not is_paged:
        raise NotImplementedError(
            "Multi-token and packed KV-cache attention needs the paged merged"
            " cache (block_table); the contiguous K/V pair serves single-token"
            " decode only.")
    cache_dtype = _arrays.dtype_name(k_cache.dtype)
    if is_paged:
        if v_cache is not None:
            raise ValueError(
                "With block_table, pass one merged (num_pages, page_size,"
                " cache_heads, head_dim) cache as k_cache and v_cache=None;"
                " separate paged K and V caches are not supported.")
        if cache_batch_idx is not None:
            raise ValueError(
                "block_table and cache_batch_idx are mutually exclusive: the"
                " block table already maps each query row to its pages.")
        if k_cache.ndim != 4:
            raise ValueError(
                "With block_table, k_cache must be (num_pages, page_size,"
                " cache_heads, head_dim), the KV heads' K and V rows"
                f" interleaved; got {tuple(k_cache.shape)=}.")
        if nheads_k is None and k is not None:
            nheads_k = k.shape[-2]
        pool_heads = resolve_merged_kv_heads(k_cache.shape[2], k_cache.dtype,
                                             nheads_k)
        if k_cache.shape[1] % PAGE_SIZE_MULTIPLE:
            raise ValueError(
                "page_size (k_cache.shape[1]) must be a multiple of"
                f" {PAGE_SIZE_MULTIPLE}; got {k_cache.shape[1]}.")
        if not _arrays.is_integer(block_table):
            raise ValueError(
                "block_table must be an integer array; got"
                f" {_arrays.dtype_name(block_table.dtype)}.")
        if block_table.ndim != 2 or block_table.shape[0] != batch:
            raise ValueError(
                f"block_table must be (batch={batch}, max_pages_per_seq); got"
                f" {tuple(block_table.shape)}.")
        cache_shape = (*k_cache.shape[:2], pool_heads, k_cache.shape[3])
        cache_operands = (k_cache,)
    else:
        if v_cache is None:
            raise ValueError(
                "Without block_table, k_cache and v_cache must be separate"
                " (batch_cache, capacity, nheads_k, head_dim) caches; got"
                " v_cache=None (a merged cache must be paged).")
        if k_cache.ndim != 4 or tuple(v_cache.shape) != tuple(k_cache.shape):
            raise ValueError(
                "k_cache and v_cache must share the shape (batch_cache,"
                f" capacity, nheads_k, head_dim); got {tuple(k_cache.shape)=},"
                f" {tuple(v_cache.shape)=}.")
        if nheads_k is not None and nheads_k != k_cache.shape[2]:
            raise ValueError(
                f"{nheads_k=} must match the contiguous caches'"
                f" {k_cache.shape[2]}.")
        if k_cache.shape[1] % PAGE_SIZE_MULTIPLE:
            raise ValueError(
                "capacity (k_cache.shape[1]) must be a multiple of"
                f" {PAGE_SIZE_MULTIPLE}; got {k_cache.shape[1]}.")
        cache_shape = tuple(k_cache.shape)
        cache_operands = (k_cache, v_cache)
    nheads_k = cache_shape[2]
    if cache_shape[3] != head_dim:
        raise ValueError(
            f"cache head_dim {cache_shape[3]} must match q's {head_dim}.")
    if nheads_k <= 0 or nheads <= 0 or nheads % nheads_k:
        raise ValueError(f"{nheads=} must be a multiple of {nheads_k=}.")
    has_new = k is not None
    if has_new != (v is not None):
        raise ValueError("k and v must be passed together, or both left out.")
    kv_operands = (*cache_operands, k, v) if has_new else cache_operands
    if (_arrays.dtype_name(q.dtype) != "bfloat16"
            or any(_arrays.dtype_name(op.dtype) != cache_dtype for op in kv_operands)
            or (not is_paged and cache_dtype != "bfloat16")
            or cache_dtype not in _native.DTYPE_CODE):
        kv_dtypes = tuple(_arrays.dtype_name(op.dtype) for op in kv_operands)
        raise NotImplementedError(
            "q must be bfloat16 and the KV operands share one dtype, bfloat16"
            " or (paged pool) float8_e4m3fn / float8_e5m2; got q"
            f" {_arrays.dtype_name(q.dtype)}, KV {kv_dtypes}.")
    expected_new_shape = (*q.shape[:-2], nheads_k, head_dim)
    if has_new and (tuple(k.shape) != expected_new_shape
                    or tuple(v.shape) != expected_new_shape):
        raise ValueError(
            f"k and v must be {expected_new_shape} (matching q's token layout);"
            f" got {tuple(k.shape)=}, {tuple(v.shape)=}.")
    if head_dim not in DECODE_HEAD_DIMS:
        raise NotImplementedError(
            f"head_dim {head_dim} is not built; this library serves"
            f" {DECODE_HEAD_DIMS}.")
    if head_dim not in SUPPORTED_HEAD_DIMS and cache_dtype != "bfloat16":
        raise NotImplementedError(
            f"head_dim {head_dim} is built for bfloat16 caches; fp8 caches take"
            f" head_dim {SUPPORTED_HEAD_DIMS}.")

    device = _arrays.pick_device(k_cache, q)
    lengths = _arrays.to_device(cache_seqlens, device, dtype="int32")
    if lengths.ndim == 0:
        lengths = _arrays.broadcast_scalar(lengths, batch, device)
    if tuple(lengths.shape) != (batch,):
        raise ValueError(
            f"cache_seqlens must be a scalar or ({batch},) int array; got"
            f" {tuple(lengths.shape)}.")
    lengths = lengths.contiguous()
    if cache_batch_idx is not None:
        cache_batch_idx = _arrays.to_device(cache_batch_idx, device, dtype="int32")
        if tuple(cache_batch_idx.shape) != (batch,):
            raise ValueError(
                f"cache_batch_idx must be a scalar or ({batch},) int array; got"
                f" {tuple(cache_batch_idx.shape)}.")
        cache_batch_idx = cache_batch_idx.contiguous()

    softmax_scale = (1.0 / math.sqrt(head_dim) if softmax_scale is None
                     else float(softmax_scale))
    window = resolve_window(window_size, bool(causal))
    if is_extend:
        check_paged_window(window, window_size)
    elif window[1] not in (None, 0):
        # A single query token sits on the last key: a right reach adds nothing.
        window = (window[0], None)
    is_causal = window[1] == 0
    sinks = sinks_operand(learnable_sink, nheads, device)
    k_scale = descale_operand(k_descale, "k_descale", device)
    v_scale = descale_operand(v_descale, "v_descale", device)
    active = _num_active_operand(num_active, batch, device)

    q_dev = _arrays.to_device(q, device).contiguous()
    cache_dev = [_arrays.to_device(c, device) for c in cache_operands]
    if any(not c.is_contiguous() for c in cache_dev):
        raise ValueError("the KV cache must be contiguous.")
    k_dev = _arrays.to_device(k, device).contiguous() if has_new else None
    v_dev = _arrays.to_device(v, device).contiguous() if has_new else None
    table = (_arrays.to_device(block_table, device, dtype="int32").contiguous()
             if is_paged else None)

    group = nheads // nheads_k
    is_folded = (is_extend and not is_ragged
                 and seqlen_q * group <= max_folded_query_rows(head_dim))
    lib = _native.library()
    stream = _native.current_stream(device)
    lse = None
    if not is_extend or is_folded:
        out = _arrays.empty_like(q_dev)
        if return_softmax_lse:
            lse = _arrays.empty((batch, nheads, seqlen_q), "float32", device)
        kernel_has_new = has_new
        args = _native.FwDecodeArgs(
            q=q_dev.data_ptr(), out=out.data_ptr(), lse=_arrays.data_ptr(lse),
            kv_cache=cache_dev[0].data_ptr(),
            v_cache=0 if is_paged else cache_dev[1].data_ptr(),
            k_new=_arrays.data_ptr(k_dev), v_new=_arrays.data_ptr(v_dev),
            cache_seqlens=lengths.data_ptr(),
            block_table=_arrays.data_ptr(table),
            cache_batch_idx=_arrays.data_ptr(cache_batch_idx),
            num_active=_arrays.data_ptr(active),
            k_descale=_arrays.data_ptr(k_scale),
            v_descale=_arrays.data_ptr(v_scale), sinks=_arrays.data_ptr(sinks),
            partial_out=0, partial_lse=0, workspace=0, workspace_bytes=0,
            num_pages=cache_dev[0].shape[0], page_size=cache_dev[0].shape[1],
            pages_per_seq=table.shape[1] if is_paged else 1, batch=batch,
            seqlen_q=seqlen_q, nheads=nheads, nheads_k=nheads_k,
            head_dim=head_dim, kv_dtype=_native.DTYPE_CODE[cache_dtype],
            causal=int(is_causal),
            window_left=-1 if window[0] is None else int(window[0]),
            softmax_scale=softmax_scale, softcap=float(softcap), num_ctas=0)
        # The kernel takes up to MAX_DECODE_BATCH rows per launch (its per-CTA
        # scan of the batch lives in shared memory); larger batches go in slices.
        # Rows are independent, so slicing changes nothing but num_active, which
        # is rebased on the device.
        for first in range(0, batch, MAX_DECODE_BATCH):
            rows = min(MAX_DECODE_BATCH, batch - first)
            part = _native.FwDecodeArgs.from_buffer_copy(args)
            part.batch = rows
            part.q = q_dev[first:].data_ptr()
            part.out = out[first:].data_ptr()
            part.lse = 0 if lse is None else lse[first:].data_ptr()
            part.cache_seqlens = lengths[first:].data_ptr()
            if has_new and kernel_has_new:
                part.k_new, part.v_new = k_dev[first:].data_ptr(), v_dev[first:].data_ptr()
            if is_paged:
                part.block_table = table[first:].data_ptr()
            elif cache_batch_idx is not None:
                part.cache_batch_idx = cache_batch_idx[first:].data_ptr()
            elif first:
                # identity mapping of a later slice: spell the cache rows out
                rows_idx = _arrays.arange_scaled(rows, 1, device, first=first)
                part.cache_batch_idx = rows_idx.data_ptr()
            if active is not None and first:
                rebased = _arrays.rebase_count(active, first, rows)
                part.num_active = rebased.data_ptr()
            nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(part))
            if nbytes == 0:
                _native.check(lib.fw_decode_kvcache(ctypes.byref(part), stream))
                raise RuntimeError(_native.last_error())
            scratch = _native.workspace(device, nbytes)
            part.workspace, part.workspace_bytes = scratch.data_ptr(), scratch.numel()
            _native.check(lib.fw_decode_kvcache(ctypes.byref(part), stream))
            _native.raise_on_status(scratch, device)
    else:
        if head_dim not in SUPPORTED_HEAD_DIMS:
            raise NotImplementedError(
                f"head_dim {head_dim} is served by the decode kernel only (one"
                " query token, or a (batch, seqlen_q, ...) window of up to"
                f" {max_folded_query_rows(head_dim)} query rows per KV head);"
                f" packed and longer calls need head_dim {SUPPORTED_HEAD_DIMS}.")
        from flywheel_tpu.softmax_attention.prefill import paged_prefill_device
        if is_ragged:
            cu = _arrays.to_device(cu_seqlens_q, device, dtype="int32").contiguous()
            packed_q, packed_k, packed_v = q_dev, k_dev, v_dev
            packed_max = max_seqlen_q
        else:
            cu = _arrays.arange_scaled(batch + 1, seqlen_q, device)
            packed_q = q_dev.reshape(-1, nheads, head_dim)
            packed_k = k_dev.reshape(-1, nheads_k, head_dim) if has_new else None
            packed_v = v_dev.reshape(-1, nheads_k, head_dim) if has_new else None
            packed_max = seqlen_q
        if has_new:
            append_ragged(cache_dev[0], packed_k, packed_v, cu, lengths, table,
                          active, nheads_k=nheads_k)
            # seqused_k = cache_seqlens + this request's new tokens.  (Index
            # arithmetic on metadata; the attention itself is the CUDA kernel.)
            seqused = _arrays.add_token_counts(lengths, cu)
        else:
            seqused = lengths
        out, lse = paged_prefill_device(
            packed_q, cache_dev[0], cu, seqused.contiguous(), table, active,
            max_seqlen_q=packed_max, nheads_k=nheads_k,
            softmax_scale=softmax_scale, causal=is_causal,
            window_left=window[0], softcap=float(softcap),
            return_lse=bool(return_softmax_lse), k_scale=k_scale,
            v_scale=v_scale, sinks=sinks, token_major=True)
        if not is_ragged:
            out = out.reshape(q_dev.shape)
            if lse is not None:
                lse = _arrays.heads_first_to_batch_first(lse, nheads, batch, seqlen_q)

    caches_out = tuple(
        original if _arrays.is_device_resident(original) else _arrays.like(updated, original)
        for original, updated in zip(cache_operands, cache_dev))
    out = _arrays.like(out, q)
    if return_softmax_lse:
        return (out, _arrays.like(lse, q), *caches_out)
    return (out, *caches_out)
