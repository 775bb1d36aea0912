"""flash_attn_varlen_func on B200: chunked prefill over the paged merged cache,
and packed K/V through the same tensor-core kernel.

Mirrors flywheel_tpu/softmax_attention/prefill.py of the reference project
(flash_attn_varlen_func :664-963, paged_varlen_attn :437-661).  The packed-K/V
branch and flash_attn_func live in packed.py.
"""

from __future__ import annotations

import ctypes
import math

from flywheel_tpu.softmax_attention import _arrays, _native
from flywheel_tpu.softmax_attention.config import (
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
from flywheel_tpu.softmax_attention.packed import flash_attn_func, packed_varlen_attn

__all__ = ["flash_attn_func", "flash_attn_varlen_func", "paged_prefill_device"]

# Kernel a paged call runs on: "auto" (the library chooses by chunk length),
# "tcgen05" or "splitkv".  Tests and profiling sessions set this attribute to
# pin one; it travels to the library in FwPrefillArgs.route with every call.
FORCED_ROUTE = "auto"


def paged_prefill_device(q, kv_cache, cu_seqlens_q, seqused_k, block_table,
                         num_active, *, max_seqlen_q, nheads_k, softmax_scale,
                         causal, window_left, softcap, return_lse, k_scale,
                         v_scale, sinks, token_major, rotary=None):
    """Launches the paged prefill kernel on CUDA tensors; returns (out, lse or
    None).  q is (nheads, total_q, d), or (total_q, nheads, d) when
    token_major; lse is (nheads, total_q) either way."""
    device = q.device
    if token_major:
        total_q, nheads, head_dim = q.shape
    else:
        nheads, total_q, head_dim = q.shape
    out = _arrays.empty_like(q)
    lse = _arrays.empty((nheads, total_q), "float32", device) if return_lse else None
    if total_q == 0:
        return out, lse
    args = _native.FwPrefillArgs(
        q=q.data_ptr(), out=out.data_ptr(), lse=_arrays.data_ptr(lse),
        kv_cache=kv_cache.data_ptr(), cu_seqlens_q=cu_seqlens_q.data_ptr(),
        seqused_k=seqused_k.data_ptr(), block_table=block_table.data_ptr(),
        num_active=_arrays.data_ptr(num_active),
        k_descale=_arrays.data_ptr(k_scale), v_descale=_arrays.data_ptr(v_scale),
        sinks=_arrays.data_ptr(sinks), workspace=0, workspace_bytes=0,
        num_pages=kv_cache.shape[0], page_size=kv_cache.shape[1],
        pages_per_seq=block_table.shape[1], batch=seqused_k.shape[0],
        total_q=total_q, max_seqlen_q=int(max_seqlen_q), nheads=nheads,
        nheads_k=nheads_k, head_dim=head_dim,
        kv_dtype=_native.DTYPE_CODE[_arrays.dtype_name(kv_cache.dtype)],
        causal=int(bool(causal)),
        window_left=-1 if window_left is None else int(window_left),
        softmax_scale=float(softmax_scale), softcap=float(softcap),
        token_major=int(bool(token_major)),
        route=_native.ROUTE_CODE[FORCED_ROUTE])
    if rotary is not None:
        cos, sin, interleaved = rotary
        args.rotary_cos, args.rotary_sin = cos.data_ptr(), sin.data_ptr()
        args.rotary_len = cos.shape[0]
        args.rotary_interleaved = int(bool(interleaved))
        args.rotary_bf16 = int(_arrays.dtype_name(cos.dtype) == "bfloat16")
    lib = _native.library()
    stream = _native.current_stream(device)
    nbytes = lib.fw_prefill_workspace_bytes(ctypes.byref(args))
    if nbytes == 0:
        _native.check(lib.fw_prefill_paged(ctypes.byref(args), stream))
        raise RuntimeError(_native.last_error())
    scratch = _native.workspace(device, nbytes)
    args.workspace, args.workspace_bytes = scratch.data_ptr(), scratch.numel()
    _native.check(lib.fw_prefill_paged(ctypes.byref(args), stream))
    _native.raise_on_status(scratch, device)
    return out, lse


def flash_attn_varlen_func(
    q,
    k,
    v,
    cu_seqlens_q,
    cu_seqlens_k,
    max_seqlen_q,
    max_seqlen_k,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    window_size=(-1, -1),
    softcap=0.0,
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    return_softmax_lse=False,
    interpret=False,
    head_dim=None,
    token_major=False,
    block_sizes=None,
    *,
    rotary_cos=None,
    rotary_sin=None,
    rotary_interleaved=False,
    rotary_k=True,
    block_table=None,
    seqused_k=None,
    num_active=None,
    k_descale=None,
    v_descale=None,
    nheads_k=None,
    learnable_sink=None,
    guard_replay_unroll=1,
):
    """Packed-sequence attention, forward only.

    Packed K/V (no block_table): q (nheads, total_q, d), k / v (nheads_k,
    total_k, d) bf16 with d 64, 128 or 256, or token-major (total, nheads *
    head_dim) with head_dim= given; cu_seqlens_q / cu_seqlens_k are (num_seqs + 1,) cumulative
    offsets; causal / window masks are bottom-right aligned per sequence (right
    bound -1 or 0); rows past cu_seqlens_q[-1] return out = 0, lse = -inf; RoPE
    rotates K at its own positions and Q from len_k - len_q on.

    Paged KV cache (block_table given; read-only): q is head-major (nheads,
    total_q, headdim) bf16, k is one merged (num_pages, page_size, cache_heads,
    headdim) pool laid out as flash_attn_with_kvcache's and v is None;
    cu_seqlens_k must be None and seqused_k ((batch,) int) is each sequence's
    kv length, its new tokens included, which the cache must already hold.
    cu_seqlens_q[0] must be 0.  causal and window_size are bottom-right aligned
    per sequence; the window right bound is -1 or 0.  num_active keeps only the
    first num_active sequences; rows past the last kept one, and buffer rows
    past cu_seqlens_q[-1], return out = 0 and lse = -inf.  learnable_sink:
    (nheads,) sink logits.  max_seqlen_q / max_seqlen_k must be concrete
    positive ints.  Returns out (nheads, total_q, headdim), or (out, lse) with
    lse (nheads, total_q) float32 when return_softmax_lse.  rotary_cos /
    rotary_sin ((seqlen_ro, headdim / 2), q's dtype or float32) with
    rotary_k=False rotate Q only, token t of a sequence at position seqused_k -
    len_q + t (the cache holds K already rotated); the table must cover
    max_seqlen_k.  block_sizes and interpret are accepted and ignored.
    Forward-only.
    """
    del interpret, block_sizes
    window_size = check_common_kwargs(
        window_size, dropout_p=dropout_p, softcap=softcap,
        alibi_slopes=alibi_slopes, deterministic=deterministic,
        return_attn_probs=return_attn_probs)
    if block_table is None:
        if seqused_k is not None or num_active is not None:
            raise ValueError(
                "seqused_k and num_active describe a paged KV cache and need"
                " block_table; packed K/V takes cu_seqlens_k.")
        if any(arg is not None for arg in (k_descale, v_descale, nheads_k)):
            raise ValueError(
                "k_descale, v_descale and nheads_k describe an fp8 paged pool and"
                " need block_table; packed K/V is bf16.")
        return packed_varlen_attn(
            q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
            softmax_scale=softmax_scale, causal=causal, window_size=window_size,
            softcap=softcap, return_softmax_lse=bool(return_softmax_lse),
            head_dim=head_dim, token_major=bool(token_major), rotary_cos=rotary_cos,
            rotary_sin=rotary_sin, rotary_interleaved=rotary_interleaved,
            rotary_k=rotary_k, learnable_sink=learnable_sink)
    if guard_replay_unroll != 1:
        raise ValueError(
            "guard_replay_unroll applies to packed K/V; a paged KV cache"
            " always unrolls its replay.")
    if token_major:
        raise NotImplementedError(
            "a paged KV cache takes head-major q (nheads, total_q, headdim);"
            " token_major=True is not supported.")
    if head_dim is not None:
        raise ValueError(
            "head_dim is only meaningful for token-major inputs; a paged call"
            " takes head-major q.")
    if cu_seqlens_k is not None:
        raise ValueError(
            "with block_table, pass cu_seqlens_k=None: seqused_k gives each"
            " sequence's kv length.")
    if v is not None:
        raise ValueError(
            "with block_table, pass one merged (num_pages, page_size,"
            " cache_heads, headdim) cache as k and v=None; separate paged K and"
            " V caches are not supported.")
    if seqused_k is None:
        raise ValueError(
            "block_table needs seqused_k, the (batch,) kv length of each"
            " sequence (its new tokens included).")
    if rotary_cos is not None and rotary_k:
        raise NotImplementedError(
            "a paged KV cache holds K already rotated; pass rotary_k=False to"
            " rotate Q only.")
    if type(rotary_interleaved) is not bool:
        raise ValueError("rotary_interleaved must be a static bool.")
    if (rotary_cos is None) != (rotary_sin is None):
        raise ValueError("rotary_cos and rotary_sin must be provided together.")
    for arg_name, bound in (("max_seqlen_q", max_seqlen_q),
                            ("max_seqlen_k", max_seqlen_k)):
        if not isinstance(bound, int):
            raise ValueError(
                f"{arg_name} must be a concrete int (it picks the kernel's"
                " block sizes); pass a static bucket bound, not a traced"
                " value.")
        if bound <= 0:
            raise ValueError(f"{arg_name} must be positive; got {bound}.")
    if q.ndim != 3:
        raise ValueError(
            "with block_table, q must be (nheads, total_q, headdim); got"
            f" {tuple(q.shape)=}.")
    cu_shape = _arrays.shape(cu_seqlens_q)
    if (len(cu_shape) != 1 or cu_shape[0] < 2
            or not _arrays.is_integer(cu_seqlens_q)):
        raise ValueError(
            "cu_seqlens_q must be a 1-D integer array of batch + 1 boundaries;"
            f" got {cu_shape} {_arrays.dtype_name(cu_seqlens_q.dtype)}.")
    batch = cu_shape[0] - 1
    if _arrays.is_host(cu_seqlens_q) and int(cu_seqlens_q[0]) != 0:
        raise ValueError(
            "with block_table, cu_seqlens_q must start at 0; got"
            f" cu_seqlens_q[0]={int(cu_seqlens_q[0])}.")
    if isinstance(num_active, int) and not 0 <= num_active <= batch:
        raise ValueError(
            f"num_active must be in [0, {batch}]; got {num_active}.")
    nheads, total_q, head_dim_qk = q.shape
    if k.ndim != 4:
        raise ValueError(
            "with block_table, k must be the merged (num_pages, page_size,"
            f" cache_heads, headdim) pool; got {tuple(k.shape)=}.")
    num_kv_heads = resolve_merged_kv_heads(k.shape[2], k.dtype, nheads_k)
    if _arrays.dtype_name(q.dtype) != "bfloat16":
        raise NotImplementedError(
            f"q must be bfloat16; got {_arrays.dtype_name(q.dtype)}.")
    if k.shape[3] != head_dim_qk or head_dim_qk not in SUPPORTED_HEAD_DIMS:
        raise ValueError(
            f"headdim must be one of {SUPPORTED_HEAD_DIMS} and match the"
            f" cache's; got q {head_dim_qk}, cache {k.shape[3]}.")
    if k.shape[1] % PAGE_SIZE_MULTIPLE:
        raise ValueError(
            "page_size (k.shape[1]) must be a multiple of"
            f" {PAGE_SIZE_MULTIPLE}; got {k.shape[1]}.")
    if nheads % num_kv_heads:
        raise ValueError(f"{nheads=} must be a multiple of nheads_k={num_kv_heads}.")
    if block_table.ndim != 2 or block_table.shape[0] != batch:
        raise ValueError(
            f"block_table must be (batch={batch}, max_pages_per_seq); got"
            f" {tuple(block_table.shape)}.")
    if tuple(_arrays.shape(seqused_k)) != (batch,):
        raise ValueError(
            f"seqused_k must be ({batch},); got {tuple(_arrays.shape(seqused_k))}.")

    softmax_scale = (1.0 / math.sqrt(head_dim_qk) if softmax_scale is None
                     else float(softmax_scale))
    window = resolve_window(window_size, bool(causal))
    check_paged_window(window, window_size)
    device = _arrays.pick_device(k, q)
    sinks = sinks_operand(learnable_sink, nheads, device)
    k_scale = descale_operand(k_descale, "k_descale", device)
    v_scale = descale_operand(v_descale, "v_descale", device)
    active = None
    if num_active is not None:
        active = _arrays.to_device(num_active, device, dtype="int32")
        if active.numel() != 1:
            raise ValueError(
                f"num_active must be one integer; got {tuple(active.shape)}.")
        active = active.reshape(1)
    q_dev = _arrays.to_device(q, device).contiguous()
    pool = _arrays.to_device(k, device)
    if not pool.is_contiguous():
        raise ValueError("the KV cache must be contiguous.")
    rotary = None
    if rotary_cos is not None:
        cos_shape, sin_shape = _arrays.shape(rotary_cos), _arrays.shape(rotary_sin)
        if len(cos_shape) != 2 or sin_shape != cos_shape:
            raise ValueError("rotary_cos and rotary_sin must have the same 2-D shape.")
        if 2 * cos_shape[1] != head_dim_qk:
            raise ValueError(
                f"rotary_dim ({2 * cos_shape[1]}) must equal head_dim ({head_dim_qk});"
                " partial rotary is not supported.")
        names = (_arrays.dtype_name(rotary_cos.dtype), _arrays.dtype_name(rotary_sin.dtype))
        if names[0] != names[1] or names[0] not in ("bfloat16", "float32"):
            raise ValueError("rotary_cos and rotary_sin must share Q's dtype or be float32.")
        if cos_shape[0] < max_seqlen_k:
            raise ValueError("rotary table is shorter than the KV sequence bound.")
        rotary = (_arrays.to_device(rotary_cos, device).contiguous(),
                  _arrays.to_device(rotary_sin, device).contiguous(), rotary_interleaved)
    out, lse = paged_prefill_device(
        q_dev, pool,
        _arrays.to_device(cu_seqlens_q, device, dtype="int32").contiguous(),
        _arrays.to_device(seqused_k, device, dtype="int32").contiguous(),
        _arrays.to_device(block_table, device, dtype="int32").contiguous(),
        active, max_seqlen_q=max_seqlen_q, nheads_k=num_kv_heads,
        softmax_scale=softmax_scale, causal=window[1] == 0,
        window_left=window[0], softcap=float(softcap),
        return_lse=bool(return_softmax_lse), k_scale=k_scale, v_scale=v_scale,
        sinks=sinks, token_major=False, rotary=rotary)
    if return_softmax_lse:
        return _arrays.like(out, q), _arrays.like(lse, q)
    return _arrays.like(out, q)
