"""Forward attention over packed (non-paged) K/V on B200: flash_attn_func and the
cu_seqlens_k branch of flash_attn_varlen_func.

Mirrors flywheel_tpu/softmax_attention/prefill.py:62-341 (flash_attn_func) and
:818-963 (packed flash_attn_varlen_func) of the reference project, forward
only.  Both run the tcgen05 prefill kernel with K and V addressed by token row
(fw_attention_packed).  Built: bfloat16, head_dim 64, 128 and 256, nheads / nheads_k up to 128, causal / full / (left, right) window masks, softcap,
sinks, lse, fused RoPE on Q and K.  Not built (raise NotImplementedError):
other head dims, head_dim_v != head_dim, heads_outer_fold, attention_chunk.
"""

from __future__ import annotations

import ctypes
import math


from flywheel_tpu.softmax_attention import _arrays, _native
from flywheel_tpu.softmax_attention.inputs import (
    check_common_kwargs,
    resolve_window,
    sinks_operand,
)

PACKED_HEAD_DIMS = (64, 128, 256)
MAX_PACKED_GROUP = 128


def parse_qkv(q, k, v, head_dim, token_major, expected_rank, layout):
    """nheads, nheads_k, head_dim of q / k / v (inputs.py:154-215 of the
    reference).  `layout` names the head-major axes for the message."""
    if token_major:
        if q.ndim != expected_rank:
            raise ValueError(
                f"token_major=True expects {expected_rank}-D (..., seqlen,"
                f" nheads * head_dim) q/k/v; got {tuple(q.shape)=}. Pass"
                f" token_major=False for {expected_rank + 1}-D inputs.")
        if head_dim is None:
            raise ValueError(
                "token-major (fused head_dim) inputs require head_dim=; the fused"
                f" width alone cannot determine the head split (got {tuple(q.shape)=}).")
        if type(head_dim) is not int:
            raise ValueError(f"head_dim must be a static python int; got {head_dim!r}.")
        if head_dim <= 0 or (head_dim % 128 and head_dim != 64):
            raise ValueError(
                "token-major inputs require head_dim % 128 == 0 or head_dim == 64"
                f" (paired); got {head_dim}.")
        if k.ndim != expected_rank or v.ndim != expected_rank:
            raise ValueError(
                f"q/k/v ranks must match; got {tuple(q.shape)=}, {tuple(k.shape)=},"
                f" {tuple(v.shape)=}.")
        if q.shape[-1] % head_dim or k.shape[-1] % head_dim:
            raise ValueError(
                f"head_dim {head_dim} must divide q/k fused widths; got"
                f" {tuple(q.shape)=}, {tuple(k.shape)=}.")
        nheads, nheads_k = q.shape[-1] // head_dim, k.shape[-1] // head_dim
        head_dim_qk, head_dim_v = head_dim, v.shape[-1] // max(nheads_k, 1)
        batch_axes = range(expected_rank - 2)
    else:
        if head_dim is not None:
            raise ValueError(
                "head_dim is only meaningful for token-major (..., seqlen,"
                f" nheads * head_dim) inputs; {expected_rank}-D inputs carry"
                " the split in their shape.")
        if any(operand.ndim != expected_rank for operand in (q, k, v)):
            raise ValueError(
                f"q/k/v must be {expected_rank}-D ({layout}); got {tuple(q.shape)=},"
                f" {tuple(k.shape)=}, {tuple(v.shape)=}.")
        if q.shape[-1] != k.shape[-1]:
            raise ValueError(f"Incompatible shapes: {tuple(q.shape)=} vs {tuple(k.shape)=}.")
        head_axis = expected_rank - 3
        nheads, head_dim_qk = q.shape[head_axis], q.shape[-1]
        nheads_k, head_dim_v = k.shape[head_axis], v.shape[-1]
        batch_axes = range(head_axis)
    if any(q.shape[axis] != k.shape[axis] for axis in batch_axes):
        raise ValueError(f"Incompatible shapes: {tuple(q.shape)=} vs {tuple(k.shape)=}.")
    if tuple(k.shape[:-1]) != tuple(v.shape[:-1]):
        raise ValueError(
            f"k and v must share every axis but head_dim; got {tuple(k.shape)=},"
            f" {tuple(v.shape)=}.")
    if nheads_k == 0 or nheads % nheads_k:
        raise ValueError(f"{nheads=} must be a multiple of {nheads_k=}.")
    names = {_arrays.dtype_name(x.dtype) for x in (q, k, v)}
    if names != {"bfloat16"}:
        raise NotImplementedError(f"Only bfloat16 is supported; got {sorted(names)}.")
    if head_dim_v != head_dim_qk:
        raise NotImplementedError(
            f"head_dim_v ({head_dim_v}) != head_dim ({head_dim_qk}) is not built.")
    if head_dim_qk not in PACKED_HEAD_DIMS:
        raise NotImplementedError(
            f"packed K/V attention is built for head_dim {PACKED_HEAD_DIMS}; got {head_dim_qk}.")
    group = nheads // nheads_k
    if group > MAX_PACKED_GROUP:
        raise NotImplementedError(
            f"packed K/V attention is built for nheads / nheads_k up to {MAX_PACKED_GROUP};"
            f" got {nheads} / {nheads_k}.")
    return nheads, nheads_k, head_dim_qk


def check_rotary(rotary_cos, rotary_sin, rotary_interleaved, rotary_k, head_dim, min_len):
    """Validates the RoPE arguments (rotary.py:27-215 of the reference: full-head
    tables (seqlen_ro, head_dim / 2) in bf16 or f32); True when tables are given."""
    if type(rotary_interleaved) is not bool:
        raise ValueError("rotary_interleaved must be a static bool.")
    if type(rotary_k) is not bool:
        raise ValueError("rotary_k must be a static bool.")
    if (rotary_cos is None) != (rotary_sin is None):
        raise ValueError("rotary_cos and rotary_sin must be provided together.")
    if rotary_cos is None:
        if not rotary_k:
            raise ValueError("rotary_k=False needs rotary_cos and rotary_sin.")
        return False
    cos_shape, sin_shape = _arrays.shape(rotary_cos), _arrays.shape(rotary_sin)
    if len(cos_shape) != 2 or tuple(sin_shape) != tuple(cos_shape):
        raise ValueError("rotary_cos and rotary_sin must have the same 2-D shape.")
    if 2 * cos_shape[1] != head_dim:
        raise ValueError(
            f"rotary_dim ({2 * cos_shape[1]}) must equal head_dim ({head_dim});"
            " partial rotary is not supported.")
    names = (_arrays.dtype_name(rotary_cos.dtype), _arrays.dtype_name(rotary_sin.dtype))
    if names[0] != names[1] or names[0] not in ("bfloat16", "float32"):
        raise ValueError("rotary_cos and rotary_sin must share Q's dtype or be float32.")
    if cos_shape[0] < min_len:
        raise ValueError("rotary table is shorter than the KV sequence bound.")
    return True


def rotary_operand(rotary_cos, rotary_sin, rotary_interleaved, rotary_k, device):
    """(cos, sin, interleaved, rotate_k) with the tables on the device."""
    return (_arrays.to_device(rotary_cos, device).contiguous(),
            _arrays.to_device(rotary_sin, device).contiguous(), rotary_interleaved, rotary_k)


def packed_attention_device(q, k, v, cu_seqlens_q, cu_seqlens_k, *, nheads, nheads_k, total_q,
                            total_k, token_major, max_seqlen_q, softmax_scale, causal, window_left,
                            softcap, return_lse, sinks, sink_period=0, rotary=None, window_right=0):
    """Launches fw_attention_packed on contiguous CUDA tensors.  q is (nheads,
    total_q, d) or, token-major, (total_q, nheads, d); k / v likewise with
    nheads_k and total_k.  Returns (out shaped like q, lse (nheads, total_q) or
    None)."""
    device = q.device
    out = _arrays.empty_like(q)
    lse = _arrays.empty((nheads, total_q), "float32", device) if return_lse else None
    if total_q == 0:
        return out, lse
    if total_k == 0:
        out.zero_()
        if lse is not None:
            lse.fill_(float("-inf"))
        return out, lse
    batch = cu_seqlens_q.shape[0] - 1
    args = _native.FwPrefillArgs(
        q=q.data_ptr(), out=out.data_ptr(), lse=_arrays.data_ptr(lse), kv_cache=k.data_ptr(),
        v_packed=v.data_ptr(), cu_seqlens_q=cu_seqlens_q.data_ptr(), cu_seqlens_k=cu_seqlens_k.data_ptr(),
        sinks=_arrays.data_ptr(sinks), workspace=0, workspace_bytes=0, batch=batch, total_q=total_q,
        total_k=total_k, max_seqlen_q=int(max_seqlen_q), nheads=nheads, nheads_k=nheads_k,
        head_dim=q.shape[-1], kv_dtype=_native.DTYPE_CODE["bfloat16"], causal=int(bool(causal)),
        window_left=-1 if window_left is None else int(window_left), softmax_scale=float(softmax_scale),
        softcap=float(softcap), token_major=int(bool(token_major)), kv_token_major=int(bool(token_major)),
        sink_period=int(sink_period), window_right=int(window_right))
    if rotary is not None:
        cos, sin, interleaved, rotate_k = rotary
        args.rotary_cos, args.rotary_sin = cos.data_ptr(), sin.data_ptr()
        args.rotary_len = cos.shape[0]
        args.rotary_interleaved = int(bool(interleaved))
        args.rotary_bf16 = int(_arrays.dtype_name(cos.dtype) == "bfloat16")
        args.rotary_k = int(bool(rotate_k))
    lib = _native.library()
    stream = _native.current_stream(device)
    nbytes = lib.fw_attention_packed_workspace_bytes(ctypes.byref(args))
    if nbytes == 0:
        _native.check(lib.fw_attention_packed(ctypes.byref(args), stream))
        raise RuntimeError(_native.last_error())
    scratch = _native.workspace(device, nbytes)
    args.workspace, args.workspace_bytes = scratch.data_ptr(), scratch.numel()
    _native.check(lib.fw_attention_packed(ctypes.byref(args), stream))
    _native.raise_on_status(scratch, device)
    return out, lse


def packed_window(window_size, causal):
    """(left or None, causal flag, positive right reach or 0) for the kernel."""
    left, right = resolve_window(window_size, bool(causal))
    return left, right == 0, (right if right else 0)


def flash_attn_func(
    q,
    k,
    v,
    dropout_p=0.0,
    softmax_scale=None,
    causal=False,
    window_size=(-1, -1),
    attention_chunk=None,
    softcap=0.0,
    alibi_slopes=None,
    deterministic=False,
    return_attn_probs=False,
    return_softmax_lse=False,
    interpret=False,
    head_dim=None,
    token_major=False,
    *,
    rotary_cos=None,
    rotary_sin=None,
    rotary_interleaved=False,
    rotary_k=True,
    heads_outer_fold=False,
    learnable_sink=None,
):
    """flash_attn.flash_attn_func, forward only.

    Head-major (default): q (batch, nheads, seqlen_q, headdim), k / v (batch,
    nheads_k, seqlen_k, headdim), out like q, headdim 64, 128 or 256.  Token-major
    (token_major=True): the heads fused into the last axis, (batch, seqlen,
    nheads * head_dim), with head_dim= given.  All bfloat16; nheads / nheads_k up to 128.
    causal is bottom-right aligned: query i attends key j iff j <= i + seqlen_k -
    seqlen_q; window_size=(left, right) bounds the reach either side of that
    diagonal.  Rows with no
    reachable key return out = 0 and lse = -inf (or the sink).
    return_softmax_lse adds lse (batch, nheads, seqlen_q) float32, natural log.
    softcap > 0 applies tanh(scale * q k^T / softcap) * softcap.  rotary_cos /
    rotary_sin: full-head RoPE tables (seqlen_ro, headdim / 2), q's dtype or float32; K
    is rotated at positions 0..seqlen_k - 1 (unless rotary_k=False) and Q from
    seqlen_k - seqlen_q on.  learnable_sink: (nheads,) sink logits joining the
    softmax denominator.  Unlike the reference, seqlen_k needs no alignment.
    """
    del interpret
    window_size = check_common_kwargs(
        window_size, dropout_p=dropout_p, softcap=softcap, alibi_slopes=alibi_slopes,
        deterministic=deterministic, return_attn_probs=return_attn_probs)
    if attention_chunk is not None:
        raise NotImplementedError("attention_chunk is not implemented.")
    if type(heads_outer_fold) is not bool:
        raise TypeError("heads_outer_fold must be a bool.")
    if heads_outer_fold:
        raise NotImplementedError("heads_outer_fold is not built; pass (batch, nheads, seqlen, headdim).")
    expected_rank = 3 if token_major else 4
    nheads, nheads_k, head_dim_qk = parse_qkv(
        q, k, v, head_dim, token_major, expected_rank, "batch, nheads, seqlen, headdim")
    batch = q.shape[0]
    seq_axis = 1 if token_major else 2
    seqlen_q, seqlen_k = q.shape[seq_axis], k.shape[seq_axis]
    left, is_causal, right = packed_window(window_size, causal)
    has_rotary = check_rotary(rotary_cos, rotary_sin, rotary_interleaved, rotary_k, head_dim_qk, seqlen_k)
    if has_rotary and seqlen_q > seqlen_k:
        raise ValueError("fused RoPE rotates Q from seqlen_k - seqlen_q on, so seqlen_q <= seqlen_k.")
    device = _arrays.pick_device(q, k)
    rotary = (rotary_operand(rotary_cos, rotary_sin, rotary_interleaved, rotary_k, device)
              if has_rotary else None)
    sinks = sinks_operand(learnable_sink, nheads, device)
    scale = 1.0 / math.sqrt(head_dim_qk) if softmax_scale is None else float(softmax_scale)
    q_dev, k_dev, v_dev = (_arrays.to_device(x, device).contiguous() for x in (q, k, v))
    if token_major:
        # packed tokens (batch * seqlen, nheads, d): one sequence per batch row
        cu_q = _arrays.arange_scaled(batch + 1, seqlen_q, device)
        cu_k = _arrays.arange_scaled(batch + 1, seqlen_k, device)
        out, lse = packed_attention_device(
            q_dev.view(batch * seqlen_q, nheads, head_dim_qk), k_dev.view(batch * seqlen_k, nheads_k, head_dim_qk),
            v_dev.view(batch * seqlen_k, nheads_k, head_dim_qk), cu_q, cu_k, nheads=nheads, nheads_k=nheads_k,
            total_q=batch * seqlen_q, total_k=batch * seqlen_k, token_major=True, max_seqlen_q=max(seqlen_q, 1),
            softmax_scale=scale, causal=is_causal, window_left=left, softcap=softcap,
            return_lse=return_softmax_lse, sinks=sinks, rotary=rotary, window_right=right)
        out = out.view(q_dev.shape)
        if lse is not None:
            lse = _arrays.heads_first_to_batch_first(lse, nheads, batch, seqlen_q)
    else:
        # the batch folds into the head axis: batch * nheads heads over one sequence
        cu_q = _arrays.int32_array([0, seqlen_q], device)
        cu_k = _arrays.int32_array([0, seqlen_k], device)
        out, lse = packed_attention_device(
            q_dev.view(batch * nheads, seqlen_q, head_dim_qk), k_dev.view(batch * nheads_k, seqlen_k, head_dim_qk),
            v_dev.view(batch * nheads_k, seqlen_k, head_dim_qk), cu_q, cu_k, nheads=batch * nheads,
            nheads_k=batch * nheads_k, total_q=seqlen_q, total_k=seqlen_k, token_major=False,
            max_seqlen_q=max(seqlen_q, 1), softmax_scale=scale, causal=is_causal, window_left=left,
            softcap=softcap, return_lse=return_softmax_lse, sinks=sinks, sink_period=nheads, rotary=rotary,
            window_right=right)
        out = out.view(q_dev.shape)
        if lse is not None:
            lse = lse.view(batch, nheads, seqlen_q)
    if return_softmax_lse:
        return _arrays.like(out, q), _arrays.like(lse, q)
    return _arrays.like(out, q)


def packed_varlen_attn(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, *, softmax_scale,
                       causal, window_size, softcap, return_softmax_lse, head_dim, token_major,
                       rotary_cos, rotary_sin, rotary_interleaved, rotary_k, learnable_sink):
    """The cu_seqlens_k branch of flash_attn_varlen_func (prefill.py:818-963 of
    the reference): q (nheads, total_q, d), k / v (nheads_k, total_k, d), or
    token-major (total, nheads * head_dim)."""
    expected_rank = 2 if token_major else 3
    nheads, nheads_k, head_dim_qk = parse_qkv(
        q, k, v, head_dim, token_major, expected_rank, "nheads, total tokens, headdim")
    token_axis = 0 if token_major else 1
    total_q, total_k = q.shape[token_axis], k.shape[token_axis]
    if cu_seqlens_q is None or cu_seqlens_k is None:
        raise ValueError("packed K/V needs cu_seqlens_q and cu_seqlens_k.")
    shape_q, shape_k = tuple(_arrays.shape(cu_seqlens_q)), tuple(_arrays.shape(cu_seqlens_k))
    if len(shape_q) != 1 or shape_q != shape_k or shape_q[0] < 2:
        raise ValueError(
            "cu_seqlens_q and cu_seqlens_k must be equal-shaped 1-D arrays; got"
            f" cu_seqlens_q.shape={shape_q}, cu_seqlens_k.shape={shape_k}.")
    for arg_name, bound in (("max_seqlen_q", max_seqlen_q), ("max_seqlen_k", max_seqlen_k)):
        if not isinstance(bound, int):
            raise ValueError(
                f"{arg_name} must be a concrete int (it picks the kernel's block sizes); pass a"
                " static bucket bound, not a traced value.")
        if bound <= 0:
            raise ValueError(f"{arg_name} must be positive; got {bound}.")
    left, is_causal, right = packed_window(window_size, causal)
    has_rotary = check_rotary(rotary_cos, rotary_sin, rotary_interleaved, rotary_k, head_dim_qk, max_seqlen_k)
    device = _arrays.pick_device(q, k)
    rotary = (rotary_operand(rotary_cos, rotary_sin, rotary_interleaved, rotary_k, device)
              if has_rotary else None)
    sinks = sinks_operand(learnable_sink, nheads, device)
    scale = 1.0 / math.sqrt(head_dim_qk) if softmax_scale is None else float(softmax_scale)
    q_dev, k_dev, v_dev = (_arrays.to_device(x, device).contiguous() for x in (q, k, v))
    if token_major:
        q_dev = q_dev.view(total_q, nheads, head_dim_qk)
        k_dev, v_dev = (x.view(total_k, nheads_k, head_dim_qk) for x in (k_dev, v_dev))
    out, lse = packed_attention_device(
        q_dev, k_dev, v_dev, _arrays.to_device(cu_seqlens_q, device, dtype="int32").contiguous(),
        _arrays.to_device(cu_seqlens_k, device, dtype="int32").contiguous(), nheads=nheads,
        nheads_k=nheads_k, total_q=total_q, total_k=total_k, token_major=token_major,
        max_seqlen_q=max_seqlen_q, softmax_scale=scale, causal=is_causal, window_left=left,
        softcap=softcap, return_lse=return_softmax_lse, sinks=sinks, rotary=rotary, window_right=right)
    if token_major:
        out = out.view(total_q, nheads * head_dim_qk)
    if return_softmax_lse:
        return _arrays.like(out, q), _arrays.like(lse, q)
    return _arrays.like(out, q)
