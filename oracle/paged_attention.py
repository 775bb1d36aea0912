"""CPU oracle for FlyWheel's paged-KV softmax attention path (NumPy + ml_dtypes).

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is
compared against; nothing in the shipped package imports it.  Only the test
suite, the smoke check and the benchmark's CPU-baseline leg may call it.

It restates, in plain NumPy, the semantics of the reference's own NumPy test
oracle and layout helpers (paths are relative to the reference project):

* merged cache row order ``[k0, v0, k1, v1, ...]`` with an odd fp8 head count
  padded by one zero head: ``flywheel_tpu/softmax_attention/kv_layout.py:39-46,
  67-70`` and ``tests/softmax_attention/util.py:40-59``;
* append of new tokens at ``cache_seqlens + t`` through the block table:
  ``tests/softmax_attention/test_paged.py:80-95`` and
  ``flywheel_tpu/softmax_attention/kernels/kv_append.py:56-73``;
* ragged attention with causal / left-window / softcap / sinks:
  ``tests/softmax_attention/test_paged.py:98-206``;
* contiguous-pair decode: ``tests/softmax_attention/test_regression.py:901-970``;
* the log-sum-exp merge of two partial states:
  ``patches/tpu-inference.patch:7174-7186``.

Parity pin: ``tests/golden/make_golden.py`` executes the reference's own
``append_to_pages`` / ``ragged_reference`` source (pure NumPy) on seeded inputs
and stores the results; ``tests/test_oracle_golden.py`` checks this module
against those files, and against the reference tests' deterministic
known-answer constructions.
"""

from __future__ import annotations

import math

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)
E4M3 = np.dtype(ml_dtypes.float8_e4m3fn)
E5M2 = np.dtype(ml_dtypes.float8_e5m2)
CACHE_DTYPES = (BF16, E4M3, E5M2)


# ----------------------------------------------------------------------------
# Layout (kv_layout.py:67-70; tests/softmax_attention/util.py:40-59)
# ----------------------------------------------------------------------------
def kv_heads_per_word(dtype) -> int:
    """KV heads whose (K, V) pair fills one 32-bit word per lane: 1 for bf16,
    2 for fp8 (kv_layout.py:57-64)."""
    return (4 // np.dtype(dtype).itemsize) // 2


def merged_cache_heads(num_kv_heads: int, dtype) -> int:
    """Head rows of one merged-cache token (kv_layout.py:67-70)."""
    per_word = kv_heads_per_word(dtype)
    return 2 * (-(-num_kv_heads // per_word) * per_word)


def merge_kv_heads(k: np.ndarray, v: np.ndarray) -> np.ndarray:
    """(..., nheads_k, d) K and V rows -> merged (..., cache_heads, d) rows,
    each head's K row then its V row, an odd fp8 head count padded by one zero
    head (tests/softmax_attention/util.py:40-52).  Moves bits, never values."""
    assert k.shape == v.shape and k.dtype == v.dtype
    *leading, nheads_k, d = k.shape
    pad = merged_cache_heads(nheads_k, k.dtype) // 2 - nheads_k
    bits = np.dtype(f"uint{8 * k.dtype.itemsize}")
    kb, vb = k.view(bits), v.view(bits)
    if pad:
        zeros = np.zeros((*leading, pad, d), bits)
        kb = np.concatenate([kb, zeros], axis=-2)
        vb = np.concatenate([vb, zeros], axis=-2)
    merged = np.stack([kb, vb], axis=-2).reshape(*leading, -1, d)
    return np.ascontiguousarray(merged).view(k.dtype)


def split_kv_heads(kv: np.ndarray, nheads_k: int):
    """merge_kv_heads' inverse (tests/softmax_attention/util.py:55-59)."""
    *leading, cache_heads, d = kv.shape
    pairs = kv.reshape(*leading, cache_heads // 2, 2, d)
    return pairs[..., :nheads_k, 0, :], pairs[..., :nheads_k, 1, :]


# ----------------------------------------------------------------------------
# Append (test_paged.py:80-95; kv_append.py:56-73, 113)
# ----------------------------------------------------------------------------
def append_to_pool(pool, k, v, cu_seqlens_q, cache_seqlens, block_table,
                   nheads_k=None, num_active=None):
    """A copy of the merged pool with request r's tokens [cu[r], cu[r+1])
    written at positions cache_seqlens[r] + t through block_table.  Whole
    merged rows are written (the fp8 pad head as zeros); every other byte is
    unchanged.  Requests >= num_active append nothing."""
    pool = pool.copy()
    if k is None:
        return pool
    cu = np.asarray(cu_seqlens_q).astype(np.int64)
    lengths = np.asarray(cache_seqlens).astype(np.int64)
    table = np.asarray(block_table)
    page_size = pool.shape[1]
    rows = merge_kv_heads(np.asarray(k), np.asarray(v))
    assert rows.shape[-2] == pool.shape[2], (rows.shape, pool.shape)
    active = len(lengths) if num_active is None else int(num_active)
    for seq in range(min(active, len(lengths))):
        start, end = int(cu[seq]), int(cu[seq + 1])
        positions = lengths[seq] + np.arange(end - start)
        pages = table[seq, positions // page_size]
        pool[pages, positions % page_size] = rows[start:end]
    return pool


def write_kv_cache_pages(pool, k, v, slices, num_slices):
    """A copy of the merged pool with the slice-table pieces written: column
    j < num_slices of slices (i32[3, n]) is (cache_row_start, new_row_start,
    length) in rows of the flat (pages * page_size) view and of k / v
    (flywheel_tpu/softmax_attention/page.py:35-73; the reference's own check is
    tests/softmax_attention/test_page.py:32-69)."""
    pool = pool.copy()
    flat = pool.reshape(-1, *pool.shape[2:])
    rows = merge_kv_heads(np.asarray(k), np.asarray(v))
    slices = np.asarray(slices)
    for column in range(int(np.asarray(num_slices).reshape(-1)[0])):
        cache_row, new_row, length = (int(x) for x in slices[:, column])
        flat[cache_row:cache_row + length] = rows[new_row:new_row + length]
    return pool


def append_contiguous(k_cache, v_cache, k, v, cache_seqlens, cache_batch_idx,
                      num_active=None):
    """Contiguous pair: k_cache[cache_batch_idx[b], cache_seqlens[b]] = k[b, 0]
    (tests/softmax_attention/test_regression.py:1093-1096)."""
    k_cache, v_cache = k_cache.copy(), v_cache.copy()
    if k is None:
        return k_cache, v_cache
    lengths = np.asarray(cache_seqlens)
    active = len(lengths) if num_active is None else int(num_active)
    for b in range(min(active, len(lengths))):
        row = int(cache_batch_idx[b])
        k_cache[row, int(lengths[b])] = k[b, 0]
        v_cache[row, int(lengths[b])] = v[b, 0]
    return k_cache, v_cache


# ----------------------------------------------------------------------------
# Attention core (test_paged.py:98-206)
# ----------------------------------------------------------------------------
def attend_rows(q, keys, values, *, total, causal, window_left, softcap,
                scale, sinks, row_chunk=256, window_right=None):
    """f32 softmax attention of (q_len, heads, d) query rows against one
    request's (total, kv_heads, d) keys/values.  Row r sits on the bottom-right
    diagonal ``total - q_len + r``; causal hides keys past it, window_left
    hides keys more than window_left before it; softcap maps a scaled score s
    to softcap * tanh(s / softcap) before masking; exp(sinks[h]) joins head h's
    denominator.  Returns out (q_len, heads, d) and natural-log lse
    (heads, q_len); rows that see no key give out 0, lse -inf (or the sink)."""
    q_len, heads, d = q.shape
    kv_heads = keys.shape[1]
    group = heads // kv_heads
    out = np.zeros((q_len, heads, values.shape[-1]), np.float32)
    lse = np.full((heads, q_len), -np.inf, np.float32)
    if sinks is not None:
        head_sinks = np.asarray(sinks, np.float32).reshape(kv_heads, group, 1)
    if q_len == 0:
        return out, lse
    positions = np.arange(total)
    kt = np.ascontiguousarray(keys[:total].transpose(1, 2, 0))    # (hk, d, total)
    vt = np.ascontiguousarray(values[:total].transpose(1, 0, 2))  # (hk, total, d)
    for lo in range(0, q_len, row_chunk):
        rows = np.arange(lo, min(lo + row_chunk, q_len))
        qc = q[rows].reshape(len(rows), kv_heads, group, d).transpose(1, 0, 2, 3)
        qc = np.ascontiguousarray(qc).reshape(kv_heads, len(rows) * group, d)
        raw = np.matmul(qc, kt).reshape(kv_heads, len(rows), group, total) * scale
        scores = softcap * np.tanh(raw / softcap) if softcap else raw
        diagonal = (total - q_len + rows)[:, None]
        if causal:
            visible = positions[None] <= diagonal
        else:
            visible = np.ones((len(rows), total), bool)
        if window_left is not None:
            visible = visible & (positions[None] >= diagonal - window_left)
        if window_right is not None and not causal:
            visible = visible & (positions[None] <= diagonal + window_right)
        seen = visible.any(axis=-1)                                # (rows,)
        scores = np.where(visible[None, :, None, :], scores, -np.inf)
        anchor = np.where(
            seen[None, :, None, None],
            scores.max(axis=-1, keepdims=True, initial=-np.inf), 0.0)
        if sinks is not None:
            sink = head_sinks[:, None]                             # (hk,1,g,1)
            anchor = np.where(seen[None, :, None, None],
                              np.maximum(anchor, sink), sink)
            anchor = np.where(np.isneginf(anchor), 0.0, anchor)
        weights = np.exp(scores - anchor)
        denom = weights.sum(axis=-1, keepdims=True)
        if sinks is not None:
            denom = denom + np.exp(sink - anchor)
        probs = weights / np.where(denom > 0, denom, 1)
        result = np.matmul(
            probs.reshape(kv_heads, len(rows) * group, total), vt
        ).reshape(kv_heads, len(rows), group, -1).transpose(1, 0, 2, 3)
        result = result.reshape(len(rows), heads, -1)
        out[rows] = np.where(seen[:, None, None], result, 0)
        with np.errstate(divide="ignore"):
            row_lse = anchor + np.log(denom)                       # (hk,rows,g,1)
        row_lse = row_lse[..., 0].transpose(1, 0, 2).reshape(len(rows), heads)
        if sinks is None:
            row_lse = np.where(seen[:, None], row_lse, -np.inf)
        lse[:, rows] = row_lse.T
    return out, lse


def gather_request(pool, table_row, total, nheads_k, k_descale=1.0,
                   v_descale=1.0):
    """Logical f32 (total, nheads_k, d) keys and values of one request: pool
    rows gathered in position order through the block table row, split into K
    and V planes and multiplied by the per-tensor descales (an fp8 pool stores
    K / k_descale: tests/softmax_attention/test_prefill.py:614-625)."""
    page_size = pool.shape[1]
    positions = np.arange(total)
    pages = np.asarray(table_row)[positions // page_size]
    rows = pool[pages, positions % page_size]
    k_rows, v_rows = split_kv_heads(rows, nheads_k)
    return (k_rows.astype(np.float32) * np.float32(k_descale),
            v_rows.astype(np.float32) * np.float32(v_descale))


def ragged_paged_attention(q, pool, cu_seqlens_q, seqused_k, block_table, *,
                           nheads_k, causal, window_left=None, softcap=0.0,
                           softmax_scale=None, sinks=None, k_descale=1.0,
                           v_descale=1.0, num_active=None):
    """Read-only attention of packed token-major q (total_q, heads, d) over a
    merged pool that already holds every request's seqused_k tokens
    (flash_attn_varlen_func with block_table; test_paged.py:98-206 with k=None).
    Rows past cu_seqlens_q[num_active] are padding: out 0, lse -inf.
    Returns out (total_q, heads, d) f32 and lse (heads, total_q) f32."""
    q32 = np.asarray(q).astype(np.float32)
    total_q, heads, d = q32.shape
    cu = np.asarray(cu_seqlens_q).astype(np.int64)
    seqused = np.asarray(seqused_k).astype(np.int64)
    batch = len(cu) - 1
    active = batch if num_active is None else int(num_active)
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    out = np.zeros((total_q, heads, d), np.float32)
    lse = np.full((heads, total_q), -np.inf, np.float32)
    for seq in range(min(active, batch)):
        start, end = int(cu[seq]), int(cu[seq + 1])
        if end <= start:
            continue
        total = int(seqused[seq])
        keys, values = gather_request(pool, np.asarray(block_table)[seq], total,
                                      nheads_k, k_descale, v_descale)
        o, l = attend_rows(q32[start:end], keys, values, total=total,
                           causal=causal, window_left=window_left,
                           softcap=softcap, scale=scale, sinks=sinks)
        out[start:end] = o
        lse[:, start:end] = l
    return out, lse


def kvcache_paged(q, pool, k, v, cache_seqlens, block_table, *, nheads_k,
                  cu_seqlens_q=None, num_active=None, causal=False,
                  window_left=None, softcap=0.0, softmax_scale=None,
                  sinks=None, k_descale=1.0, v_descale=1.0):
    """flash_attn_with_kvcache on the paged merged cache: append k/v (when
    given) after each request's cache_seqlens, then attend the updated cache.

    q is (batch, seqlen_q, heads, d), or packed (total_q, heads, d) with
    cu_seqlens_q.  Returns (out in q's shape, f32; lse (batch, heads, seqlen_q)
    or packed (heads, total_q); updated pool)."""
    q = np.asarray(q)
    packed = cu_seqlens_q is not None
    if packed:
        cu = np.asarray(cu_seqlens_q).astype(np.int64)
        batch = len(cu) - 1
        q_rows, k_rows, v_rows = q, k, v
    else:
        batch, seqlen_q = q.shape[:2]
        cu = np.arange(batch + 1, dtype=np.int64) * seqlen_q
        q_rows = q.reshape(-1, *q.shape[2:])
        k_rows = None if k is None else np.asarray(k).reshape(-1, *k.shape[2:])
        v_rows = None if v is None else np.asarray(v).reshape(-1, *v.shape[2:])
    lengths = np.broadcast_to(np.asarray(cache_seqlens), (batch,)).astype(np.int64)
    new_pool = append_to_pool(pool, k_rows, v_rows, cu, lengths, block_table,
                              nheads_k, num_active)
    seqused = lengths + (np.diff(cu) if k is not None else 0)
    out, lse = ragged_paged_attention(
        q_rows, new_pool, cu, seqused, block_table, nheads_k=nheads_k,
        causal=causal, window_left=window_left, softcap=softcap,
        softmax_scale=softmax_scale, sinks=sinks, k_descale=k_descale,
        v_descale=v_descale, num_active=num_active)
    if not packed:
        out = out.reshape(q.shape)
        lse = lse.reshape(q.shape[2], batch, seqlen_q).transpose(1, 0, 2)
    return out, lse, new_pool


def kvcache_contiguous(q, k_cache, v_cache, k, v, cache_seqlens,
                       cache_batch_idx=None, *, num_active=None, causal=False,
                       window_left=None, softcap=0.0, softmax_scale=None,
                       sinks=None):
    """Single-token decode on the contiguous (batch_cache, capacity, nheads_k,
    d) K/V pair (test_regression.py:901-970): append k/v[b, 0] at
    cache_seqlens[b] of cache row cache_batch_idx[b], attend positions
    < cache_seqlens[b] + new.  Returns (out (batch, 1, heads, d) f32,
    lse (batch, heads, 1), k_cache, v_cache)."""
    q = np.asarray(q)
    batch, seqlen_q, heads, d = q.shape
    assert seqlen_q == 1
    lengths = np.broadcast_to(np.asarray(cache_seqlens), (batch,)).astype(np.int64)
    rows = (np.arange(batch) if cache_batch_idx is None
            else np.asarray(cache_batch_idx).astype(np.int64))
    k_cache, v_cache = append_contiguous(k_cache, v_cache, k, v, lengths, rows,
                                         num_active)
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    out = np.zeros(q.shape, np.float32)
    lse = np.full((batch, heads, 1), -np.inf, np.float32)
    active = batch if num_active is None else int(num_active)
    for b in range(min(active, batch)):
        total = int(lengths[b]) + (0 if k is None else 1)
        keys = k_cache[rows[b], :total].astype(np.float32)
        values = v_cache[rows[b], :total].astype(np.float32)
        o, l = attend_rows(q[b].astype(np.float32), keys, values, total=total,
                           causal=causal, window_left=window_left,
                           softcap=softcap, scale=scale, sinks=sinks)
        out[b], lse[b] = o, l
    return out, lse, k_cache, v_cache


def rotate_packed_q(q, cos, sin, cu_seqlens_q, seqused_k, interleaved=False):
    """RoPE on packed token-major q (total_q, heads, d): token t of request r at
    position seqused_k[r] - len_q(r) + t, f32 rotation rounded once to q's
    dtype; rows outside every request and positions past the table stay as they
    are (tests/softmax_attention/util.py:105-150 of the reference; positions:
    flywheel_tpu/softmax_attention/prefill.py:494-498)."""
    q = np.asarray(q)
    out = q.copy()
    cu = np.asarray(cu_seqlens_q).astype(np.int64)
    cos32, sin32 = np.asarray(cos).astype(np.float32), np.asarray(sin).astype(np.float32)
    for r in range(len(cu) - 1):
        start, end = int(cu[r]), int(cu[r + 1])
        if end <= start:
            continue
        pos = int(seqused_k[r]) - (end - start) + np.arange(end - start)
        ok = (pos >= 0) & (pos < cos32.shape[0])
        rows = np.arange(start, end)[ok]
        c, s_ = cos32[pos[ok]][:, None, :], sin32[pos[ok]][:, None, :]
        x = q[rows].astype(np.float32)
        if interleaved:
            x1, x2 = x[..., 0::2], x[..., 1::2]
            y = np.stack((x1 * c - x2 * s_, x1 * s_ + x2 * c), axis=-1).reshape(x.shape)
        else:
            half = x.shape[-1] // 2
            x1, x2 = x[..., :half], x[..., half:]
            y = np.concatenate((x1 * c - x2 * s_, x1 * s_ + x2 * c), axis=-1)
        out[rows] = y.astype(q.dtype)
    return out


# ----------------------------------------------------------------------------
# Packed (non-paged) K/V: flash_attn_varlen_func with cu_seqlens_k and
# flash_attn_func.  Semantics of tests/softmax_attention/util.py:181-273 of the
# reference (attention_ref: f32, bottom-right aligned causal / window masks on
# each sequence's own lengths, sink as one more logit, rows with no visible key
# out 0 / lse -inf or the sink).
# That function is jax.numpy code and cannot run here, so these two restate it
# through attend_rows, which the golden vectors pin.
# ----------------------------------------------------------------------------
def packed_varlen_attention(q, k, v, cu_seqlens_q, cu_seqlens_k, *, causal=False,
                            window_left=None, softcap=0.0, softmax_scale=None,
                            sinks=None, window_right=None):
    """q (total_q, heads, d), k / v (total_k, kv_heads, d) token-major.  Returns
    out (total_q, heads, d) f32 and lse (heads, total_q); rows outside every
    sequence give out 0, lse -inf."""
    q32 = np.asarray(q).astype(np.float32)
    k32, v32 = np.asarray(k).astype(np.float32), np.asarray(v).astype(np.float32)
    total_q, heads, d = q32.shape
    cu_q = np.asarray(cu_seqlens_q).astype(np.int64)
    cu_k = np.asarray(cu_seqlens_k).astype(np.int64)
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    out = np.zeros((total_q, heads, d), np.float32)
    lse = np.full((heads, total_q), -np.inf, np.float32)
    for seq in range(len(cu_q) - 1):
        qs, qe, ks, ke = int(cu_q[seq]), int(cu_q[seq + 1]), int(cu_k[seq]), int(cu_k[seq + 1])
        if qe <= qs:
            continue
        o, l = attend_rows(q32[qs:qe], k32[ks:ke], v32[ks:ke], total=ke - ks, causal=causal,
                           window_left=window_left, softcap=softcap, scale=scale, sinks=sinks,
                           window_right=window_right)
        out[qs:qe] = o
        lse[:, qs:qe] = l
    return out, lse


def dense_attention(q, k, v, **kwargs):
    """q (batch, seqlen_q, heads, d), k / v (batch, seqlen_k, kv_heads, d).
    Returns out like q (f32) and lse (batch, heads, seqlen_q)."""
    q, k, v = np.asarray(q), np.asarray(k), np.asarray(v)
    batch, seqlen_q, heads, d = q.shape
    seqlen_k = k.shape[1]
    out, lse = packed_varlen_attention(
        q.reshape(batch * seqlen_q, heads, d), k.reshape(batch * seqlen_k, -1, d),
        v.reshape(batch * seqlen_k, -1, d), np.arange(batch + 1) * seqlen_q,
        np.arange(batch + 1) * seqlen_k, **kwargs)
    return out.reshape(q.shape), lse.reshape(heads, batch, seqlen_q).transpose(1, 0, 2)


# ----------------------------------------------------------------------------
# LSE merge (patches/tpu-inference.patch:7174-7186)
# ----------------------------------------------------------------------------
def merge_states(outs, lses, sinks=None):
    """Merge sink-free partial attention states over disjoint key sets.

    outs: (parts, ..., d) normalised partial outputs; lses: (parts, ...) their
    natural-log lse (-inf for an empty part).  sinks, broadcastable to lses[0],
    joins the denominator once.  All parts empty -> out 0, lse -inf (or the
    sink)."""
    outs = np.asarray(outs, np.float32)
    lses = np.asarray(lses, np.float32)
    terms = lses if sinks is None else np.concatenate(
        [lses, np.broadcast_to(np.asarray(sinks, np.float32), lses[:1].shape)])
    top = terms.max(axis=0)
    safe = np.where(np.isneginf(top), 0.0, top)
    weights = np.exp(lses - safe)
    denom = np.exp(terms - safe).sum(axis=0)
    safe_denom = np.where(denom == 0, 1.0, denom)
    out = (outs * weights[..., None]).sum(axis=0) / safe_denom[..., None]
    with np.errstate(divide="ignore"):
        lse = np.where(denom == 0, -np.inf, safe + np.log(safe_denom))
    return out.astype(np.float32), lse.astype(np.float32)


# ----------------------------------------------------------------------------
# fp8 helpers (tests/softmax_attention/test_prefill.py:535-537, 614-625)
# ----------------------------------------------------------------------------
def quantize_per_tensor(x, dtype, descale=None):
    """(stored, descale): stored = (x / descale) cast to the fp8 dtype, with
    descale = amax|x| / finfo(dtype).max unless given."""
    x = np.asarray(x, np.float32)
    if descale is None:
        amax = float(np.abs(x).max()) if x.size else 1.0
        descale = max(amax, 1e-12) / float(ml_dtypes.finfo(dtype).max)
    limit = float(ml_dtypes.finfo(dtype).max)
    stored = np.clip(x / np.float32(descale), -limit, limit).astype(dtype)
    return stored, np.float32(descale)
