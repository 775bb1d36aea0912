"""Seeded synthetic inputs for the paged-KV attention path.

The serving benchmark configurations are described by shape and value
distribution only (standard-normal bf16 values, uniform integer lengths, a
random permutation of pool pages as the block table), so seeded draws stand in
for them.  Value construction follows the reference's own benchmark generator
(benchmarks/softmax_attention/kvcache_scenarios.py:351-356, 413-461 of the
reference project): f32 standard-normal draws cast to the storage type; each
request's table row lists its pages and repeats its last page in the unused
tail entries.

Two generators: `host_case` builds everything in NumPy (small cases, fed to the
CPU checker too); `device_decode_case` fills large pools directly on the GPU.
"""

from __future__ import annotations

import dataclasses
import math

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)
E4M3 = np.dtype(ml_dtypes.float8_e4m3fn)
E5M2 = np.dtype(ml_dtypes.float8_e5m2)


def merge_rows(k, v):
    """(..., hk, d) K and V -> merged (..., cache_heads, d) rows [k0, v0, ...];
    an odd fp8 head count gets one zero pad head."""
    *lead, hk, d = k.shape
    pad = (-hk) % (2 // k.dtype.itemsize) if k.dtype.itemsize == 1 else 0
    carrier = np.dtype(f"uint{8 * k.dtype.itemsize}")
    kb, vb = k.view(carrier), v.view(carrier)
    if pad:
        zeros = np.zeros((*lead, pad, d), carrier)
        kb, vb = np.concatenate([kb, zeros], -2), np.concatenate([vb, zeros], -2)
    return np.ascontiguousarray(
        np.stack([kb, vb], axis=-2).reshape(*lead, -1, d)).view(k.dtype)


@dataclasses.dataclass
class HostCase:
    q: np.ndarray            # (batch, q_len, hq, d) bf16
    pool: np.ndarray         # (pages, page_size, cache_heads, d) cache dtype
    k_new: np.ndarray        # (batch, q_len, hk, d) cache dtype
    v_new: np.ndarray
    cache_seqlens: np.ndarray
    block_table: np.ndarray
    k_descale: float
    v_descale: float
    nheads_k: int


def host_case(seed, *, lens, q_len=1, hq=8, hk=2, d=128, page_size=64,
              dtype=BF16, extra_pages=3, poison=False, bad_tail=False,
              max_pages=None) -> HostCase:
    """A small paged decode case.  lens are the cached lengths before the
    append.  poison fills every slot past a request's cached length with NaN
    (or the largest fp8 magnitude) so a kernel that reads past the valid length
    is caught; bad_tail writes -1 into the unused block-table entries."""
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, np.int32)
    batch = len(lens)
    pages_b = [max(1, math.ceil((int(n) + q_len) / page_size)) for n in lens]
    total_pages = sum(pages_b) + extra_pages
    perm = rng.permutation(total_pages)
    width = max_pages or max(pages_b) + 1
    table = np.zeros((batch, width), np.int32)
    cursor = 0
    for b, n in enumerate(pages_b):
        table[b, :n] = perm[cursor:cursor + n]
        table[b, n:] = -1 if bad_tail else table[b, n - 1]
        cursor += n

    def draw(shape):
        return rng.standard_normal(shape, dtype=np.float32)

    kf, vf = draw((total_pages, page_size, hk, d)), draw((total_pages, page_size, hk, d))
    knf, vnf = draw((batch, q_len, hk, d)), draw((batch, q_len, hk, d))
    if dtype == BF16:
        kd = vd = 1.0
        cast = lambda x, s: x.astype(BF16)
    else:
        limit = float(ml_dtypes.finfo(dtype).max)
        kd = float(np.abs(kf).max()) / limit
        vd = float(np.abs(vf).max()) / limit
        cast = lambda x, s: np.clip(x / np.float32(s), -limit, limit).astype(dtype)
    k_pages, v_pages = cast(kf, kd), cast(vf, vd)
    if poison:
        bad = np.float32(np.nan) if dtype == BF16 else np.float32(
            float(ml_dtypes.finfo(dtype).max))
        live = np.zeros((total_pages, page_size), bool)
        for b, n in enumerate(lens):
            pos = np.arange(int(n))
            live[table[b, pos // page_size], pos % page_size] = True
        k_pages[~live] = np.asarray(bad).astype(dtype)
        v_pages[~live] = np.asarray(bad).astype(dtype)
    return HostCase(
        q=draw((batch, q_len, hq, d)).astype(BF16), pool=merge_rows(k_pages, v_pages),
        k_new=cast(knf, kd), v_new=cast(vnf, vd), cache_seqlens=lens,
        block_table=table, k_descale=kd, v_descale=vd, nheads_k=hk)


def decode_kv_bytes(cache_seqlens, q_len, hk, d, itemsize, window_left=None):
    """Algorithmic KV bytes one decode step must read: visible keys x 2 x hk x d
    x itemsize (kv_bytes_read of the reference's benchmark,
    benchmarks/softmax_attention/kvcache_scenarios.py:313-325)."""
    total = np.asarray(cache_seqlens, np.int64) + q_len
    visible = total if window_left is None else np.minimum(total, window_left + q_len)
    return int(visible.sum()) * 2 * hk * d * itemsize


def prefill_flops(prefix, chunk, hq, d):
    """4 x causal (query, key) pairs x heads x head_dim (attn_flops of the
    reference's benchmark, kvcache_scenarios.py:332-348, 1198)."""
    prefix = np.asarray(prefix, np.int64)
    chunk = np.asarray(chunk, np.int64)
    pairs = int((chunk * prefix + chunk * (chunk + 1) // 2).sum())
    return 4 * pairs * hq * d


def paged_table(rng, lens, q_len, page_size, slack=0.10):
    """(block_table, pool_pages): pool sized to the pages in use plus `slack`,
    table rows a slice of one seeded permutation of pool pages, unused tail
    entries repeating the row's last page."""
    pages_b = np.maximum(1, -(-(np.asarray(lens, np.int64) + q_len) // page_size))
    pool_pages = int(math.ceil(float(pages_b.sum()) * (1.0 + slack)))
    perm = rng.permutation(pool_pages).astype(np.int32)
    width = int(pages_b.max()) + 1
    table = np.zeros((len(lens), width), np.int32)
    cursor = 0
    for b, n in enumerate(pages_b):
        n = int(n)
        table[b, :n] = perm[cursor:cursor + n]
        table[b, n:] = table[b, n - 1]
        cursor += n
    return table, pool_pages
