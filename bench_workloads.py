"""Seeded synthetic workload sizing for bench.py and the tests.

The serving benchmark configurations are described by shape and value
distribution only (standard-normal bf16 values, uniform integer lengths, a
random permutation of pool pages as the block table), so seeded draws stand in
for them.  Table construction follows the reference's own benchmark generator
(benchmarks/softmax_attention/kvcache_scenarios.py:413-461 of the reference
project): each request's table row lists its pages and repeats its last page in
the unused tail entries.  Byte and FLOP accounting follows the same file
(:313-348, :1198).
"""

from __future__ import annotations

import math

import numpy as np


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
