"""Small seeded paged-decode cases in NumPy for the parity tests and the smoke
check (fed to the CUDA path and to the CPU oracle alike).  Values follow the
reference's generators: f32 standard-normal draws cast to the storage type
(tests/softmax_attention/util.py:32-37 of the reference project)."""

from __future__ import annotations

import dataclasses
import math

import ml_dtypes
import numpy as np

from oracle import paged_attention as oracle

BF16, E4M3, E5M2 = oracle.BF16, oracle.E4M3, oracle.E5M2


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
        q=draw((batch, q_len, hq, d)).astype(BF16), pool=oracle.merge_kv_heads(k_pages, v_pages),
        k_new=cast(knf, kd), v_new=cast(vnf, vd), cache_seqlens=lens,
        block_table=table, k_descale=kd, v_descale=vd, nheads_k=hk)
