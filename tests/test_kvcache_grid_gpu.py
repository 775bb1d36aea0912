"""A seeded random grid over flash_attn_with_kvcache's options, after the shape
of the reference's FlashAttention-style grid
(tests/softmax_attention/test_prefill.py:504-824 of the reference): contiguous
/ paged, page sizes, bf16 / e4m3 / e5m2 with power-of-two descales, causal /
local, softcap, with and without new K/V, batch and packed q, MHA / MQA / GQA."""

import itertools

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu


def cuda_view(array):
    import torch
    if array.dtype == oracle.BF16:
        return torch.from_numpy(array.view(np.int16)).cuda().view(torch.bfloat16)
    kind = torch.float8_e4m3fn if array.dtype == oracle.E4M3 else torch.float8_e5m2
    return torch.from_numpy(array.view(np.uint8)).cuda().view(kind)


GRID = list(itertools.product(
    [(6, 6), (6, 1), (6, 3), (8, 2)],                   # heads, kv heads
    [(1, 128), (3, 1024), (64, 256), (5, 700)],         # seqlen_q, cached length bound
    [64, 128, 256],                                     # page size
    ["bf16", "e4m3", "e5m2"]))


@pytest.mark.parametrize("index", range(0, len(GRID), 3))
def test_random_grid(index):
    from flywheel_tpu import flash_attn_with_kvcache
    (hq, hk), (sq, sk), page, kind = GRID[index]
    rng = np.random.default_rng(1000 + index)
    dtype = {"bf16": oracle.BF16, "e4m3": oracle.E4M3, "e5m2": oracle.E5M2}[kind]
    batch, d = 5, 128
    causal = bool(rng.integers(0, 2)) or sq > 1
    window_left = int(rng.integers(0, sk)) if rng.integers(0, 2) else None
    softcap = 15.0 if rng.integers(0, 2) else 0.0
    new_kv = bool(rng.integers(0, 2))
    packed = bool(rng.integers(0, 2)) and sq > 1
    kd, vd = (2.0 ** -3, 2.0 ** -2) if kind != "bf16" else (1.0, 1.0)
    lens = rng.integers(0, sk + 1, batch).astype(np.int32)
    pages_b = [max(1, -(-(int(n) + sq) // page)) for n in lens]
    n_pages = sum(pages_b) + 1
    perm = rng.permutation(n_pages)
    table = np.full((batch, max(pages_b) + 1), -1, np.int32)
    cursor = 0
    for b, n in enumerate(pages_b):
        table[b, :n] = perm[cursor:cursor + n]
        cursor += n

    def draw(shape, scale=1.0):
        x = rng.standard_normal(shape, dtype=np.float32)
        if dtype == oracle.BF16:
            return x.astype(dtype)
        return oracle.quantize_per_tensor(x, dtype, descale=scale)[0]

    pool = oracle.merge_kv_heads(draw((n_pages, page, hk, d), kd), draw((n_pages, page, hk, d), vd))
    q = rng.standard_normal((batch, sq, hq, d), dtype=np.float32).astype(oracle.BF16)
    k = draw((batch, sq, hk, d), kd) if new_kv else None
    v = draw((batch, sq, hk, d), vd) if new_kv else None
    common = dict(causal=causal, softcap=softcap)
    scale_kwargs = dict(k_descale=kd, v_descale=vd) if kind != "bf16" else {}
    pool_t = cuda_view(pool)
    if packed:
        cu = (np.arange(batch + 1) * sq).astype(np.int32)
        flat = lambda a: None if a is None else a.reshape(-1, *a.shape[2:])
        out, lse, _ = flash_attn_with_kvcache(
            flat(q), pool_t, None, flat(k), flat(v), cache_seqlens=lens, block_table=table, cu_seqlens_q=cu,
            max_seqlen_q=sq, window_size=(-1 if window_left is None else window_left, -1),
            return_softmax_lse=True, nheads_k=hk, **common, **scale_kwargs)
        out = out.reshape(q.shape)
        lse = lse.reshape(hq, batch, sq).transpose(1, 0, 2)
    else:
        out, lse, _ = flash_attn_with_kvcache(
            q, pool_t, None, k, v, cache_seqlens=lens, block_table=table,
            window_size=(-1 if window_left is None else window_left, -1), return_softmax_lse=True,
            nheads_k=hk, **common, **scale_kwargs)
    want, want_lse, want_pool = oracle.kvcache_paged(
        q, pool, k, v, lens, table, nheads_k=hk, window_left=window_left, k_descale=kd, v_descale=vd, **common)
    from flywheel_tpu.softmax_attention import _arrays
    carrier = np.uint16 if dtype == oracle.BF16 else np.uint8
    np.testing.assert_array_equal(_arrays.to_host_numpy(pool_t).view(carrier), want_pool.view(carrier))
    # rows that see no key are unspecified on multi-token calls: compare where the oracle attends
    seen = np.isfinite(want_lse).transpose(0, 2, 1)[..., None]           # (batch, sq, heads, 1)
    tol = dict(rtol=1e-2, atol=2e-2) if kind == "bf16" else dict(rtol=1e-2, atol=5e-2)
    np.testing.assert_allclose(np.where(seen, out.astype(np.float32), 0), np.where(seen, want, 0), **tol)
    finite = np.isfinite(want_lse)
    np.testing.assert_allclose(lse[finite], want_lse[finite], rtol=2e-3, atol=4e-3)
