"""Decode behaviours over several calls and constructions that turn an
off-by-one in key visibility into an O(1) error (shapes after the reference's
tests/softmax_attention/test_regression.py:1187-1269 and test_paged.py:698-848,
978-1011; values drawn here)."""

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu
TOL = dict(rtol=1e-2, atol=2e-2)


def bf16_cuda(array):
    import torch
    return torch.from_numpy(array.view(np.int16)).cuda().view(torch.bfloat16)


def test_step_after_step_appends_track_the_oracle():
    """40 consecutive decode steps on the same device-resident pool, lengths
    advancing by one, crossing page edges; the pool must equal the oracle's bit
    for bit after every step."""
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    import paged_cases as workloads
    # pages are allocated for the final lengths, so every appended token has a page of its own request
    case = workloads.host_case(51, lens=(40, 90, 160), hq=8, hk=2, page_size=64, max_pages=4)
    rng = np.random.default_rng(1)
    pool_t, pool_ref = bf16_cuda(case.pool), case.pool.copy()
    lens = case.cache_seqlens - 40
    for step in range(40):
        draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)
        q, k, v = draw((3, 1, 8, 128)), draw((3, 1, 2, 128)), draw((3, 1, 2, 128))
        out, pool_t = flash_attn_with_kvcache(q, pool_t, None, k, v, cache_seqlens=lens,
                                              block_table=case.block_table, causal=True)
        want, _, pool_ref = oracle.kvcache_paged(q, pool_ref, k, v, lens, case.block_table,
                                                 nheads_k=2, causal=True)
        np.testing.assert_allclose(out.astype(np.float32), want, **TOL)
        lens = lens + 1
    np.testing.assert_array_equal(pool_t.cpu().view(torch.int16).numpy(), pool_ref.view(np.int16))


def test_table_and_lengths_change_between_calls_on_one_workspace():
    """All-ones K, all-twos V: out is exactly 2 whatever the table, and the
    second call (other table, other lengths, same cached workspace) must not see
    anything of the first."""
    from flywheel_tpu import flash_attn_with_kvcache
    pages, page, hk, hq = 12, 64, 2, 8
    k_pages = np.ones((pages, page, hk, 128), np.float32).astype(oracle.BF16)
    v_pages = np.full((pages, page, hk, 128), 2.0, np.float32).astype(oracle.BF16)
    pool_t = bf16_cuda(oracle.merge_kv_heads(k_pages, v_pages))
    q = np.ones((2, 1, hq, 128), np.float32).astype(oracle.BF16)
    new = np.ones((2, 1, hk, 128), np.float32).astype(oracle.BF16)
    for table, lens in ((np.array([[0, 1, 2, 3], [4, 5, 6, 7]], np.int32), np.array([200, 3], np.int32)),
                        (np.array([[9, 8, 11, 10], [3, 2, 1, 0]], np.int32), np.array([17, 255], np.int32))):
        out, lse, pool_t = flash_attn_with_kvcache(
            q, pool_t, None, new, (2 * new.astype(np.float32)).astype(oracle.BF16), cache_seqlens=lens,
            block_table=table, causal=True, return_softmax_lse=True)
        np.testing.assert_allclose(out.astype(np.float32), 2.0, atol=1e-2)
        want_lse = 128 * 128 ** -0.5 + np.log(lens + 1.0)
        np.testing.assert_allclose(lse[:, :, 0], np.repeat(want_lse[:, None], hq, 1), rtol=2e-3)


@pytest.mark.parametrize("target", [0, 15, 16, 63, 64, 127, 128, 1023, 1024, 2047])
def test_needle_probe_finds_exactly_the_target_position(target):
    """Unit-norm random key codes; q aims at one position with a 16-nat margin,
    so the output is that position's value row unless a key is mis-masked or a
    neighbour is read in its place.  Stale slots past the length hold live
    codes too."""
    from flywheel_tpu import flash_attn_with_kvcache
    rng = np.random.default_rng(7)
    n, page, d = 2048, 64, 128
    codes = rng.standard_normal((n + page, 1, d)).astype(np.float32)
    codes /= np.linalg.norm(codes, axis=-1, keepdims=True)
    values = rng.standard_normal((n + page, 1, d)).astype(np.float32)
    pool = oracle.merge_kv_heads(codes.astype(oracle.BF16), values.astype(oracle.BF16))
    pool = pool.reshape(-1, page, 2, d)
    perm = rng.permutation(pool.shape[0]).astype(np.int32)
    shuffled = np.empty_like(pool)
    shuffled[perm] = pool
    length = n                                   # the stale page past it also holds codes
    q = (codes[target, 0] * 16.0 * np.sqrt(d)).astype(oracle.BF16).reshape(1, 1, 1, d)
    out, _ = flash_attn_with_kvcache(q, bf16_cuda(shuffled), None, cache_seqlens=np.array([length], np.int32),
                                     block_table=perm[None], causal=True)
    got = out.astype(np.float32)[0, 0, 0]
    want = values[target, 0].astype(oracle.BF16).astype(np.float32)
    assert np.abs(got - want).max() < 3e-2, (target, float(np.abs(got - want).max()))
    # with a window that just excludes the target the needle must vanish
    if target < length - 8:
        out2, _ = flash_attn_with_kvcache(
            q, bf16_cuda(shuffled), None, cache_seqlens=np.array([length], np.int32), block_table=perm[None],
            causal=True, window_size=(length - 2 - target, 0))
        assert np.abs(out2.astype(np.float32)[0, 0, 0] - want).max() > 0.2


def test_two_hundred_nat_jump_mid_stream():
    """Scores of 0 for 512 keys, then one key 200 nats higher: the running
    maximum has to move by 200 nats without overflow and the result is that
    key's value."""
    from flywheel_tpu import flash_attn_with_kvcache
    d, n, page = 128, 1024, 64
    keys = np.zeros((n, 1, d), np.float32)
    keys[512, 0, :] = 200.0 * np.sqrt(d) / d
    values = np.ones((n, 1, d), np.float32)
    values[512] = -3.0
    pool = oracle.merge_kv_heads(keys.astype(oracle.BF16), values.astype(oracle.BF16)).reshape(-1, page, 2, d)
    q = np.ones((1, 1, 4, d), np.float32).astype(oracle.BF16)
    out, lse, _ = flash_attn_with_kvcache(
        q, bf16_cuda(pool), None, cache_seqlens=np.array([n], np.int32),
        block_table=np.arange(n // page, dtype=np.int32)[None], causal=True, return_softmax_lse=True)
    np.testing.assert_allclose(out.astype(np.float32), -3.0, atol=2e-2)
    k512 = keys[512, 0].astype(oracle.BF16).astype(np.float32)
    np.testing.assert_allclose(lse, float(k512.sum() * d ** -0.5), rtol=2e-3)


def test_kv_head_shards_reproduce_the_full_call():
    """KV-head sharding needs no communication: each shard's decode over its own
    heads of every page is a slice of the full output (two shards run one after
    the other on this GPU)."""
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    from flywheel_tpu.softmax_attention import distributed as d
    import paged_cases as workloads
    from oracle import paged_attention as oracle
    case = workloads.host_case(5, lens=(3, 64, 700, 1500), hq=16, hk=4, page_size=64)
    to_t = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    full_pool = to_t(case.pool)
    full, full_lse, _ = flash_attn_with_kvcache(
        case.q, full_pool, None, case.k_new, case.v_new, cache_seqlens=case.cache_seqlens,
        block_table=case.block_table, causal=True, return_softmax_lse=True)
    k_pages, v_pages = oracle.split_kv_heads(case.pool, 4)
    for rank in range(2):
        q_heads, kv_heads = d.kv_head_shard(16, 4, 2, rank)
        shard_pool = to_t(oracle.merge_kv_heads(k_pages[:, :, kv_heads], v_pages[:, :, kv_heads]))
        out, lse, _ = flash_attn_with_kvcache(
            np.ascontiguousarray(case.q[:, :, q_heads]), shard_pool, None,
            np.ascontiguousarray(case.k_new[:, :, kv_heads]), np.ascontiguousarray(case.v_new[:, :, kv_heads]),
            cache_seqlens=case.cache_seqlens, block_table=case.block_table, causal=True,
            return_softmax_lse=True)
        # the same math per head; only the split of the key range over CTAs may differ
        np.testing.assert_allclose(out.astype(np.float32), full[:, :, q_heads].astype(np.float32), rtol=0, atol=1e-2)
        np.testing.assert_allclose(lse, full_lse[:, q_heads], rtol=0, atol=1e-4)
        # the shard's pool after the append = the shard's heads of the full pool
        got_k, got_v = oracle.split_kv_heads(shard_pool.cpu().view(torch.int16).numpy().view(oracle.BF16), 2)
        want_k, want_v = oracle.split_kv_heads(full_pool.cpu().view(torch.int16).numpy().view(oracle.BF16), 4)
        np.testing.assert_array_equal(got_k.view(np.uint16), want_k[:, :, kv_heads].view(np.uint16))
        np.testing.assert_array_equal(got_v.view(np.uint16), want_v[:, :, kv_heads].view(np.uint16))


@pytest.mark.parametrize("dtype,q_len", [("bf16", 1), ("bf16", 4), ("e4m3", 4)])
def test_repeated_calls_return_the_same_bits(dtype, q_len):
    """The same call 200 times on one workspace (no new tokens): every output
    must equal the first bit for bit.  A ring stage released before a warp's
    last read of it had been performed would show here as rare, small changes."""
    import ml_dtypes
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    import paged_cases as workloads
    lens = tuple(int(x) for x in np.random.default_rng(5).integers(200, 1400, 24))
    fp8 = dtype == "e4m3"
    case = workloads.host_case(77, lens=lens, q_len=q_len, hq=32 if q_len == 1 else 64, hk=8, page_size=64,
                               dtype=ml_dtypes.float8_e4m3fn if fp8 else oracle.BF16)
    if fp8:
        pool = torch.from_numpy(case.pool.view(np.uint8)).cuda().view(torch.float8_e4m3fn)
        scales = dict(k_descale=np.float32(case.k_descale), v_descale=np.float32(case.v_descale), nheads_k=8)
    else:
        pool, scales = bf16_cuda(case.pool), {}
    q_t = bf16_cuda(case.q)
    lens_t = torch.from_numpy(case.cache_seqlens).cuda()
    table_t = torch.from_numpy(case.block_table).cuda()
    first = None
    for _ in range(200):
        out, _ = flash_attn_with_kvcache(q_t, pool, None, None, None, cache_seqlens=lens_t, block_table=table_t,
                                         causal=True, **scales)
        bits = out.view(torch.int16)
        if first is None:
            first = bits.clone()
        else:
            assert bool((bits == first).all())
