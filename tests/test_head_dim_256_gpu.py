"""head_dim 256 (the reference's serving shapes: 32 q heads, 4 or 32 KV heads,
docs/v7x.md:129-150 of the reference) through the same entry points: decode
with fused append, verify windows, fp8, the contiguous pair, chunked prefill
with Q-only RoPE, and the state merge."""

import ctypes

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu

D = 256
TOL = {"bf16": dict(rtol=1e-2, atol=2e-2), "fp8": dict(rtol=1e-2, atol=5e-2)}
LSE_TOL = dict(rtol=2e-3, atol=4e-3)


def to_cuda(array):
    import torch
    if array.dtype == oracle.BF16:
        return torch.from_numpy(array.view(np.int16)).cuda().view(torch.bfloat16)
    if array.dtype in (oracle.E4M3, oracle.E5M2):
        kind = torch.float8_e4m3fn if array.dtype == oracle.E4M3 else torch.float8_e5m2
        return torch.from_numpy(array.view(np.uint8)).cuda().view(kind)
    return torch.from_numpy(array).cuda()


def paged_inputs(seed, lens, sq, hq, hk, page, dtype):
    rng = np.random.default_rng(seed)
    batch = len(lens)
    lens = np.asarray(lens, np.int32)
    pages_b = [max(1, -(-(int(n) + sq) // page)) for n in lens]
    n_pages = sum(pages_b) + 1
    perm = rng.permutation(n_pages)
    table = np.full((batch, max(pages_b) + 1), -1, np.int32)
    cursor = 0
    for b, n in enumerate(pages_b):
        table[b, :n] = perm[cursor:cursor + n]
        cursor += n
    kd, vd = (2.0 ** -3, 2.0 ** -2) if dtype != oracle.BF16 else (1.0, 1.0)

    def draw(shape, scale):
        x = rng.standard_normal(shape, dtype=np.float32)
        return x.astype(dtype) if dtype == oracle.BF16 else oracle.quantize_per_tensor(x, dtype, descale=scale)[0]

    pool = oracle.merge_kv_heads(draw((n_pages, page, hk, D), kd), draw((n_pages, page, hk, D), vd))
    q = rng.standard_normal((batch, sq, hq, D), dtype=np.float32).astype(oracle.BF16)
    k, v = draw((batch, sq, hk, D), kd), draw((batch, sq, hk, D), vd)
    return q, pool, k, v, lens, table, kd, vd


@pytest.mark.parametrize("hq,hk", [(32, 4), (32, 32), (8, 1), (6, 3)])
@pytest.mark.parametrize("kind", ["bf16", "e4m3", "e5m2"])
@pytest.mark.parametrize("sq", [1, 4])
def test_paged_decode(hq, hk, kind, sq):
    from flywheel_tpu import flash_attn_with_kvcache
    from flywheel_tpu.softmax_attention import _arrays
    dtype = {"bf16": oracle.BF16, "e4m3": oracle.E4M3, "e5m2": oracle.E5M2}[kind]
    if sq * (hq // hk) > 64:
        pytest.skip("more than 64 query rows per KV head at head_dim 256")
    q, pool, k, v, lens, table, kd, vd = paged_inputs(
        7 + hq + sq, (0, 1, 15, 16, 127, 128, 700, 1500), sq, hq, hk, 128, dtype)
    sinks = np.random.default_rng(3).standard_normal(hq).astype(np.float32)
    pool_t = to_cuda(pool)
    scales = dict(k_descale=kd, v_descale=vd) if kind != "bf16" else {}
    out, lse, _ = flash_attn_with_kvcache(
        q, pool_t, None, k, v, cache_seqlens=lens, block_table=table, causal=True, window_size=(600, -1),
        softcap=30.0, learnable_sink=sinks, return_softmax_lse=True, nheads_k=hk, **scales)
    want, want_lse, want_pool = oracle.kvcache_paged(
        q, pool, k, v, lens, table, nheads_k=hk, causal=True, window_left=600, softcap=30.0, sinks=sinks,
        k_descale=kd, v_descale=vd)
    carrier = np.uint16 if kind == "bf16" else np.uint8
    np.testing.assert_array_equal(_arrays.to_host_numpy(pool_t).view(carrier), want_pool.view(carrier))
    np.testing.assert_allclose(out.astype(np.float32), want, **TOL["bf16" if kind == "bf16" else "fp8"])
    np.testing.assert_allclose(lse, want_lse, **LSE_TOL)


def test_contiguous_pair():
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    rng = np.random.default_rng(11)
    batch, cap, hq, hk = 5, 512, 32, 4
    k_cache = rng.standard_normal((batch + 2, cap, hk, D), dtype=np.float32).astype(oracle.BF16)
    v_cache = rng.standard_normal((batch + 2, cap, hk, D), dtype=np.float32).astype(oracle.BF16)
    q = rng.standard_normal((batch, 1, hq, D), dtype=np.float32).astype(oracle.BF16)
    k = rng.standard_normal((batch, 1, hk, D), dtype=np.float32).astype(oracle.BF16)
    v = rng.standard_normal((batch, 1, hk, D), dtype=np.float32).astype(oracle.BF16)
    lens = np.array([0, 17, 300, 511, 64], np.int32)
    idx = np.array([6, 0, 3, 2, 5], np.int32)
    kc, vc = to_cuda(k_cache), to_cuda(v_cache)
    out, lse, _, _ = flash_attn_with_kvcache(q, kc, vc, k, v, cache_seqlens=lens, cache_batch_idx=idx,
                                             causal=True, return_softmax_lse=True)
    want, want_lse, want_k, want_v = oracle.kvcache_contiguous(q, k_cache, v_cache, k, v, lens, idx, causal=True)
    from flywheel_tpu.softmax_attention import _arrays
    np.testing.assert_array_equal(_arrays.to_host_numpy(kc).view(np.uint16), want_k.view(np.uint16))
    np.testing.assert_array_equal(_arrays.to_host_numpy(vc).view(np.uint16), want_v.view(np.uint16))
    np.testing.assert_allclose(out.astype(np.float32), want, **TOL["bf16"])
    np.testing.assert_allclose(lse, want_lse, **LSE_TOL)


@pytest.mark.parametrize("kernel", ["tcgen05", "splitkv"])
@pytest.mark.parametrize("hq,hk", [(32, 4), (8, 8), (6, 2)])
@pytest.mark.parametrize("rotary", [False, True])
def test_chunked_prefill(hq, hk, rotary, kernel, monkeypatch):
    from flywheel_tpu import flash_attn_varlen_func
    monkeypatch.setattr("flywheel_tpu.softmax_attention.prefill.FORCED_ROUTE", kernel)
    rng = np.random.default_rng(23)
    page = 128
    prefixes, chunks = (0, 300, 1000, 77), (200, 64, 130, 1)
    cu = np.concatenate(([0], np.cumsum(chunks))).astype(np.int32)
    total_q = int(cu[-1]) + 3
    seqused = (np.asarray(prefixes) + np.asarray(chunks)).astype(np.int32)
    pages_b = [-(-int(n) // page) for n in seqused]
    n_pages = sum(pages_b) + 2
    perm = rng.permutation(n_pages)
    table = np.full((len(chunks), max(pages_b) + 1), -1, np.int32)
    cursor = 0
    for b, n in enumerate(pages_b):
        table[b, :n] = perm[cursor:cursor + n]
        cursor += n
    pool = oracle.merge_kv_heads(
        rng.standard_normal((n_pages, page, hk, D), dtype=np.float32).astype(oracle.BF16),
        rng.standard_normal((n_pages, page, hk, D), dtype=np.float32).astype(oracle.BF16))
    q = rng.standard_normal((total_q, hq, D), dtype=np.float32).astype(oracle.BF16)
    kwargs, q_ref = {}, q
    if rotary:
        angles = rng.uniform(0, 2 * np.pi, (int(seqused.max()) + 4, D // 2)).astype(np.float32)
        cos, sin = np.cos(angles), np.sin(angles)
        kwargs = dict(rotary_cos=cos, rotary_sin=sin, rotary_k=False)
        q_ref = oracle.rotate_packed_q(q, cos, sin, cu, seqused)
    sinks = rng.standard_normal(hq).astype(np.float32)
    out, lse = flash_attn_varlen_func(
        np.ascontiguousarray(q.transpose(1, 0, 2)), to_cuda(pool), None, cu, None, int(max(chunks)),
        int(seqused.max()), causal=True, window_size=(400, 0), softcap=20.0, learnable_sink=sinks,
        return_softmax_lse=True, block_table=table, seqused_k=seqused, **kwargs)
    want, want_lse = oracle.ragged_paged_attention(q_ref, pool, cu, seqused, table, nheads_k=hk, causal=True,
                                                   window_left=400, softcap=20.0, sinks=sinks)
    end = int(cu[-1])
    np.testing.assert_allclose(out.astype(np.float32).transpose(1, 0, 2)[:end], want[:end], **TOL["bf16"])
    np.testing.assert_allclose(lse[:, :end], want_lse[:, :end], **LSE_TOL)
    assert not out.astype(np.float32)[:, end:].any() and np.isneginf(lse[:, end:]).all()


def test_state_merge():
    import torch
    from flywheel_tpu.softmax_attention import _native
    rng = np.random.default_rng(5)
    parts, rows, heads = 3, 24, 8
    outs = rng.standard_normal((parts, rows, D)).astype(np.float32)
    lses = rng.standard_normal((parts, rows)).astype(np.float32)
    lses[1, 4] = -np.inf
    sinks = rng.standard_normal(heads).astype(np.float32)
    want, want_lse = oracle.merge_states(outs, lses, sinks=np.tile(sinks, rows // heads))
    o_t, l_t, s_t = (torch.from_numpy(x).cuda() for x in (outs, lses, sinks))
    out = torch.empty((rows, D), dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(rows, dtype=torch.float32, device="cuda")
    args = _native.FwCombineArgs(
        partial_out=o_t.data_ptr(), partial_lse=l_t.data_ptr(), sinks=s_t.data_ptr(), out=out.data_ptr(),
        lse=lse.data_ptr(), parts=parts, rows=rows, nheads=heads, head_dim=D, lse_head_stride=1,
        lse_token_stride=heads)
    _native.check(_native.library().fw_lse_combine(ctypes.byref(args), _native.current_stream(out.device)))
    torch.cuda.synchronize()
    np.testing.assert_allclose(out.float().cpu().numpy(), want, **TOL["bf16"])
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, **LSE_TOL)


def test_multi_token_kvcache_call_appends_then_prefills():
    """(batch, seqlen_q > fold limit) goes through the ragged append and the
    head_dim 256 tensor-core prefill kernel."""
    from flywheel_tpu import flash_attn_with_kvcache
    from flywheel_tpu.softmax_attention import _arrays
    hq, hk, sq = 8, 2, 100
    q, pool, k, v, lens, table, kd, vd = paged_inputs(31, (0, 77, 300), sq, hq, hk, 128, oracle.BF16)
    pool_t = to_cuda(pool)
    out, lse, _ = flash_attn_with_kvcache(q, pool_t, None, k, v, cache_seqlens=lens, block_table=table,
                                          causal=True, return_softmax_lse=True)
    want, want_lse, want_pool = oracle.kvcache_paged(q, pool, k, v, lens, table, nheads_k=hk, causal=True)
    np.testing.assert_array_equal(_arrays.to_host_numpy(pool_t).view(np.uint16), want_pool.view(np.uint16))
    np.testing.assert_allclose(out.astype(np.float32), want, **TOL["bf16"])
    np.testing.assert_allclose(lse, want_lse, **LSE_TOL)


@pytest.mark.parametrize("kernel", ["tcgen05", "splitkv"])
@pytest.mark.parametrize("kind", ["e4m3", "e5m2"])
def test_chunked_prefill_fp8_pool(kind, kernel, monkeypatch):
    """fp8 pools at head_dim 256: widened into bf16 scratch and run on the
    tensor-core kernel, or read in place by the split-KV kernel."""
    from flywheel_tpu import flash_attn_varlen_func
    monkeypatch.setattr("flywheel_tpu.softmax_attention.prefill.FORCED_ROUTE", kernel)
    dtype = oracle.E4M3 if kind == "e4m3" else oracle.E5M2
    rng = np.random.default_rng(29)
    hq, hk, page = 8, 2, 64
    prefixes, chunks = (0, 500, 90), (300, 70, 129)
    cu = np.concatenate(([0], np.cumsum(chunks))).astype(np.int32)
    seqused = (np.asarray(prefixes) + np.asarray(chunks)).astype(np.int32)
    pages_b = [-(-int(n) // page) for n in seqused]
    n_pages = sum(pages_b) + 1
    perm = rng.permutation(n_pages)
    table = np.full((len(chunks), max(pages_b)), -1, np.int32)
    cursor = 0
    for b, n in enumerate(pages_b):
        table[b, :n] = perm[cursor:cursor + n]
        cursor += n
    kd, vd = 2.0 ** -3, 2.0 ** -2
    k_pages = oracle.quantize_per_tensor(rng.standard_normal((n_pages, page, hk, D), dtype=np.float32), dtype, descale=kd)[0]
    v_pages = oracle.quantize_per_tensor(rng.standard_normal((n_pages, page, hk, D), dtype=np.float32), dtype, descale=vd)[0]
    pool = oracle.merge_kv_heads(k_pages, v_pages)
    q = rng.standard_normal((int(cu[-1]), hq, D), dtype=np.float32).astype(oracle.BF16)
    out, lse = flash_attn_varlen_func(
        np.ascontiguousarray(q.transpose(1, 0, 2)), to_cuda(pool), None, cu, None, int(max(chunks)),
        int(seqused.max()), causal=True, return_softmax_lse=True, block_table=table, seqused_k=seqused,
        k_descale=kd, v_descale=vd, nheads_k=hk)
    want, want_lse = oracle.ragged_paged_attention(q, pool, cu, seqused, table, nheads_k=hk, causal=True,
                                                   k_descale=kd, v_descale=vd)
    np.testing.assert_allclose(out.astype(np.float32).transpose(1, 0, 2), want, **TOL["fp8"])
    np.testing.assert_allclose(lse, want_lse, **LSE_TOL)
