"""GPU parity of flash_attn_with_kvcache (decode + fused append) against the
CPU oracle and the golden vectors.  Bars: appended cache pages bit-exact;
outputs within max-abs 2e-2 / rel 1e-2 for bf16 caches and 5e-2 for fp8."""

import ctypes

import numpy as np
import pytest

import cases
from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu

BF16_TOL = dict(rtol=1e-2, atol=2e-2)
FP8_TOL = dict(rtol=1e-2, atol=5e-2)
LSE_TOL = dict(rtol=2e-3, atol=4e-3)


def run_case(case, *, causal=True, window_left=None, softcap=0.0, sinks=None,
             num_active=None, append=True, lse=True, tol=BF16_TOL):
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    pool = torch.from_numpy(case.pool.view(
        np.int16 if case.pool.dtype.itemsize == 2 else np.uint8)).cuda()
    torch_dtype = {2: torch.bfloat16}.get(case.pool.dtype.itemsize)
    if torch_dtype is None:
        torch_dtype = (torch.float8_e4m3fn if case.pool.dtype == oracle.E4M3
                       else torch.float8_e5m2)
    pool = pool.view(torch_dtype)
    fp8 = case.pool.dtype.itemsize == 1
    kwargs = dict(
        cache_seqlens=case.cache_seqlens, block_table=case.block_table,
        causal=causal, softcap=softcap, return_softmax_lse=lse,
        window_size=(-1 if window_left is None else window_left, -1),
        learnable_sink=sinks, num_active=num_active, nheads_k=case.nheads_k)
    if fp8:
        kwargs.update(k_descale=case.k_descale, v_descale=case.v_descale)
    k, v = (case.k_new, case.v_new) if append else (None, None)
    outs = flash_attn_with_kvcache(case.q, pool, None, k, v, **kwargs)
    torch.cuda.synchronize()
    out = outs[0].astype(np.float32)
    got_lse = outs[1] if lse else None
    new_pool = outs[-1]
    assert new_pool is pool                      # updated in place
    from flywheel_tpu.softmax_attention import _arrays
    new_pool_np = _arrays.to_host_numpy(new_pool)

    want, want_lse, want_pool = oracle.kvcache_paged(
        case.q, case.pool, k, v, case.cache_seqlens, case.block_table,
        nheads_k=case.nheads_k, causal=causal, window_left=window_left,
        softcap=softcap, sinks=sinks, k_descale=case.k_descale,
        v_descale=case.v_descale, num_active=num_active)
    carrier = np.uint16 if case.pool.dtype.itemsize == 2 else np.uint8
    np.testing.assert_array_equal(new_pool_np.view(carrier), want_pool.view(carrier))
    np.testing.assert_allclose(out, want, **tol)
    if lse:
        finite = np.isfinite(want_lse)
        np.testing.assert_array_equal(np.isfinite(got_lse), finite)
        np.testing.assert_allclose(got_lse[finite], want_lse[finite], **LSE_TOL)
    return out


def host_case(*args, **kwargs):
    import paged_cases as workloads
    return workloads.host_case(*args, **kwargs)


@pytest.mark.parametrize("hq,hk", [(8, 1), (16, 2), (64, 8), (4, 4), (6, 3), (32, 16)])
@pytest.mark.parametrize("page_size", [64, 128])
def test_decode_head_tilings(hq, hk, page_size):
    case = host_case(1, lens=(0, 1, 15, 16, 63, 64, 300, 1027), hq=hq, hk=hk,
                     page_size=page_size)
    run_case(case)


@pytest.mark.parametrize("page_size", [16, 48, 64, 192, 384])
def test_decode_page_sizes(page_size):
    case = host_case(2, lens=(5, 47, 48, 191, 192, 777), page_size=page_size)
    run_case(case)


def test_decode_without_append_and_empty_rows():
    case = host_case(3, lens=(0, 0, 37, 128, 4))
    out = run_case(case, append=False)
    assert not out[:2].any()                     # nothing to attend: out 0


def test_decode_poisoned_stale_slots_and_bad_table_tail():
    case = host_case(4, lens=(2, 0, 65, 130), poison=True, bad_tail=True)
    out = run_case(case)
    assert np.isfinite(out).all()


def test_decode_num_active():
    case = host_case(5, lens=(40, 70, 100, 9))
    out = run_case(case, num_active=2)
    assert not out[2:].any()


@pytest.mark.parametrize("window_left,softcap", [(31, 0.0), (100, 30.0), (0, 0.0), (4095, 50.0)])
def test_decode_window_softcap(window_left, softcap):
    case = host_case(6, lens=(0, 17, 31, 32, 33, 500, 1100))
    run_case(case, window_left=window_left, softcap=softcap)


def test_decode_sinks():
    rng = np.random.default_rng(7)
    sinks = rng.uniform(-2, 8, 8).astype(np.float32)
    sinks[3] = -np.inf
    case = host_case(7, lens=(0, 3, 64, 400))
    run_case(case, sinks=sinks)
    run_case(host_case(8, lens=(0, 0, 9)), sinks=sinks, append=False)


@pytest.mark.parametrize("q_len", [1, 4])
def test_decode_sinks_leave_inactive_rows_alone(q_len):
    """Rows of requests past num_active are not attention rows: out 0 and lse
    -inf even when sinks are given (decode.py:600-617 of the reference masks the
    lse of inactive rows to -inf)."""
    rng = np.random.default_rng(10)
    sinks = rng.uniform(-2, 8, 8).astype(np.float32)
    case = host_case(10, lens=(40, 0, 100, 9, 0), q_len=q_len)
    run_case(case, sinks=sinks, num_active=3)
    run_case(case, sinks=sinks, num_active=3, append=False)


@pytest.mark.parametrize("q_len,hq,hk", [(4, 32, 8), (16, 32, 8), (16, 8, 1), (3, 6, 3), (2, 64, 8)])
def test_verify_window_on_decode_kernel(q_len, hq, hk):
    case = host_case(9, lens=(0, 60, 61, 64, 127, 129, 700), q_len=q_len, hq=hq, hk=hk)
    run_case(case)
    run_case(case, window_left=50, softcap=20.0, num_active=5)


@pytest.mark.parametrize("dtype", ["e4m3", "e5m2"])
@pytest.mark.parametrize("hk,q_len", [(2, 1), (3, 1), (8, 4)])
def test_decode_fp8(dtype, hk, q_len):
    np_dtype = oracle.E4M3 if dtype == "e4m3" else oracle.E5M2
    case = host_case(10, lens=(0, 1, 33, 64, 257, 900), hq=hk * 8, hk=hk,
                     q_len=q_len, dtype=np_dtype)
    rng = np.random.default_rng(3)
    sinks = rng.standard_normal(hk * 8).astype(np.float32)
    run_case(case, tol=FP8_TOL)
    run_case(case, window_left=200, softcap=50.0, sinks=sinks, tol=FP8_TOL)


def test_decode_fp8_poisoned():
    case = host_case(11, lens=(2, 70, 0), hq=16, hk=2, dtype=oracle.E4M3, poison=True)
    run_case(case, tol=FP8_TOL)


@pytest.mark.parametrize("name,q_len", [("page64_gqa8", 1), ("verify4_window", 4),
                                        ("fp8_e4m3_pow2_decode", 1), ("fp8_e4m3_amax_verify4", 4)])
def test_golden_single_token_and_verify_cases(name, q_len):
    """The decode kernel (single token and folded verify window) on the golden
    cases whose requests all have q_len tokens; outputs come from the reference's
    own NumPy oracle.  The fp8 ones include the serving verify-window setting in
    small (window 4095, softcap 50, sinks, 4 query tokens, amax descales)."""
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    from flywheel_tpu.softmax_attention import _arrays
    c = cases.build(name)
    golden = np.load(f"{cases.__file__.rsplit('/', 1)[0]}/{name}.npz")
    batch = len(c["lengths"])
    fp8 = c["kv_dtype"] != oracle.BF16
    pool = oracle.merge_kv_heads(c["k_pages"], c["v_pages"])
    carrier = np.uint8 if fp8 else np.int16
    torch_dtype = {oracle.BF16: torch.bfloat16, oracle.E4M3: torch.float8_e4m3fn,
                   oracle.E5M2: torch.float8_e5m2}[c["kv_dtype"]]
    pool_t = torch.from_numpy(pool.view(carrier)).cuda().view(torch_dtype)
    shape = (batch, q_len, -1, 128)
    extra = dict(k_descale=c["k_descale"], v_descale=c["v_descale"], nheads_k=c["kv_heads"]) if fp8 else {}
    out, lse, new_pool = flash_attn_with_kvcache(
        c["q"].reshape(shape), pool_t, None, c["k"].reshape(shape),
        c["v"].reshape(shape), cache_seqlens=c["lengths"],
        block_table=c["table"], causal=c["causal"], softcap=c["softcap"],
        window_size=(-1 if c["window_left"] is None else c["window_left"], -1),
        learnable_sink=c["sinks"], return_softmax_lse=True, **extra)
    want = golden["out"].reshape(out.shape)
    np.testing.assert_allclose(out.astype(np.float32), want, **(FP8_TOL if fp8 else BF16_TOL))
    want_lse = golden["lse"].reshape(-1, batch, q_len).transpose(1, 0, 2)
    np.testing.assert_allclose(lse, want_lse, **LSE_TOL)
    want_pool = oracle.append_to_pool(pool, c["k"], c["v"], c["cu"], c["lengths"], c["table"],
                                      nheads_k=c["kv_heads"])
    np.testing.assert_array_equal(_arrays.to_host_numpy(new_pool).view(carrier), want_pool.view(carrier))


def test_contiguous_pair_with_cache_batch_idx():
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    rng = np.random.default_rng(12)
    b, cap, hk, hq, d = 5, 256, 8, 32, 128
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)
    kc, vc = draw((7, cap, hk, d)), draw((7, cap, hk, d))
    q, k, v = draw((b, 1, hq, d)), draw((b, 1, hk, d)), draw((b, 1, hk, d))
    lengths = np.array([0, 1, 128, 200, 255], np.int32)
    rows = np.array([6, 2, 0, 5, 3], np.int32)
    to_t = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    kc_t, vc_t = to_t(kc), to_t(vc)
    for idx in (rows, None):
        want, want_lse, kc2, vc2 = oracle.kvcache_contiguous(
            q, kc, vc, k, v, lengths, idx, causal=True)
        a, b_ = to_t(kc), to_t(vc)
        out, lse, ko, vo = flash_attn_with_kvcache(
            q, a, b_, k, v, cache_seqlens=lengths, cache_batch_idx=idx,
            causal=True, return_softmax_lse=True)
        np.testing.assert_allclose(out.astype(np.float32), want, **BF16_TOL)
        np.testing.assert_allclose(lse, want_lse, **LSE_TOL)
        np.testing.assert_array_equal(ko.cpu().view(torch.int16).numpy(), kc2.view(np.int16))
        np.testing.assert_array_equal(vo.cpu().view(torch.int16).numpy(), vc2.view(np.int16))
    del kc_t, vc_t


def test_known_answer_high_scores_late_in_cache():
    # Scores 0 for the first 1024 keys, 32 for the rest; values 1 then 3: the
    # running maximum has to move by 32 nats mid-stream and the result is 3.
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    d, n, page = 128, 2048, 64
    q = np.ones((1, 1, 8, d), np.float32).astype(oracle.BF16)
    keys = np.zeros((n, 1, d), np.float32)
    keys[1024:] = 32.0 * np.sqrt(d) / d
    values = np.ones((n, 1, d), np.float32)
    values[1024:] = 3.0
    pool = oracle.merge_kv_heads(keys.astype(oracle.BF16), values.astype(oracle.BF16))
    pool = pool.reshape(n // page, page, 2, d)
    pool_t = torch.from_numpy(pool.view(np.int16)).cuda().view(torch.bfloat16)
    table = np.arange(n // page, dtype=np.int32)[None]
    out, lse, _ = flash_attn_with_kvcache(
        q, pool_t, None, cache_seqlens=np.array([n], np.int32), block_table=table,
        causal=True, return_softmax_lse=True)
    np.testing.assert_allclose(out.astype(np.float32), 3.0, atol=2e-2)
    np.testing.assert_allclose(lse, 32.0 * np.sqrt(d) / d * np.sqrt(d) + np.log(1024.0), rtol=2e-3)


@pytest.mark.parametrize("num_ctas", [1, 3, 7, 148, 400])
def test_split_count_does_not_change_results(num_ctas):
    """Calls the C ABI directly with a pinned CTA count: a request cut into any
    number of segments merges to the same answer."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    case = host_case(13, lens=(900, 17, 0, 2100, 64), hq=16, hk=2)
    dev = torch.device("cuda")
    t = lambda a, dt: torch.from_numpy(a.view(np.int16)).to(dev).view(dt)
    q, pool = t(case.q, torch.bfloat16), t(case.pool, torch.bfloat16)
    k, v = t(case.k_new, torch.bfloat16), t(case.v_new, torch.bfloat16)
    lens = torch.from_numpy(case.cache_seqlens).to(dev)
    table = torch.from_numpy(case.block_table).to(dev)
    out = torch.empty_like(q)
    lse = torch.empty((5, 16, 1), dtype=torch.float32, device=dev)
    args = _native.FwDecodeArgs(
        q=q.data_ptr(), out=out.data_ptr(), lse=lse.data_ptr(),
        kv_cache=pool.data_ptr(), k_new=k.data_ptr(), v_new=v.data_ptr(),
        cache_seqlens=lens.data_ptr(), block_table=table.data_ptr(),
        num_pages=pool.shape[0], page_size=pool.shape[1],
        pages_per_seq=table.shape[1], batch=5, seqlen_q=1, nheads=16,
        nheads_k=2, head_dim=128, kv_dtype=0, causal=1, window_left=-1,
        softmax_scale=128 ** -0.5, softcap=0.0, num_ctas=num_ctas)
    lib = _native.library()
    nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
    assert nbytes > 0, _native.last_error()
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    _native.check(lib.fw_decode_kvcache(ctypes.byref(args), 0))
    torch.cuda.synchronize()
    assert _native.read_status(ws, dev) == 0
    want, want_lse, want_pool = oracle.kvcache_paged(
        case.q, case.pool, case.k_new, case.v_new, case.cache_seqlens,
        case.block_table, nheads_k=2, causal=True)
    np.testing.assert_allclose(out.float().cpu().numpy(), want, **BF16_TOL)
    np.testing.assert_allclose(lse.cpu().numpy(), want_lse, **LSE_TOL)
    np.testing.assert_array_equal(
        pool.cpu().view(torch.int16).numpy(), want_pool.view(np.int16))


def test_repeatable_bitwise():
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    case = host_case(14, lens=(3000, 500, 1234), hq=64, hk=8)
    pool = torch.from_numpy(case.pool.view(np.int16)).cuda().view(torch.bfloat16)
    first = None
    for _ in range(5):
        out, _ = flash_attn_with_kvcache(
            case.q, pool, None, case.k_new, case.v_new,
            cache_seqlens=case.cache_seqlens, block_table=case.block_table, causal=True)
        bits = out.view(np.uint16)
        first = bits if first is None else first
        np.testing.assert_array_equal(bits, first)


def test_batch_larger_than_one_launch_is_sliced():
    """2500 requests: the host entry runs the kernel in slices of 2048 rows;
    num_active falls inside the second slice."""
    case = host_case(16, lens=tuple(int(x) for x in np.random.default_rng(3).integers(0, 40, 2500)),
                     hq=4, hk=1, page_size=16, extra_pages=1)
    out = run_case(case, num_active=2300)
    assert not out[2300:].any()


@pytest.mark.parametrize("hq,hk", [(64, 8), (8, 8), (6, 3), (16, 1)])
def test_decode_head_dim_64_with_sinks(hq, hk):
    """head_dim 64 on the paged decode kernel, the gpt-oss shape of the
    reference's tests (tests/softmax_attention/test_paged.py:1157-1182 there: 64
    query heads over 8 KV heads, head_dim 64, sinks): single token, a folded
    verify window, window + softcap, and without the append."""
    rng = np.random.default_rng(64)
    sinks = rng.uniform(-2, 8, hq).astype(np.float32)
    case = host_case(64, lens=(0, 1, 63, 64, 65, 300, 1027), hq=hq, hk=hk, d=64, page_size=64)
    run_case(case, sinks=sinks)
    run_case(case, sinks=sinks, append=False, window_left=127, softcap=30.0)
    if hq // hk <= 8:
        run_case(host_case(65, lens=(5, 60, 200), q_len=4, hq=hq, hk=hk, d=64, page_size=128), sinks=sinks,
                 num_active=2)


def test_decode_head_dim_64_contiguous_and_rejections():
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    rng = np.random.default_rng(66)
    b, cap, hk, hq, d = 3, 128, 4, 16, 64
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)
    kc, vc = draw((b, cap, hk, d)), draw((b, cap, hk, d))
    q, k, v = draw((b, 1, hq, d)), draw((b, 1, hk, d)), draw((b, 1, hk, d))
    lengths = np.array([0, 17, 127], np.int32)
    to_t = lambda a: torch.from_numpy(a.view(np.int16)).cuda().view(torch.bfloat16)
    want, want_lse, kc2, vc2 = oracle.kvcache_contiguous(q, kc, vc, k, v, lengths, None, causal=True)
    out, lse, ko, vo = flash_attn_with_kvcache(q, to_t(kc), to_t(vc), k, v, cache_seqlens=lengths, causal=True,
                                               return_softmax_lse=True)
    np.testing.assert_allclose(out.astype(np.float32), want, **BF16_TOL)
    np.testing.assert_allclose(lse, want_lse, **LSE_TOL)
    np.testing.assert_array_equal(ko.cpu().view(torch.int16).numpy(), kc2.view(np.int16))
    # fp8 at head_dim 64 and the packed route are not built: say so, do not fall back
    pool8 = torch.zeros((4, 64, 2 * hk, d), dtype=torch.uint8).cuda().view(torch.float8_e4m3fn)
    table = np.zeros((b, 1), np.int32)
    with pytest.raises(NotImplementedError, match="bfloat16 caches"):
        flash_attn_with_kvcache(q, pool8, None, cache_seqlens=lengths, block_table=table, nheads_k=hk)
    pool = torch.zeros((4, 64, 2 * hk, d), dtype=torch.bfloat16).cuda()
    with pytest.raises(NotImplementedError, match="decode kernel only"):
        flash_attn_with_kvcache(draw((b, 40, hq, d)), pool, None, cache_seqlens=lengths, block_table=table)
