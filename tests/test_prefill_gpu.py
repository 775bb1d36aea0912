"""GPU parity of chunked prefill over the paged cache: flash_attn_varlen_func
(block_table=...) and flash_attn_with_kvcache's packed / multi-token calls
(ragged append + attend), against the golden vectors and the CPU oracle."""

import pathlib

import numpy as np
import pytest

import cases
from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu

OUT_TOL = dict(rtol=1e-2, atol=2e-2)
FP8_TOL = dict(rtol=1e-2, atol=5e-2)
LSE_TOL = dict(rtol=2e-3, atol=4e-3)
GOLDEN_DIR = pathlib.Path(cases.__file__).resolve().parent


@pytest.fixture(autouse=True, params=["splitkv", "tcgen05"])
def prefill_kernel(request, monkeypatch):
    """Every case runs once per prefill kernel; shapes the tensor-core kernel
    does not take (fp8 pools, odd GQA groups) stay on the split-KV kernel."""
    monkeypatch.setattr("flywheel_tpu.softmax_attention.prefill.FORCED_ROUTE", request.param)
    return request.param


def to_cuda(array):
    import torch
    if array.dtype == oracle.BF16:
        return torch.from_numpy(array.view(np.int16)).cuda().view(torch.bfloat16)
    if array.dtype == oracle.E4M3:
        return torch.from_numpy(array.view(np.uint8)).cuda().view(torch.float8_e4m3fn)
    if array.dtype == oracle.E5M2:
        return torch.from_numpy(array.view(np.uint8)).cuda().view(torch.float8_e5m2)
    return torch.from_numpy(array).cuda()


def check_rows(out, lse, want, want_lse, tol):
    finite = np.isfinite(want_lse)
    np.testing.assert_allclose(out, want, **tol)
    np.testing.assert_array_equal(np.isfinite(lse), finite)
    np.testing.assert_allclose(lse[finite], want_lse[finite], **LSE_TOL)


def fp8_kwargs(c):
    """Descales and the KV head count an fp8 golden case needs (an fp8 pool's
    head axis may carry a pad head, so nheads_k is always passed)."""
    if c["kv_dtype"] == oracle.BF16:
        return {}
    return dict(k_descale=c["k_descale"], v_descale=c["v_descale"], nheads_k=c["kv_heads"])


def bits(array):
    return np.ascontiguousarray(array).view(np.uint16 if array.dtype.itemsize == 2 else np.uint8)


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_packed_kvcache_call_matches_golden(name):
    """flash_attn_with_kvcache with cu_seqlens_q: append, then attend.  The
    golden outputs come from the reference's own NumPy oracle (fp8 cases: fed
    stored * descale, as the reference's fp8 tests do)."""
    from flywheel_tpu import flash_attn_with_kvcache
    from flywheel_tpu.softmax_attention import _arrays
    c = cases.build(name)
    golden = np.load(GOLDEN_DIR / f"{name}.npz")
    tol = OUT_TOL if c["kv_dtype"] == oracle.BF16 else FP8_TOL
    pool = oracle.merge_kv_heads(c["k_pages"], c["v_pages"])
    pool_t = to_cuda(pool)
    max_q = max(1, int(np.diff(c["cu"]).max(initial=0)))
    out, lse, new_pool = flash_attn_with_kvcache(
        c["q"], pool_t, None, c["k"], c["v"], cache_seqlens=c["lengths"],
        block_table=c["table"], cu_seqlens_q=c["cu"], max_seqlen_q=max_q,
        causal=c["causal"], softcap=c["softcap"],
        window_size=(-1 if c["window_left"] is None else c["window_left"], -1),
        learnable_sink=c["sinks"], return_softmax_lse=True, **fp8_kwargs(c))
    check_rows(out.astype(np.float32), lse, golden["out"], golden["lse"], tol)
    end = int(c["cu"][-1])
    assert not out[end:].astype(np.float32).any()            # packed padding
    assert np.isneginf(lse[:, end:]).all()
    want_pool = oracle.append_to_pool(pool, c["k"], c["v"], c["cu"], c["lengths"], c["table"],
                                      nheads_k=c["kv_heads"])
    np.testing.assert_array_equal(bits(_arrays.to_host_numpy(new_pool)), bits(want_pool))


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_varlen_func_reads_pool_matches_golden(name):
    """flash_attn_varlen_func(block_table=...): head-major q, read-only."""
    from flywheel_tpu import flash_attn_varlen_func
    c = cases.build(name)
    golden = np.load(GOLDEN_DIR / f"{name}.npz")
    tol = OUT_TOL if c["kv_dtype"] == oracle.BF16 else FP8_TOL
    pool = oracle.merge_kv_heads(c["k_pages"], c["v_pages"])
    seqused = c["lengths"].copy()
    if c["k"] is not None:
        pool = oracle.append_to_pool(pool, c["k"], c["v"], c["cu"], c["lengths"], c["table"],
                                     nheads_k=c["kv_heads"])
        seqused = c["lengths"] + np.diff(c["cu"]).astype(np.int32)
    before = pool.copy()
    pool_t = to_cuda(pool)
    q_hm = np.ascontiguousarray(c["q"].transpose(1, 0, 2))
    out, lse = flash_attn_varlen_func(
        q_hm, pool_t, None, c["cu"], None, max(1, int(np.diff(c["cu"]).max(initial=0))),
        max(1, int(seqused.max(initial=0))), causal=c["causal"], softcap=c["softcap"],
        window_size=(-1 if c["window_left"] is None else c["window_left"], -1),
        learnable_sink=c["sinks"], return_softmax_lse=True, block_table=c["table"],
        seqused_k=seqused, **fp8_kwargs(c))
    check_rows(out.astype(np.float32).transpose(1, 0, 2), lse, golden["out"], golden["lse"], tol)
    from flywheel_tpu.softmax_attention import _arrays
    np.testing.assert_array_equal(bits(_arrays.to_host_numpy(pool_t)), bits(before))


def random_prefill_case(seed, prefixes, chunks, hq, hk, page_size, dtype=oracle.BF16, padding=5):
    rng = np.random.default_rng(seed)
    batch = len(chunks)
    cu = np.concatenate(([0], np.cumsum(chunks))).astype(np.int32)
    total_q = int(cu[-1]) + padding
    seqused = (np.asarray(prefixes) + np.asarray(chunks)).astype(np.int32)
    pages_b = [max(1, -(-int(n) // page_size)) for n in seqused]
    n_pages = sum(pages_b) + 2
    perm = rng.permutation(n_pages)
    table = np.full((batch, max(pages_b) + 1), -1, np.int32)
    cursor = 0
    for b, n in enumerate(pages_b):
        table[b, :n] = perm[cursor:cursor + n]
        cursor += n
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32)
    kf, vf = draw((n_pages, page_size, hk, 128)), draw((n_pages, page_size, hk, 128))
    if dtype == oracle.BF16:
        kd = vd = 1.0
        k_pages, v_pages = kf.astype(dtype), vf.astype(dtype)
    else:
        k_pages, kd = oracle.quantize_per_tensor(kf, dtype)
        v_pages, vd = oracle.quantize_per_tensor(vf, dtype)
    q = draw((total_q, hq, 128)).astype(oracle.BF16)
    return dict(q=q, pool=oracle.merge_kv_heads(k_pages, v_pages), cu=cu, seqused=seqused,
                table=table, kd=float(kd), vd=float(vd), hk=hk)


@pytest.mark.parametrize("hq,hk,page_size", [(32, 8, 64), (8, 8, 128), (16, 1, 64), (6, 3, 192)])
def test_varlen_func_random(hq, hk, page_size):
    from flywheel_tpu import flash_attn_varlen_func
    c = random_prefill_case(1, prefixes=(0, 700, 64, 2000, 5), chunks=(300, 40, 129, 1, 64),
                            hq=hq, hk=hk, page_size=page_size)
    rng = np.random.default_rng(2)
    sinks = rng.uniform(-2, 6, hq).astype(np.float32)
    for kwargs in (dict(causal=True), dict(causal=False),
                   dict(causal=True, window_left=100, softcap=30.0, sinks=sinks),
                   dict(causal=True, num_active=3)):
        window_left = kwargs.get("window_left")
        out, lse = flash_attn_varlen_func(
            np.ascontiguousarray(c["q"].transpose(1, 0, 2)), to_cuda(c["pool"]), None, c["cu"], None,
            300, 2100, causal=kwargs["causal"], softcap=kwargs.get("softcap", 0.0),
            window_size=(-1 if window_left is None else window_left, -1),
            learnable_sink=kwargs.get("sinks"), return_softmax_lse=True, block_table=c["table"],
            seqused_k=c["seqused"], num_active=kwargs.get("num_active"), nheads_k=hk)
        want, want_lse = oracle.ragged_paged_attention(
            c["q"], c["pool"], c["cu"], c["seqused"], c["table"], nheads_k=hk,
            causal=kwargs["causal"], window_left=window_left, softcap=kwargs.get("softcap", 0.0),
            sinks=kwargs.get("sinks"), num_active=kwargs.get("num_active"))
        check_rows(out.astype(np.float32).transpose(1, 0, 2), lse, want, want_lse, OUT_TOL)


@pytest.mark.parametrize("dtype", [oracle.E4M3, oracle.E5M2])
def test_varlen_func_fp8(dtype):
    from flywheel_tpu import flash_attn_varlen_func
    c = random_prefill_case(3, prefixes=(130, 0, 900), chunks=(70, 33, 200), hq=12, hk=3,
                            page_size=64, dtype=dtype)
    out, lse = flash_attn_varlen_func(
        np.ascontiguousarray(c["q"].transpose(1, 0, 2)), to_cuda(c["pool"]), None, c["cu"], None,
        200, 1100, causal=True, return_softmax_lse=True, block_table=c["table"],
        seqused_k=c["seqused"], k_descale=c["kd"], v_descale=c["vd"], nheads_k=3)
    want, want_lse = oracle.ragged_paged_attention(
        c["q"], c["pool"], c["cu"], c["seqused"], c["table"], nheads_k=3, causal=True,
        k_descale=c["kd"], v_descale=c["vd"])
    check_rows(out.astype(np.float32).transpose(1, 0, 2), lse, want, want_lse, FP8_TOL)


@pytest.mark.parametrize("q_scale,rotary", [(1e-3, False), (48.0, False), (1.0, True)])
def test_varlen_func_fp8_query_ranges_and_rotary(q_scale, rotary):
    """fp8 pools go to the tensor core with f16 operands: Q is converted from
    bf16 to f16 in shared memory (after the fused rotation, when there is one).
    Small queries (elements down to f16 subnormals), large ones (logits of tens of
    nats) and rotated ones must all stay within the fp8 tolerance."""
    import ml_dtypes
    from flywheel_tpu import flash_attn_varlen_func
    c = random_prefill_case(12, prefixes=(200, 0, 700), chunks=(90, 64, 150), hq=8, hk=2,
                            page_size=64, dtype=ml_dtypes.float8_e4m3fn)
    q = (c["q"].astype(np.float32) * np.float32(q_scale)).astype(oracle.BF16)
    kwargs, q_ref = {}, q
    if rotary:
        angle = np.random.default_rng(29).random((900, 64)) * 2 * np.pi
        cos, sin = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
        kwargs = dict(rotary_cos=cos, rotary_sin=sin, rotary_interleaved=False, rotary_k=False)
        q_ref = oracle.rotate_packed_q(q, cos, sin, c["cu"], c["seqused"], False)
    out, lse = flash_attn_varlen_func(
        np.ascontiguousarray(q.transpose(1, 0, 2)), to_cuda(c["pool"]), None, c["cu"], None, 150, 900,
        causal=True, return_softmax_lse=True, block_table=c["table"], seqused_k=c["seqused"],
        k_descale=c["kd"], v_descale=c["vd"], nheads_k=2, **kwargs)
    want, want_lse = oracle.ragged_paged_attention(
        q_ref, c["pool"], c["cu"], c["seqused"], c["table"], nheads_k=2, causal=True,
        k_descale=c["kd"], v_descale=c["vd"])
    check_rows(out.astype(np.float32).transpose(1, 0, 2), lse, want, want_lse, FP8_TOL)


@pytest.mark.parametrize("window_left", [None, 700])
def test_needle_probes_at_tile_and_page_edges(window_left):
    """The needle-probe construction of the reference's paged tests
    (tests/softmax_attention/test_paged.py:698-848 of the reference project) on
    the prefill kernels: unit-norm key codes, every (row, head) query aimed with
    a 20-nat logit at one visible position - the row's own, the one before it, a
    position next to a 16 / 64 / 128 / 256 / 512 / 1024-token tile or page edge,
    or a random one - and, on every third row, ALSO at the first hidden key.
    The output is the target's value row unless a key is mis-masked, skipped with
    its tile, or a neighbour is read in its place.  Stale slots past the length
    hold live codes.  With a left window the edge targets move to the first
    visible key, and the extra aim goes to the last key the window hides."""
    from flywheel_tpu import flash_attn_varlen_func
    rng = np.random.default_rng(7)
    prefix, chunk, heads, kv_heads, d, page = 1100, 320, 4, 2, 128, 64
    total, group = prefix + chunk, heads // kv_heads
    slots = -(-total // page) * page + page                      # a stale page past the end holds codes too
    codes = rng.standard_normal((slots, kv_heads, d)).astype(np.float32)
    codes /= np.linalg.norm(codes, axis=-1, keepdims=True)
    values = rng.standard_normal((slots, kv_heads, d)).astype(np.float32)
    edges = [0, 1, 15, 16, 63, 64, 65, 127, 128, 129, 255, 256, 511, 512, 1023, 1024, 1087, 1088, 1099, 1100]
    q = np.zeros((chunk, heads, d), np.float32)
    want = np.zeros((chunk, heads, d), np.float32)
    aim = 20.0 * np.sqrt(d)
    for r in range(chunk):
        diag = prefix + r
        first_visible = 0 if window_left is None else max(0, diag - window_left)
        for h in range(heads):
            kind = (r * heads + h) % 4
            if kind == 0:
                target = diag
            elif kind == 1:
                target = diag - 1
            elif kind == 2:
                target = edges[(r + h) % len(edges)] if window_left is None else first_visible
            else:
                target = int(rng.integers(first_visible, diag + 1))
            q[r, h] = codes[target, h // group] * aim
            want[r, h] = values[target, h // group]
            if r % 3 == 0:
                hidden = diag + 1 if window_left is None or h % 2 else first_visible - 1
                if 0 <= hidden < slots:
                    q[r, h] += codes[hidden, h // group] * aim
    pool = oracle.merge_kv_heads(codes.astype(oracle.BF16), values.astype(oracle.BF16)).reshape(-1, page, 2 * kv_heads, d)
    perm = rng.permutation(pool.shape[0]).astype(np.int32)
    shuffled = np.empty_like(pool)
    shuffled[perm] = pool
    q_bf16 = q.astype(oracle.BF16)
    cu, seqused = np.array([0, chunk], np.int32), np.array([total], np.int32)
    out = flash_attn_varlen_func(
        np.ascontiguousarray(q_bf16.transpose(1, 0, 2)), to_cuda(shuffled), None, cu, None, chunk, total,
        causal=True, window_size=(-1 if window_left is None else window_left, -1),
        block_table=perm[None], seqused_k=seqused)
    got = out.astype(np.float32).transpose(1, 0, 2)
    want_bf16 = want.astype(oracle.BF16).astype(np.float32)
    worst = np.abs(got - want_bf16).max(axis=-1)
    assert worst.max() < 4e-2, np.argwhere(worst >= 4e-2)[:8].tolist()
    ref, _ = oracle.ragged_paged_attention(q_bf16, shuffled, cu, seqused, perm[None], nheads_k=kv_heads,
                                           causal=True, window_left=window_left)
    np.testing.assert_allclose(got, ref, **OUT_TOL)


def test_multi_token_batch_call_takes_prefill_route():
    """A (batch, seqlen_q, ...) call too tall for the decode kernel's query
    tile appends and runs the packed kernel."""
    from flywheel_tpu import flash_attn_with_kvcache
    import paged_cases as workloads
    case = workloads.host_case(15, lens=(0, 100, 777), q_len=48, hq=32, hk=8)
    pool_t = to_cuda(case.pool)
    out, lse, _ = flash_attn_with_kvcache(
        case.q, pool_t, None, case.k_new, case.v_new, cache_seqlens=case.cache_seqlens,
        block_table=case.block_table, causal=True, return_softmax_lse=True)
    want, want_lse, want_pool = oracle.kvcache_paged(
        case.q, case.pool, case.k_new, case.v_new, case.cache_seqlens, case.block_table,
        nheads_k=8, causal=True)
    check_rows(out.astype(np.float32), lse, want, want_lse, OUT_TOL)
    from flywheel_tpu.softmax_attention import _arrays
    np.testing.assert_array_equal(_arrays.to_host_numpy(pool_t).view(np.uint16), want_pool.view(np.uint16))


def test_zero_row_packed_buffer():
    from flywheel_tpu import flash_attn_with_kvcache
    rng = np.random.default_rng(4)
    q = rng.standard_normal((8, 4, 128), dtype=np.float32).astype(oracle.BF16)
    pool = np.zeros((4, 64, 4, 128), oracle.BF16)
    out, lse, _ = flash_attn_with_kvcache(
        q, to_cuda(pool), None, q[:, :2], q[:, :2], cache_seqlens=np.zeros(2, np.int32),
        block_table=np.arange(4, dtype=np.int32).reshape(2, 2),
        cu_seqlens_q=np.zeros(3, np.int32), max_seqlen_q=1, causal=True, return_softmax_lse=True)
    assert not out.astype(np.float32).any() and np.isneginf(lse).all()


@pytest.mark.parametrize("rotary_interleaved", [False, True])
@pytest.mark.parametrize("table_dtype", ["float32", "bfloat16"])
def test_varlen_func_rotary_q_at_cache_positions(rotary_interleaved, table_dtype):
    """Q-only RoPE (rotary_k=False): token t of a request is rotated at
    seqused_k - len_q + t; the cache holds K already rotated."""
    from flywheel_tpu import flash_attn_varlen_func
    c = random_prefill_case(6, prefixes=(127, 0, 251), chunks=(3, 1, 130), hq=8, hk=2, page_size=64)
    angle = np.random.default_rng(23).random((448, 64)) * 2 * np.pi
    dt = np.float32 if table_dtype == "float32" else oracle.BF16
    cos, sin = np.cos(angle).astype(dt), np.sin(angle).astype(dt)
    out, lse = flash_attn_varlen_func(
        np.ascontiguousarray(c["q"].transpose(1, 0, 2)), to_cuda(c["pool"]), None, c["cu"], None, 130,
        448, causal=True, return_softmax_lse=True, block_table=c["table"], seqused_k=c["seqused"],
        rotary_cos=cos, rotary_sin=sin, rotary_interleaved=rotary_interleaved, rotary_k=False)
    q_ro = oracle.rotate_packed_q(c["q"], cos, sin, c["cu"], c["seqused"], rotary_interleaved)
    want, want_lse = oracle.ragged_paged_attention(
        q_ro, c["pool"], c["cu"], c["seqused"], c["table"], nheads_k=2, causal=True)
    check_rows(out.astype(np.float32).transpose(1, 0, 2), lse, want, want_lse, OUT_TOL)
    with pytest.raises(NotImplementedError, match="rotary_k=False"):
        flash_attn_varlen_func(
            np.ascontiguousarray(c["q"].transpose(1, 0, 2)), to_cuda(c["pool"]), None, c["cu"], None, 130,
            448, block_table=c["table"], seqused_k=c["seqused"], rotary_cos=cos, rotary_sin=sin)
