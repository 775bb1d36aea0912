"""The allocation-free decode entry point (fw_decode_kvcache_static) against the
ordinary one.

A host that cannot allocate device memory (its HBM is fully committed to the KV
pool, or it runs where the allocator must not be called) uses the variant whose
scratch is a fixed array inside the library.  Both entry points launch the same
deterministic kernels, so on the same inputs they must agree bit for bit, and
both must sit within the decode parity bar of the CPU oracle; the check runs
twice in a row because the built-in array is shared by every call and still
holds the first call's partial states when the second one starts (here with
other lengths, so stale states would show).  The status word of the built-in
array is read through fw_read_status_static.  Collected last on purpose: a
failure here cannot hide one elsewhere under `pytest -x`.
"""

import ctypes

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu

TOL = dict(rtol=1e-2, atol=2e-2)   # the bf16 bar of the decode parity tests


def static_status(lib):
    from flywheel_tpu.softmax_attention import _native
    word = ctypes.c_int32(-1)
    _native.check(lib.fw_read_status_static(0, ctypes.byref(word)))
    return word.value


def decode_args(case, tensors, out, lse):
    from flywheel_tpu.softmax_attention import _native
    batch, q_len, hq, d = case.q.shape
    return _native.FwDecodeArgs(
        q=tensors["q"].data_ptr(), out=out.data_ptr(), lse=lse.data_ptr(),
        kv_cache=tensors["pool"].data_ptr(), k_new=tensors["k"].data_ptr(),
        v_new=tensors["v"].data_ptr(), cache_seqlens=tensors["lens"].data_ptr(),
        block_table=tensors["table"].data_ptr(), num_pages=case.pool.shape[0],
        page_size=case.pool.shape[1], pages_per_seq=case.block_table.shape[1],
        batch=batch, seqlen_q=q_len, nheads=hq, nheads_k=case.nheads_k,
        head_dim=d, kv_dtype=0, causal=1, window_left=-1,
        softmax_scale=d ** -0.5, softcap=0.0, num_ctas=0)


def test_static_scratch_entry_matches_workspace_entry_twice():
    import torch
    from flywheel_tpu.softmax_attention import _native
    import paged_cases as workloads
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    for seed, lens in ((21, (700, 0, 3000, 65, 1290)), (22, (15, 2500, 64, 9, 4000))):
        case = workloads.host_case(seed, lens=lens, hq=32, hk=4, page_size=64)
        bf16 = lambda a: torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
        results = []
        for entry in ("fw_decode_kvcache", "fw_decode_kvcache_static"):
            tensors = {"q": bf16(case.q), "pool": bf16(case.pool), "k": bf16(case.k_new),
                       "v": bf16(case.v_new),
                       "lens": torch.from_numpy(case.cache_seqlens).to(dev),
                       "table": torch.from_numpy(case.block_table).to(dev)}
            out = torch.empty_like(tensors["q"])
            lse = torch.empty((len(lens), 32, 1), dtype=torch.float32, device=dev)
            args = decode_args(case, tensors, out, lse)
            if entry == "fw_decode_kvcache":
                nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
                assert 0 < nbytes, _native.last_error()
                scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
                args.workspace, args.workspace_bytes = scratch.data_ptr(), nbytes
            _native.check(getattr(lib, entry)(ctypes.byref(args), 0))
            torch.cuda.synchronize()
            if entry == "fw_decode_kvcache_static":
                assert static_status(lib) == 0
            results.append((out.float().cpu().numpy(), lse.cpu().numpy(),
                            tensors["pool"].cpu().view(torch.int16).numpy()))
        (out_a, lse_a, pool_a), (out_b, lse_b, pool_b) = results
        np.testing.assert_array_equal(out_b, out_a)       # the same kernels on the same inputs
        np.testing.assert_array_equal(lse_b, lse_a)
        np.testing.assert_array_equal(pool_b, pool_a)     # appended pages bit-exact
        want, want_lse, want_pool = oracle.kvcache_paged(
            case.q, case.pool, case.k_new, case.v_new, case.cache_seqlens, case.block_table,
            nheads_k=case.nheads_k, causal=True)
        np.testing.assert_allclose(out_b, want, **TOL)
        np.testing.assert_allclose(lse_b, want_lse, rtol=2e-3, atol=4e-3)
        np.testing.assert_array_equal(pool_b.view(np.uint16), want_pool.view(np.uint16))


def test_static_scratch_entry_reports_a_bad_page_through_its_own_status_reader():
    """A block-table entry outside the pool on the static entry point: status 2
    (FW_STATUS_BAD_PAGE) comes back through fw_read_status_static, once, and a
    clean call afterwards reads 0."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    import paged_cases as workloads
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    case = workloads.host_case(23, lens=(200, 70), hq=32, hk=4, page_size=64)
    bf16 = lambda a: torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
    for bad in (True, False):
        table = case.block_table.copy()
        if bad:
            table[0, 1] = 10 ** 6
        tensors = {"q": bf16(case.q), "pool": bf16(case.pool), "k": bf16(case.k_new), "v": bf16(case.v_new),
                   "lens": torch.from_numpy(case.cache_seqlens).to(dev), "table": torch.from_numpy(table).to(dev)}
        out = torch.empty_like(tensors["q"])
        lse = torch.empty((2, 32, 1), dtype=torch.float32, device=dev)
        _native.check(lib.fw_decode_kvcache_static(ctypes.byref(decode_args(case, tensors, out, lse)), 0))
        torch.cuda.synchronize()
        assert static_status(lib) == (2 if bad else 0)
        assert static_status(lib) == 0                    # cleared once reported


def test_static_scratch_entry_refuses_oversized_calls():
    from flywheel_tpu.softmax_attention import _native
    lib = _native.library()
    # 2048 requests x 128 heads x 4 query tokens of partial state cannot fit.
    args = _native.FwDecodeArgs(
        q=256, out=256, kv_cache=256, cache_seqlens=256, block_table=256,
        num_pages=8, page_size=64, pages_per_seq=2, batch=2048, seqlen_q=4,
        nheads=128, nheads_k=16, head_dim=128, kv_dtype=0, causal=1,
        window_left=-1, softmax_scale=0.1, softcap=0.0, num_ctas=8)
    with pytest.raises(ValueError, match="built-in scratch"):
        _native.check(lib.fw_decode_kvcache_static(ctypes.byref(args), None))
