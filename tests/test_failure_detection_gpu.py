"""Failure detection without a GPU fault: a bounded device-side wait that can
never be satisfied runs out, reports through the status word, and leaves the
context usable for the next (correct) call."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_reports_status():
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    from flywheel_tpu.softmax_attention import _native
    import paged_cases as workloads
    from oracle import paged_attention as oracle
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    scratch = torch.zeros(256, dtype=torch.uint8, device=dev)
    _native.check(lib.fw_selftest_wait_timeout(scratch.data_ptr(), 1 << 12, 0))
    torch.cuda.synchronize()
    assert _native.read_status(scratch, dev) == 1          # FW_STATUS_WAIT_TIMEOUT
    assert _native.read_status(scratch, dev) == 0          # cleared once reported
    # the context still works
    case = workloads.host_case(31, lens=(100, 7), hq=8, hk=2)
    pool = torch.from_numpy(case.pool.view(np.int16)).cuda().view(torch.bfloat16)
    out, _ = flash_attn_with_kvcache(case.q, pool, None, case.k_new, case.v_new,
                                     cache_seqlens=case.cache_seqlens, block_table=case.block_table,
                                     causal=True)
    want, _, _ = oracle.kvcache_paged(case.q, case.pool, case.k_new, case.v_new, case.cache_seqlens,
                                      case.block_table, nheads_k=2, causal=True)
    np.testing.assert_allclose(out.astype(np.float32), want, rtol=1e-2, atol=2e-2)


def test_bad_page_id_is_reported_not_dereferenced():
    """A block-table entry outside the pool inside the valid range: the kernel
    clamps it, finishes, and says so in the status word."""
    import ctypes
    import torch
    from flywheel_tpu.softmax_attention import _native
    import paged_cases as workloads
    case = workloads.host_case(32, lens=(200,), hq=8, hk=2)
    table = case.block_table.copy()
    table[0, 1] = 10 ** 6
    dev = torch.device("cuda", torch.cuda.current_device())
    bf16 = lambda a: torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
    q, pool = bf16(case.q), bf16(case.pool)
    lens, tab = torch.from_numpy(case.cache_seqlens).to(dev), torch.from_numpy(table).to(dev)
    out = torch.empty_like(q)
    args = _native.FwDecodeArgs(
        q=q.data_ptr(), out=out.data_ptr(), kv_cache=pool.data_ptr(), cache_seqlens=lens.data_ptr(),
        block_table=tab.data_ptr(), num_pages=pool.shape[0], page_size=64, pages_per_seq=tab.shape[1],
        batch=1, seqlen_q=1, nheads=8, nheads_k=2, head_dim=128, kv_dtype=0, causal=1, window_left=-1,
        softmax_scale=128 ** -0.5, softcap=0.0)
    lib = _native.library()
    nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    args.workspace, args.workspace_bytes = scratch.data_ptr(), nbytes
    _native.check(lib.fw_decode_kvcache(ctypes.byref(args), 0))
    torch.cuda.synchronize()
    assert _native.read_status(scratch, dev) == 2          # FW_STATUS_BAD_PAGE
    assert torch.isfinite(out.float()).all()
