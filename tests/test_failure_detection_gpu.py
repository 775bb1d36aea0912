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


def test_append_to_a_bad_page_stores_nothing():
    """The fused append meets a block-table entry outside the pool, and a
    position past the table row: nothing is stored (page 0, which belongs to
    another request, keeps every bit), the row is still attended, and the status
    word says FW_STATUS_BAD_PAGE."""
    import ctypes
    import torch
    from flywheel_tpu.softmax_attention import _native
    import paged_cases as workloads
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    bf16 = lambda a: torch.from_numpy(a.view(np.int16)).to(dev).view(torch.bfloat16)
    # request 0 appends at position 128 = the first slot of its third page; request 1 at position 64
    case = workloads.host_case(33, lens=(128, 64), hq=8, hk=2, page_size=64, max_pages=3)
    for how in ("entry outside the pool", "position past the table row"):
        table = case.block_table.copy()
        width = table.shape[1]
        if how == "entry outside the pool":
            table[0, 2] = -7
        else:
            width = 2                     # request 0's append position 128 needs a third column
            table = np.ascontiguousarray(table[:, :2])
        q, pool = bf16(case.q), bf16(case.pool)
        k, v = bf16(case.k_new), bf16(case.v_new)
        before = pool.clone()
        lens, tab = torch.from_numpy(case.cache_seqlens).to(dev), torch.from_numpy(table).to(dev)
        out = torch.empty_like(q)
        args = _native.FwDecodeArgs(
            q=q.data_ptr(), out=out.data_ptr(), kv_cache=pool.data_ptr(), k_new=k.data_ptr(), v_new=v.data_ptr(),
            cache_seqlens=lens.data_ptr(), block_table=tab.data_ptr(), num_pages=pool.shape[0], page_size=64,
            pages_per_seq=width, batch=2, seqlen_q=1, nheads=8, nheads_k=2, head_dim=128, kv_dtype=0, causal=1,
            window_left=-1, softmax_scale=128 ** -0.5, softcap=0.0)
        nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
        scratch = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
        args.workspace, args.workspace_bytes = scratch.data_ptr(), nbytes
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), 0))
        torch.cuda.synchronize()
        assert _native.read_status(scratch, dev) == 2, how
        # request 1's append landed; nothing else in the pool changed, page 0 included
        page1, slot1 = int(case.block_table[1, 1]), 0
        changed = (pool.view(torch.int16) != before.view(torch.int16)).any(dim=(2, 3)).nonzero().cpu().tolist()
        assert changed == [[page1, slot1]], (how, changed)
        assert torch.isfinite(out.float()).all()


def test_a_reported_status_does_not_switch_later_prefills_off():
    """The tensor-core prefill shares its workspace with earlier calls.  A status
    some earlier launch left in the word (here: a bad page id met by a decode
    call) must not make it skip its work: its output still matches the oracle,
    and the word still carries the earlier report afterwards."""
    import torch
    from flywheel_tpu import flash_attn_varlen_func
    from flywheel_tpu.softmax_attention import _native, prefill
    from oracle import paged_attention as oracle
    dev = torch.device("cuda", torch.cuda.current_device())
    rng = np.random.default_rng(34)
    hq, hk, d, page = 8, 2, 128, 64
    chunks, prefixes = (130, 70), (0, 200)
    cu = np.concatenate(([0], np.cumsum(chunks))).astype(np.int32)
    seqused = (np.asarray(prefixes) + np.asarray(chunks)).astype(np.int32)
    pages_b = [-(-int(n) // page) for n in seqused]
    table = np.full((2, max(pages_b)), -1, np.int32)
    perm = rng.permutation(sum(pages_b))
    table[0, :pages_b[0]], table[1, :pages_b[1]] = perm[:pages_b[0]], perm[pages_b[0]:]
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)
    pool = oracle.merge_kv_heads(draw((sum(pages_b), page, hk, d)), draw((sum(pages_b), page, hk, d)))
    q = draw((int(cu[-1]), hq, d))
    # leave a BAD_PAGE report in the workspace the public entry points share on this stream
    from flywheel_tpu.softmax_attention import _cuda
    scratch = _native.workspace(dev, 1 << 20)
    word = torch.tensor([2], dtype=torch.int32, device=dev)
    _cuda.memcpy(scratch.data_ptr(), word.data_ptr(), 4, _cuda.MEMCPY_D2D)
    torch.cuda.synchronize()
    old = prefill.FORCED_ROUTE
    prefill.FORCED_ROUTE = "tcgen05"
    try:
        out = flash_attn_varlen_func(
            np.ascontiguousarray(q.transpose(1, 0, 2)),
            torch.from_numpy(pool.view(np.int16)).to(dev).view(torch.bfloat16), None, cu, None,
            int(max(chunks)), int(seqused.max()), causal=True, block_table=table, seqused_k=seqused)
    finally:
        prefill.FORCED_ROUTE = old
    want, _ = oracle.ragged_paged_attention(q, pool, cu, seqused, table, nheads_k=hk, causal=True)
    np.testing.assert_allclose(out.astype(np.float32).transpose(1, 0, 2), want, rtol=1e-2, atol=2e-2)
    assert _native.read_status(_native.workspace(dev, 1 << 20), dev) == 2   # the earlier report is still there


def test_status_check_switch_raises_through_the_public_api(monkeypatch):
    """FLYWHEEL_CHECK_STATUS=1: the entry point reads the device status after
    its launch and raises instead of returning a void result."""
    import torch
    from flywheel_tpu import flash_attn_with_kvcache
    import paged_cases as workloads
    case = workloads.host_case(35, lens=(200, 9), hq=8, hk=2)
    table = case.block_table.copy()
    table[0, 1] = 10 ** 6
    pool = torch.from_numpy(case.pool.view(np.int16)).cuda().view(torch.bfloat16)
    monkeypatch.setenv("FLYWHEEL_CHECK_STATUS", "1")
    with pytest.raises(RuntimeError, match="FW_STATUS_BAD_PAGE"):
        flash_attn_with_kvcache(case.q, pool, None, cache_seqlens=case.cache_seqlens, block_table=table,
                                causal=True)
    out, _ = flash_attn_with_kvcache(case.q, pool, None, cache_seqlens=case.cache_seqlens,
                                     block_table=case.block_table, causal=True)   # clean again
    assert np.isfinite(out.astype(np.float32)).all()
