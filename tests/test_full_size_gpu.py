"""Parity at the benchmark's full sizes through properties that do not need a
CPU pass over all of the data: spot requests against the CPU oracle, a checksum
of the whole pool around the append (every byte but the appended rows is
unchanged, the appended rows are the inputs bit for bit), independence of the
split count, and agreement of the two prefill kernels with each other."""

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_serving_scale_decode_properties():
    import torch
    import bench
    from flywheel_tpu.softmax_attention import _arrays, _native
    from oracle import paged_attention as oracle
    dev = torch.device("cuda", torch.cuda.current_device())
    work = bench.build_workload(0, dev)
    pool, lens, table = work["pool"], work["lens"], work["table"]
    dv = work["dev"]
    lens_l = torch.from_numpy(lens.astype(np.int64)).to(dev)
    pages = torch.from_numpy(table[np.arange(bench.BATCH), lens // bench.PAGE].astype(np.int64)).to(dev)
    slots = lens_l % bench.PAGE
    old_rows = pool[pages, slots].clone()                         # (batch, 16, 128)
    bits = lambda t: t.contiguous().view(torch.int16).to(torch.int64)
    before = sum(int(bits(pool[lo:lo + 4096]).sum()) for lo in range(0, pool.shape[0], 4096))

    (call, status), out = bench.make_decode_call(work, dev)
    call()
    torch.cuda.synchronize()
    assert status() == 0
    after = sum(int(bits(pool[lo:lo + 4096]).sum()) for lo in range(0, pool.shape[0], 4096))
    new_rows = torch.stack([dv["k"][:, 0], dv["v"][:, 0]], dim=2).reshape(bench.BATCH, 2 * bench.HK, bench.D)
    assert torch.equal(pool[pages, slots].view(torch.int16), new_rows.view(torch.int16))
    assert after - before == int(bits(new_rows).sum()) - int(bits(old_rows).sum())

    # three requests (shortest, median, longest) against the CPU oracle
    order = np.argsort(lens)
    for b in (order[0], order[len(order) // 2], order[-1]):
        n_pages = -(-(int(lens[b]) + 1) // bench.PAGE)
        sub = _arrays.to_host_numpy(pool[torch.from_numpy(table[b, :n_pages].astype(np.int64)).to(dev)])
        q = _arrays.to_host_numpy(dv["q"][b:b + 1])
        want, _ = oracle.ragged_paged_attention(
            q[0], sub, np.array([0, 1]), np.array([int(lens[b]) + 1]),
            np.arange(n_pages, dtype=np.int32)[None], nheads_k=bench.HK, causal=True)
        np.testing.assert_allclose(out[b].float().cpu().numpy(), want, rtol=1e-2, atol=2e-2)

    # the answer does not depend on how many CTAs the tiles are cut over
    first = out.clone()
    args = _native.FwDecodeArgs(
        q=dv["q"].data_ptr(), out=out.data_ptr(), kv_cache=pool.data_ptr(), k_new=dv["k"].data_ptr(),
        v_new=dv["v"].data_ptr(), cache_seqlens=dv["lens"].data_ptr(), block_table=dv["table"].data_ptr(),
        num_pages=pool.shape[0], page_size=bench.PAGE, pages_per_seq=dv["table"].shape[1],
        batch=bench.BATCH, seqlen_q=1, nheads=bench.HQ, nheads_k=bench.HK, head_dim=bench.D, kv_dtype=0,
        causal=1, window_left=-1, softmax_scale=bench.D ** -0.5, softcap=0.0, num_ctas=61)
    lib = _native.library()
    nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    _native.check(lib.fw_decode_kvcache(ctypes.byref(args), torch.cuda.current_stream(dev).cuda_stream))
    torch.cuda.synchronize()
    assert float((out.float() - first.float()).abs().max()) < 4e-3
    # and the second append of the same token left the pool as it was
    again = sum(int(bits(pool[lo:lo + 4096]).sum()) for lo in range(0, pool.shape[0], 4096))
    assert again == after


def test_chunked_prefill_kernels_agree_at_full_size(monkeypatch):
    import torch
    import bench
    from flywheel_tpu.softmax_attention import _arrays, _native
    from oracle import paged_attention as oracle
    dev = torch.device("cuda", torch.cuda.current_device())
    work = bench.build_prefill_workload(0, dev)
    results = {}
    for kernel in ("tcgen05", "splitkv"):
        call, out, scratch = bench.make_prefill_call(work, dev, route=kernel)
        call()
        torch.cuda.synchronize()
        assert _native.read_status(scratch, dev) == 0
        results[kernel] = out.float()
    diff = (results["tcgen05"] - results["splitkv"]).abs()
    assert float(diff.max()) < 2e-2 and float(diff.mean()) < 5e-4
    # shortest request against the CPU oracle
    r = int(np.argmin(work["seqused"]))
    n_pages = -(-int(work["seqused"][r]) // bench.PAGE)
    sub = _arrays.to_host_numpy(work["pool"][torch.from_numpy(work["table"][r, :n_pages].astype(np.int64)).to(dev)])
    lo, hi = int(work["cu"][r]), int(work["cu"][r + 1])
    q_rows = _arrays.to_host_numpy(work["q"][:, lo:hi]).transpose(1, 0, 2)
    want, _ = oracle.ragged_paged_attention(
        q_rows, sub, np.array([0, hi - lo]), work["seqused"][r:r + 1],
        np.arange(n_pages, dtype=np.int32)[None], nheads_k=bench.PF_HK, causal=True)
    got = results["tcgen05"][:, lo:hi].cpu().numpy().transpose(1, 0, 2)
    np.testing.assert_allclose(got, want, rtol=1e-2, atol=2e-2)


def test_split_kv_prefill_is_bit_stable_over_many_runs():
    """The split-KV route at full size, 100 times on one workspace: every run
    must reproduce the first bit for bit.  A stage of the K/V ring released
    before a warp's last ldmatrix of it had been performed showed up as one
    16-column block of a few rows changing in about one run of a hundred; the
    item order (a sort with atomics) changes from run to run and must not show
    either."""
    import torch
    import bench
    from flywheel_tpu.softmax_attention import _native
    dev = torch.device("cuda", torch.cuda.current_device())
    work = bench.build_prefill_workload(0, dev)
    call, out, scratch = bench.make_prefill_call(work, dev, route="splitkv")
    call()
    torch.cuda.synchronize()
    first = out.view(torch.int16).clone()
    for _ in range(100):
        call()
        torch.cuda.synchronize()
        assert bool((out.view(torch.int16) == first).all())
    assert _native.read_status(scratch, dev) == 0
