"""Round-robin page sharding of one long request, with the ranks emulated one
after another on a single GPU: fw_shard_step decides on the device how many
tokens each rank holds and which rank appends, fw_decode_kvcache runs in
partial-state mode with append_enable, and fw_lse_combine merges the ranks'
(o, lse) states (the merge of patches/tpu-inference.patch:7174-7186 of the
reference project).  No kernel waits on another here, so running the ranks
back to back on one device is the same computation as on several."""

import ctypes

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [1, 2, 3])
def test_round_robin_shards_match_the_oracle(world):
    import torch
    from flywheel_tpu.softmax_attention import _native, distributed as d
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    rng = np.random.default_rng(3 + world)
    heads, kv_heads, dim, page, total_pages = 16, 4, 128, 64, 9
    length, steps = 3 * page + 61, 6            # the appending rank changes after three steps
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)
    keys, values = draw((total_pages * page, kv_heads, dim)), draw((total_pages * page, kv_heads, dim))
    rows = oracle.merge_kv_heads(keys, values).reshape(total_pages, page, 2 * kv_heads, dim)
    to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.bfloat16)

    ranks = []
    for rank in range(world):
        owned = np.asarray(d.owned_pages(total_pages, world, rank))
        perm = np.random.default_rng(20 + rank).permutation(len(owned) + 2)[:len(owned)]
        pool = np.zeros((len(owned) + 2, page, 2 * kv_heads, dim), oracle.BF16)
        pool[perm] = rows[owned]
        ranks.append(dict(
            owned=owned, perm=perm, pool=to_t(pool),
            table=torch.from_numpy(perm.astype(np.int32)[None]).to(dev),
            counters=torch.tensor([length, 0, 0], dtype=torch.int32, device=dev), scratch=None))
    states = torch.empty((world, heads * (dim + 1)), dtype=torch.float32, device=dev)
    out = torch.empty((1, 1, heads, dim), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((1, heads, 1), dtype=torch.float32, device=dev)

    for _ in range(steps):
        q, k, v = draw((1, 1, heads, dim)), draw((1, 1, kv_heads, dim)), draw((1, 1, kv_heads, dim))
        q_t, k_t, v_t = to_t(q), to_t(k), to_t(v)
        appenders = 0
        for rank, state in enumerate(ranks):
            base = state["counters"].data_ptr()
            shard = _native.FwShardStepArgs(global_len=base, local_len=base + 4, append_enable=base + 8,
                                            page_size=page, world=world, rank=rank, advance=1)
            _native.check(lib.fw_shard_step(ctypes.byref(shard), stream))
            args = _native.FwDecodeArgs(
                q=q_t.data_ptr(), kv_cache=state["pool"].data_ptr(), k_new=k_t.data_ptr(), v_new=v_t.data_ptr(),
                append_enable=base + 8, cache_seqlens=base + 4, block_table=state["table"].data_ptr(),
                partial_out=states[rank].data_ptr(), partial_lse=states[rank, heads * dim:].data_ptr(),
                num_pages=state["pool"].shape[0], page_size=page, pages_per_seq=state["table"].shape[1],
                batch=1, seqlen_q=1, nheads=heads, nheads_k=kv_heads, head_dim=dim, kv_dtype=0, causal=0,
                window_left=-1, softmax_scale=dim ** -0.5, softcap=0.0)
            if state["scratch"] is None:
                nbytes = lib.fw_decode_workspace_bytes(ctypes.byref(args))
                assert nbytes, _native.last_error()
                state["scratch"] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
            args.workspace, args.workspace_bytes = state["scratch"].data_ptr(), state["scratch"].numel()
            _native.check(lib.fw_decode_kvcache(ctypes.byref(args), stream))
            torch.cuda.synchronize()
            total, local, appends = state["counters"].cpu().tolist()
            assert total == length + 1
            assert local == d.local_length(length, page, world, rank)
            assert appends == int(d.owner_of_page(length // page, world) == rank)
            appenders += appends
        assert appenders == 1
        merge = _native.FwCombineArgs(
            partial_out=states.data_ptr(), partial_lse=states[0, heads * dim:].data_ptr(), out=out.data_ptr(),
            lse=lse.data_ptr(), parts=world, rows=heads, nheads=heads, head_dim=dim, lse_head_stride=1,
            lse_token_stride=heads, part_stride_out=heads * (dim + 1), part_stride_lse=heads * (dim + 1))
        _native.check(lib.fw_lse_combine(ctypes.byref(merge), stream))
        torch.cuda.synchronize()
        keys[length], values[length] = k[0, 0], v[0, 0]
        length += 1
        want, want_lse = oracle.attend_rows(
            q[0].astype(np.float32), keys[:length].astype(np.float32), values[:length].astype(np.float32),
            total=length, causal=True, window_left=None, softcap=0.0, scale=dim ** -0.5, sinks=None)
        np.testing.assert_allclose(out.float().cpu().numpy()[0], want, rtol=1e-2, atol=2e-2)
        np.testing.assert_allclose(lse.cpu().numpy()[0, :, 0], want_lse[:, 0], rtol=2e-3, atol=4e-3)

    # every appended row landed bit-exact on the rank that owns its page, and nowhere else
    want_rows = oracle.merge_kv_heads(keys, values).reshape(total_pages, page, 2 * kv_heads, dim)
    for state in ranks:
        got = state["pool"].cpu().view(torch.int16).numpy()
        np.testing.assert_array_equal(got[state["perm"]], want_rows[state["owned"]].view(np.int16))
        assert _native.read_status(state["scratch"], dev) == 0


@pytest.mark.parametrize("world,with_sinks", [(1, False), (2, True), (3, False)])
def test_fused_sharded_step_delivers_and_merges(world, with_sinks):
    """fw_sharded_decode_step: the combine kernel writes the rank's state into
    every rank's exchange buffer as {value, epoch} pairs and the merge kernel
    reads them.  The ranks' buffers all live on this GPU; every rank first
    delivers (deliver_only), then every rank merges (fw_state_exchange_merge
    without a state), so no kernel waits for a later launch.  With one rank the
    whole step is one call.  The merge also advances the round-robin
    bookkeeping for the next step."""
    import torch
    from flywheel_tpu.softmax_attention import _native, distributed as d
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    rng = np.random.default_rng(40 + world)
    heads, kv_heads, dim, page, total_pages = 16, 4, 128, 64, 9
    length, steps = 2 * page + 62, 5            # the appending rank changes after two steps
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)
    keys, values = draw((total_pages * page, kv_heads, dim)), draw((total_pages * page, kv_heads, dim))
    rows = oracle.merge_kv_heads(keys, values).reshape(total_pages, page, 2 * kv_heads, dim)
    sinks = rng.standard_normal(heads).astype(np.float32) if with_sinks else None
    sinks_t = torch.from_numpy(sinks).to(dev) if with_sinks else None
    to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.bfloat16)

    nbytes = lib.fw_exchange_buffer_bytes(world, heads, dim)
    assert nbytes, _native.last_error()
    buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    peers = (ctypes.c_void_p * world)(*[b.data_ptr() for b in buffers])
    ranks = []
    for rank in range(world):
        owned = np.asarray(d.owned_pages(total_pages, world, rank))
        perm = np.random.default_rng(60 + rank).permutation(len(owned) + 2)[:len(owned)]
        pool = np.zeros((len(owned) + 2, page, 2 * kv_heads, dim), oracle.BF16)
        pool[perm] = rows[owned]
        state = dict(owned=owned, perm=perm, pool=to_t(pool),
                     table=torch.from_numpy(perm.astype(np.int32)[None]).to(dev),
                     counters=torch.tensor([length, 0, 0], dtype=torch.int32, device=dev), scratch=None,
                     out=torch.empty((1, 1, heads, dim), dtype=torch.bfloat16, device=dev),
                     lse=torch.empty((1, heads, 1), dtype=torch.float32, device=dev))
        base = state["counters"].data_ptr()
        prime = _native.FwShardStepArgs(global_len=base, local_len=base + 4, append_enable=base + 8,
                                        page_size=page, world=world, rank=rank, advance=0)
        _native.check(lib.fw_shard_step(ctypes.byref(prime), stream))
        ranks.append(state)

    for _ in range(steps):
        q, k, v = draw((1, 1, heads, dim)), draw((1, 1, kv_heads, dim)), draw((1, 1, kv_heads, dim))
        q_t, k_t, v_t = to_t(q), to_t(k), to_t(v)
        for rank, state in enumerate(ranks):
            base = state["counters"].data_ptr()
            args = _native.FwDecodeArgs(
                q=q_t.data_ptr(), out=state["out"].data_ptr(), lse=state["lse"].data_ptr(),
                kv_cache=state["pool"].data_ptr(), k_new=k_t.data_ptr(), v_new=v_t.data_ptr(),
                append_enable=base + 8, cache_seqlens=base + 4, block_table=state["table"].data_ptr(),
                sinks=sinks_t.data_ptr() if with_sinks else 0,
                num_pages=state["pool"].shape[0], page_size=page, pages_per_seq=state["table"].shape[1],
                batch=1, seqlen_q=1, nheads=heads, nheads_k=kv_heads, head_dim=dim, kv_dtype=0, causal=0,
                window_left=-1, softmax_scale=dim ** -0.5, softcap=0.0)
            if state["scratch"] is None:
                size = lib.fw_decode_workspace_bytes(ctypes.byref(args))
                assert size, _native.last_error()
                state["scratch"] = torch.zeros(size, dtype=torch.uint8, device=dev)
            args.workspace, args.workspace_bytes = state["scratch"].data_ptr(), state["scratch"].numel()
            whole = _native.FwShardedDecodeArgs(
                decode=args, peer_buffers=ctypes.cast(peers, ctypes.c_void_p), world=world, rank=rank,
                global_len=base, local_len=base + 4, append_enable=base + 8, advance=1,
                deliver_only=0 if world == 1 else 1)
            _native.check(lib.fw_sharded_decode_step(ctypes.byref(whole), stream))
        torch.cuda.synchronize()                # every state is delivered before any merge is enqueued
        if world > 1:
            for rank, state in enumerate(ranks):
                base = state["counters"].data_ptr()
                merge = _native.FwExchangeArgs(
                    peer_buffers=ctypes.cast(peers, ctypes.c_void_p), sinks=sinks_t.data_ptr() if with_sinks else 0,
                    out=state["out"].data_ptr(), lse=state["lse"].data_ptr(), status=state["scratch"].data_ptr(),
                    world=world, rank=rank, rows=heads, nheads=heads, head_dim=dim, lse_head_stride=1,
                    lse_token_stride=heads, global_len=base, local_len=base + 4, append_enable=base + 8,
                    page_size=page, advance=1)
                _native.check(lib.fw_state_exchange_merge(ctypes.byref(merge), stream))
            torch.cuda.synchronize()
        keys[length], values[length] = k[0, 0], v[0, 0]
        length += 1
        want, want_lse = oracle.attend_rows(
            q[0].astype(np.float32), keys[:length].astype(np.float32), values[:length].astype(np.float32),
            total=length, causal=True, window_left=None, softcap=0.0, scale=dim ** -0.5, sinks=sinks)
        first = ranks[0]["out"].view(torch.int16).cpu().numpy()
        for rank, state in enumerate(ranks):
            np.testing.assert_allclose(state["out"].float().cpu().numpy()[0], want, rtol=1e-2, atol=2e-2)
            np.testing.assert_allclose(state["lse"].cpu().numpy()[0, :, 0], want_lse[:, 0], rtol=2e-3, atol=4e-3)
            # every rank merges the same states in the same order: identical bits
            np.testing.assert_array_equal(state["out"].view(torch.int16).cpu().numpy(), first)
            total, local, appends = state["counters"].cpu().tolist()
            assert total == length
            assert local == d.local_length(length, page, world, rank)
            assert appends == int(d.owner_of_page(length // page, world) == rank)

    want_rows = oracle.merge_kv_heads(keys, values).reshape(total_pages, page, 2 * kv_heads, dim)
    for state in ranks:
        got = state["pool"].cpu().view(torch.int16).numpy()
        np.testing.assert_array_equal(got[state["perm"]], want_rows[state["owned"]].view(np.int16))
        assert _native.read_status(state["scratch"], dev) == 0


def test_merge_reports_a_state_that_never_arrives():
    """The merge's wait is bounded: with a peer that never delivers, the kernel
    gives up, reports FW_STATUS_WAIT_TIMEOUT and writes zero rows; the context
    stays usable."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    heads, dim, world = 8, 128, 2
    nbytes = lib.fw_exchange_buffer_bytes(world, heads, dim)
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=dev)       # nothing was ever delivered into it
    other = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    peers = (ctypes.c_void_p * world)(mine.data_ptr(), other.data_ptr())
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    out = torch.ones((heads, dim), dtype=torch.bfloat16, device=dev)
    lse = torch.zeros(heads, dtype=torch.float32, device=dev)
    merge = _native.FwExchangeArgs(
        peer_buffers=ctypes.cast(peers, ctypes.c_void_p), out=out.data_ptr(), lse=lse.data_ptr(),
        status=status.data_ptr(), world=world, rank=0, rows=heads, nheads=heads, head_dim=dim,
        lse_head_stride=1, lse_token_stride=heads)
    _native.check(lib.fw_state_exchange_merge(ctypes.byref(merge), stream))
    torch.cuda.synchronize()
    assert int(status[0].item()) & 1                                # FW_STATUS_WAIT_TIMEOUT
    assert float(out.float().abs().max().item()) == 0.0
    assert bool(torch.isinf(lse).all().item())
    assert int((torch.ones(4, device=dev) * 2).sum().item()) == 8   # the context still works


def test_fused_sharded_step_with_a_batch_of_one_token_requests():
    """The sharded step over a batch of one-token requests, two ranks played on
    one GPU: each rank holds half of every request's keys in its own pool; a
    request past num_active travels as the empty state and comes out as zero
    rows with lse = -inf."""
    import torch
    from flywheel_tpu.softmax_attention import _native
    lib = _native.library()
    dev = torch.device("cuda", torch.cuda.current_device())
    stream = torch.cuda.current_stream(dev).cuda_stream
    rng = np.random.default_rng(11)
    world, batch, active, heads, kv_heads, dim, page = 2, 3, 2, 8, 2, 128, 64
    lengths = [150, 64, 90]                      # whole-request key counts
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)
    keys = [draw((n, kv_heads, dim)) for n in lengths]
    values = [draw((n, kv_heads, dim)) for n in lengths]
    q = draw((batch, 1, heads, dim))
    to_t = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(dev).view(torch.bfloat16)
    q_t = to_t(q)
    nbytes = lib.fw_exchange_buffer_bytes(world, batch * heads, dim)
    buffers = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    peers = (ctypes.c_void_p * world)(*[b.data_ptr() for b in buffers])
    count = torch.tensor([active], dtype=torch.int32, device=dev)
    states = []
    for rank in range(world):
        pages_per_seq = 2
        pool = np.zeros((batch * pages_per_seq + 1, page, 2 * kv_heads, dim), oracle.BF16)
        table = np.arange(batch * pages_per_seq, dtype=np.int32).reshape(batch, pages_per_seq) + 1
        local = []
        for b, n in enumerate(lengths):
            lo, hi = (0, n // 2) if rank == 0 else (n // 2, n)
            rows = oracle.merge_kv_heads(keys[b][lo:hi], values[b][lo:hi])     # (tokens, 2 * kv_heads, dim)
            flat = pool[table[b]].reshape(pages_per_seq * page, 2 * kv_heads, dim)
            flat[:hi - lo] = rows
            pool[table[b]] = flat.reshape(pages_per_seq, page, 2 * kv_heads, dim)
            local.append(hi - lo)
        state = dict(pool=to_t(pool), table=torch.from_numpy(table).to(dev),
                     lens=torch.tensor(local, dtype=torch.int32, device=dev),
                     out=torch.full((batch, 1, heads, dim), 7.0, dtype=torch.bfloat16, device=dev),
                     lse=torch.zeros((batch, heads, 1), dtype=torch.float32, device=dev))
        args = _native.FwDecodeArgs(
            q=q_t.data_ptr(), out=state["out"].data_ptr(), lse=state["lse"].data_ptr(),
            kv_cache=state["pool"].data_ptr(), cache_seqlens=state["lens"].data_ptr(),
            block_table=state["table"].data_ptr(), num_active=count.data_ptr(),
            num_pages=pool.shape[0], page_size=page, pages_per_seq=pages_per_seq, batch=batch, seqlen_q=1,
            nheads=heads, nheads_k=kv_heads, head_dim=dim, kv_dtype=0, causal=0, window_left=-1,
            softmax_scale=dim ** -0.5, softcap=0.0)
        size = lib.fw_decode_workspace_bytes(ctypes.byref(args))
        assert size, _native.last_error()
        state["scratch"] = torch.zeros(size, dtype=torch.uint8, device=dev)
        args.workspace, args.workspace_bytes = state["scratch"].data_ptr(), size
        whole = _native.FwShardedDecodeArgs(decode=args, peer_buffers=ctypes.cast(peers, ctypes.c_void_p),
                                            world=world, rank=rank, deliver_only=1)
        _native.check(lib.fw_sharded_decode_step(ctypes.byref(whole), stream))
        states.append(state)
    torch.cuda.synchronize()
    for rank, state in enumerate(states):
        merge = _native.FwExchangeArgs(
            peer_buffers=ctypes.cast(peers, ctypes.c_void_p), out=state["out"].data_ptr(),
            lse=state["lse"].data_ptr(), status=state["scratch"].data_ptr(), world=world, rank=rank,
            rows=batch * heads, nheads=heads, head_dim=dim, lse_head_stride=1, lse_token_stride=heads)
        _native.check(lib.fw_state_exchange_merge(ctypes.byref(merge), stream))
    torch.cuda.synchronize()
    for state in states:
        got, got_lse = state["out"].float().cpu().numpy(), state["lse"].cpu().numpy()
        for b in range(active):
            want, want_lse = oracle.attend_rows(
                q[b].astype(np.float32), keys[b].astype(np.float32), values[b].astype(np.float32),
                total=lengths[b], causal=True, window_left=None, softcap=0.0, scale=dim ** -0.5, sinks=None)
            np.testing.assert_allclose(got[b], want, rtol=1e-2, atol=2e-2)
            np.testing.assert_allclose(got_lse[b, :, 0], want_lse[:, 0], rtol=2e-3, atol=4e-3)
        assert np.all(got[active:] == 0.0) and np.all(np.isneginf(got_lse[active:]))
        assert _native.read_status(state["scratch"], dev) == 0
