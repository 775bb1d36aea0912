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
