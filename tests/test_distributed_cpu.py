"""Host-side logic of the multi-GPU paths on CPU ranks (gloo, world size 2):
page partitioning, the packed (o, lse) all-gather layout, and the merge of the
gathered states, with the CPU oracle standing in for the per-rank kernel."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def test_round_robin_pages_cover_and_balance():
    from flywheel_tpu.softmax_attention import distributed as d
    for total in (1, 7, 8, 2049, 2052):
        for world in (1, 2, 4, 8):
            owned = [list(d.owned_pages(total, world, r)) for r in range(world)]
            assert sorted(page for pages in owned for page in pages) == list(range(total))
            sizes = [len(pages) for pages in owned]
            assert max(sizes) - min(sizes) <= 1
            for page in range(0, total, max(1, total // 50)):
                assert page in owned[d.owner_of_page(page, world)]
    # a rank's share of the first n tokens, against counting them one by one
    page = 64
    for world in (1, 2, 3, 8):
        for n in (0, 1, 63, 64, 65, 100, 500, 64 * world, 64 * world + 1, 4000):
            shares = [d.local_length(n, page, world, r) for r in range(world)]
            brute = [sum(1 for t in range(n) if (t // page) % world == r) for r in range(world)]
            assert shares == brute
            assert sum(shares) == n
    # the growing tail moves from rank to rank: over 8 pages of decode steps on 4
    # ranks every rank appends two pages' worth
    appends = [0] * 4
    for position in range(1000, 1000 + 8 * page):
        appends[d.owner_of_page(position // page, 4)] += 1
    assert appends == [2 * page] * 4


def _rank_main(rank, world, port, results):
    import sys
    import pathlib
    root = pathlib.Path(__file__).resolve().parent.parent
    for path in (root, root / "flywheel-tpu_b200"):
        if str(path) not in sys.path:
            sys.path.insert(0, str(path))
    from flywheel_tpu.softmax_attention import distributed as d
    from oracle import paged_attention as oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)            # same draws on every rank
        heads, kv_heads, dim, page, total_pages = 8, 2, 128, 64, 9
        length = 500                              # tokens cached; ends inside page 7
        keys = rng.standard_normal((total_pages * page, kv_heads, dim), dtype=np.float32)
        values = rng.standard_normal((total_pages * page, kv_heads, dim), dtype=np.float32)
        q = rng.standard_normal((1, heads, dim), dtype=np.float32)
        sinks = rng.standard_normal(heads).astype(np.float32)
        local = d.local_length(length, page, world, rank)
        # this rank's tokens: its pages in local order, the valid prefix of them
        mine = np.concatenate([np.arange(p * page, (p + 1) * page)
                               for p in d.owned_pages(total_pages, world, rank)])[:local]
        assert np.all(mine < length)
        out, lse = oracle.attend_rows(q, keys[mine], values[mine], total=local,
                                      causal=False, window_left=None, softcap=0.0,
                                      scale=dim ** -0.5, sinks=None)
        state = d.pack_state(torch.from_numpy(out[0]), torch.from_numpy(lse[:, 0].copy()))
        gathered = torch.empty(world * state.numel())
        dist.all_gather_into_tensor(gathered, state)
        outs, lses = d.unpack_states(gathered, world, heads, dim)
        merged, merged_lse = oracle.merge_states(outs.numpy(), lses.numpy(), sinks=sinks[None, :])
        want, want_lse = oracle.attend_rows(q, keys[:length], values[:length], total=length,
                                            causal=False, window_left=None, softcap=0.0,
                                            scale=dim ** -0.5, sinks=sinks)
        np.testing.assert_allclose(merged, want[0], rtol=1e-4, atol=1e-6)
        np.testing.assert_allclose(merged_lse, want_lse[:, 0], rtol=1e-5)
        owner = d.owner_of_page(length // page, world)
        results[rank] = (int(local), int(owner))
    finally:
        dist.destroy_process_group()


def test_sharded_state_gather_and_merge_on_two_cpu_ranks():
    world, port = 2, free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    assert results[0][0] + results[1][0] == 500
    assert results[0][1] == results[1][1] == 1      # position 500 is in page 7, an odd page: rank 1


def test_kv_head_and_request_sharding_partition_the_work():
    from flywheel_tpu.softmax_attention import distributed as d
    # KV-head sharding: disjoint slices that cover every head, groups kept together
    q_slices, kv_slices = zip(*(d.kv_head_shard(64, 8, 4, r) for r in range(4)))
    assert [s.start for s in kv_slices] == [0, 2, 4, 6] and kv_slices[-1].stop == 8
    assert [(s.start, s.stop) for s in q_slices] == [(0, 16), (16, 32), (32, 48), (48, 64)]
    with pytest.raises(ValueError):
        d.kv_head_shard(64, 8, 3, 0)
    # request sharding: every request exactly once, token loads within one request of each other
    rng = np.random.default_rng(0)
    lens = rng.integers(1024, 32769, 128)
    shards = [d.request_shard(lens, 8, r) for r in range(8)]
    assert sorted(i for shard in shards for i in shard) == list(range(128))
    loads = [int(lens[shard].sum()) for shard in shards]
    assert max(loads) - min(loads) <= int(lens.max())
