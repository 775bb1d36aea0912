"""Long-context decode with the KV pages split over 2 GPUs against the CPU
oracle, with both exchanges of the per-rank (o, lse) states: peer stores over
NVLink fused with the merge, and an NCCL all-gather + merge.  Needs 2 GPUs."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def free_port():
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _rank_main(rank, world, port, results, exchange):
    import sys
    import pathlib
    import ml_dtypes
    import torch.distributed as dist
    root = pathlib.Path(__file__).resolve().parent.parent
    for path in (root, root / "flywheel-tpu_b200"):
        if str(path) not in sys.path:
            sys.path.insert(0, str(path))
    from flywheel_tpu.softmax_attention import distributed as d
    from oracle import paged_attention as oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        bf16 = np.dtype(ml_dtypes.bfloat16)
        rng = np.random.default_rng(1)                      # same draws on every rank
        heads, kv_heads, dim, page, total_pages = 16, 2, 128, 64, 11
        length, steps = 4 * page + 60, 8                    # crosses a page edge, so the appending rank changes
        draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(bf16)
        keys, values = draw((total_pages * page, kv_heads, dim)), draw((total_pages * page, kv_heads, dim))
        sinks = rng.standard_normal(heads).astype(np.float32)
        owned = np.asarray(d.owned_pages(total_pages, world, rank))
        local_pages = len(owned)
        perm = np.random.default_rng(10 + rank).permutation(local_pages + 2)[:local_pages]
        pool = np.zeros((local_pages + 2, page, 2 * kv_heads, dim), bf16)
        rows = oracle.merge_kv_heads(keys, values).reshape(total_pages, page, 2 * kv_heads, dim)
        pool[perm] = rows[owned]
        pool_t = torch.from_numpy(pool.view(np.int16)).to(device).view(torch.bfloat16)
        table = torch.from_numpy(perm.astype(np.int32)[None]).to(device)
        decoder = d.ShardedDecoder(pool=pool_t, table=table, nheads=heads,
                                   nheads_k=kv_heads, sinks=torch.from_numpy(sinks).to(device),
                                   exchange=exchange)
        to_t = lambda a: torch.from_numpy(a.view(np.int16)).to(device).view(torch.bfloat16)
        worst = 0.0
        for step in range(steps):
            q, k, v = draw((1, 1, heads, dim)), draw((1, 1, kv_heads, dim)), draw((1, 1, kv_heads, dim))
            # the first step sets the cached length; afterwards the device counter carries on
            out, lse = decoder.step(to_t(q), to_t(k), to_t(v), length if step == 0 else None)
            torch.cuda.synchronize()
            keys[length], values[length] = k[0, 0], v[0, 0]
            length += 1
            want, want_lse = oracle.attend_rows(
                q[0].astype(np.float32), keys[:length].astype(np.float32),
                values[:length].astype(np.float32), total=length, causal=True, window_left=None,
                softcap=0.0, scale=dim ** -0.5, sinks=sinks)
            got = out.float().cpu().numpy()[0]
            np.testing.assert_allclose(got, want, rtol=1e-2, atol=2e-2)
            np.testing.assert_allclose(lse.cpu().numpy()[0, :, 0], want_lse[:, 0], rtol=2e-3, atol=4e-3)
            worst = max(worst, float(np.abs(got - want).max()))
        # appended rows landed bit-exact on the owning rank only
        got_pool = pool_t.cpu().view(torch.int16).numpy()
        want_rows = oracle.merge_kv_heads(keys, values).reshape(total_pages, page, 2 * kv_heads, dim)
        np.testing.assert_array_equal(got_pool[perm], want_rows[owned].view(np.int16))
        # the same step replayed as a CUDA graph: the cached length lives on the device
        # (peer-store exchange only: a capture right after eager NCCL work trips over
        # the process group's watchdog thread, which is not this library's concern)
        q, k, v = draw((1, 1, heads, dim)), draw((1, 1, kv_heads, dim)), draw((1, 1, kv_heads, dim))
        q_t, k_t, v_t = to_t(q), to_t(k), to_t(v)
        # 70 replays of one graph: the position crosses a page edge again, so the
        # appending rank changes under the captured launches
        replays = 70
        graph = decoder.capture(q_t, k_t, v_t, length) if exchange == "p2p" else None
        for replay in range(replays if graph is not None else 0):
            graph.replay()
            torch.cuda.synchronize()
            keys[length], values[length] = k[0, 0], v[0, 0]
            length += 1
            if replay % 23 and replay != replays - 1:
                continue
            want, _ = oracle.attend_rows(
                q[0].astype(np.float32), keys[:length].astype(np.float32),
                values[:length].astype(np.float32), total=length, causal=True, window_left=None,
                softcap=0.0, scale=dim ** -0.5, sinks=sinks)
            np.testing.assert_allclose(decoder.out.float().cpu().numpy()[0], want, rtol=1e-2, atol=2e-2)
        from flywheel_tpu.softmax_attention import _native
        assert _native.read_status(decoder.scratch, device) == 0
        decoder.close()
        results[rank] = worst
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("exchange", ["p2p", "nccl"])
def test_long_context_decode_split_over_two_gpus(exchange):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    world, port = 2, free_port()
    results = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, port, results, exchange), nprocs=world, join=True)
    assert len(results) == 2 and max(results.values()) < 2e-2
