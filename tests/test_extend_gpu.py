"""A mixed serving step through paged_extend / fw_extend_mixed: page write, then
the decode kernel over the leading one-token requests and the paged prefill over
the rest, against the CPU oracle on the whole batch (the routine mirrors
flywheel_tpu_extend, patches/tpu-inference.patch:8219-8320 of the reference
project)."""

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu

OUT_TOL = dict(rtol=1e-2, atol=2e-2)
FP8_TOL = dict(rtol=1e-2, atol=5e-2)


def to_cuda(array):
    import torch
    if array.dtype == oracle.BF16:
        return torch.from_numpy(array.view(np.int16)).cuda().view(torch.bfloat16)
    if array.dtype == oracle.E4M3:
        return torch.from_numpy(array.view(np.uint8)).cuda().view(torch.float8_e4m3fn)
    return torch.from_numpy(array).cuda()


def mixed_step(seed, decode_lens, prefill, *, hq=16, hk=4, page=64, dtype=oracle.BF16, idle_slots=2, padding=5):
    """decode_lens: cached lengths of the one-token requests; prefill: (prefix,
    chunk) pairs.  Returns the inputs of one step and the slice table that writes
    its tokens."""
    rng = np.random.default_rng(seed)
    d = 128
    before = np.array(list(decode_lens) + [p for p, _ in prefill] + [0] * idle_slots, np.int32)
    new = np.array([1] * len(decode_lens) + [c for _, c in prefill] + [0] * idle_slots, np.int32)
    after = before + new
    batch = len(before)
    cu = np.concatenate(([0], np.cumsum(new))).astype(np.int32)
    total = int(cu[-1]) + padding
    pages_b = np.maximum(1, -(-after // page))
    perm = rng.permutation(int(pages_b.sum()) + 3)
    table = np.full((batch, int(pages_b.max()) + 1), -1, np.int32)
    cursor = 0
    for r, n in enumerate(pages_b):
        table[r, :n] = perm[cursor:cursor + n]
        cursor += n
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32)
    kd = vd = 1.0
    if dtype == oracle.BF16:
        cast = lambda x, s: x.astype(oracle.BF16)
    else:
        kd, vd = 2.0 ** -3, 2.0 ** -2
        cast = lambda x, s: (x / np.float32(s)).astype(dtype)
    shape = (len(perm), page, hk, d)
    pool = oracle.merge_kv_heads(cast(draw(shape), kd), cast(draw(shape), vd))
    q = draw((total, hq, d)).astype(oracle.BF16)
    k, v = cast(draw((total, hk, d)), kd), cast(draw((total, hk, d)), vd)
    columns = []
    for r in range(batch):
        pos, row = int(before[r]), int(cu[r])
        while pos < after[r]:
            run = min(int(after[r]) - pos, page - pos % page)
            columns.append((int(table[r, pos // page]) * page + pos % page, row, run))
            pos, row = pos + run, row + run
    slices = np.zeros((3, len(columns) + 4), np.int32)
    slices[:, :len(columns)] = np.array(columns, np.int32).T
    return dict(q=q, k=k, v=v, pool=pool, before=before, after=after, cu=cu, table=table, slices=slices,
                num_slices=len(columns), num_decode=len(decode_lens), num_active=len(decode_lens) + len(prefill),
                hk=hk, kd=kd, vd=vd)


@pytest.mark.parametrize("decode_lens,prefill", [
    ((700, 0, 63, 64, 1500), ((0, 130), (200, 70), (1000, 300))),
    ((33,) * 40, ((10, 64),)),            # many decode rows, one chunk
    ((), ((0, 200), (300, 65))),          # prefill only
    ((5, 900, 128), ()),                  # decode only
])
def test_mixed_step_matches_the_oracle(decode_lens, prefill):
    from flywheel_tpu.softmax_attention import _arrays
    from flywheel_tpu.softmax_attention.extend import paged_extend
    c = mixed_step(41, decode_lens, prefill)
    pool_t = to_cuda(c["pool"])
    out, cache = paged_extend(c["q"], c["k"], c["v"], pool_t, c["after"], c["table"], c["cu"], c["slices"],
                              c["num_slices"], c["num_decode"], c["num_active"])
    assert cache is pool_t
    want_pool = oracle.append_to_pool(c["pool"], c["k"], c["v"], c["cu"], c["before"], c["table"], nheads_k=c["hk"])
    np.testing.assert_array_equal(_arrays.to_host_numpy(pool_t).view(np.uint16), want_pool.view(np.uint16))
    want, _ = oracle.ragged_paged_attention(c["q"], want_pool, c["cu"], c["after"], c["table"], nheads_k=c["hk"],
                                            causal=True, num_active=c["num_active"])
    np.testing.assert_allclose(out.astype(np.float32), want, **OUT_TOL)
    assert not out[int(c["cu"][c["num_active"]]):].astype(np.float32).any()


def test_mixed_step_options_and_prewritten_pool():
    """fp8 pool with descales, a left window, softcap and sinks; and the same step
    with the pool written beforehand (k = v = None)."""
    from flywheel_tpu.softmax_attention.extend import paged_extend
    c = mixed_step(42, (300, 64, 2000), ((100, 90), (0, 257)), hq=8, hk=2, dtype=oracle.E4M3)
    sinks = np.random.default_rng(1).uniform(-2, 8, 8).astype(np.float32)
    kwargs = dict(window_left=150, softcap=30.0, learnable_sink=sinks, k_descale=c["kd"], v_descale=c["vd"],
                  nheads_k=2)
    want_pool = oracle.append_to_pool(c["pool"], c["k"], c["v"], c["cu"], c["before"], c["table"], nheads_k=2)
    want, _ = oracle.ragged_paged_attention(
        c["q"], want_pool, c["cu"], c["after"], c["table"], nheads_k=2, causal=True, window_left=150,
        softcap=30.0, sinks=sinks, k_descale=c["kd"], v_descale=c["vd"], num_active=c["num_active"])
    out, _ = paged_extend(c["q"], c["k"], c["v"], to_cuda(c["pool"]), c["after"], c["table"], c["cu"], c["slices"],
                          c["num_slices"], c["num_decode"], c["num_active"], **kwargs)
    np.testing.assert_allclose(out.astype(np.float32), want, **FP8_TOL)
    out2, _ = paged_extend(c["q"], None, None, to_cuda(want_pool), c["after"], c["table"], c["cu"], None, None,
                           c["num_decode"], c["num_active"], **kwargs)
    np.testing.assert_allclose(out2.astype(np.float32), want, **FP8_TOL)
