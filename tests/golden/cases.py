"""Seeded input constructions shared by the golden-vector generator and the
tests that replay it.  Shapes follow the reference's own paged test cases
(tests/softmax_attention/test_paged.py:39-77, 359-407, 483-495, 901-942 in the
reference project); values are drawn here, not copied."""

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)

# name -> dict(lengths, prefixes, heads, kv_heads, head_dim, page_size,
#              capacity, padding, causal, window_left, softcap, sinks, new)
CASES = {
    "ragged_causal": dict(lengths=(3, 0, 5), prefixes=(127, 0, 251), heads=4,
                          kv_heads=2, page_size=128, capacity=512, padding=7,
                          causal=True),
    "ragged_noncausal": dict(lengths=(3, 0, 5), prefixes=(127, 0, 251), heads=4,
                             kv_heads=2, page_size=128, capacity=512, padding=7,
                             causal=False),
    "multi_block": dict(lengths=(131, 17), prefixes=(123, 255), heads=4,
                        kv_heads=1, page_size=128, capacity=512, padding=3,
                        causal=True),
    "page64_gqa8": dict(lengths=(1, 1, 1, 1), prefixes=(63, 64, 200, 0),
                        heads=16, kv_heads=2, page_size=64, capacity=320,
                        padding=0, causal=True),
    "verify4_window": dict(lengths=(4, 4, 4), prefixes=(300, 61, 5), heads=8,
                           kv_heads=2, page_size=64, capacity=384, padding=0,
                           causal=True, window_left=100, softcap=50.0,
                           sinks=True),
    "empty_between": dict(lengths=(4, 3, 9, 2), prefixes=(0, 130, 0, 5),
                          heads=6, kv_heads=3, page_size=128, capacity=256,
                          padding=2, causal=True),
    "window_softcap": dict(lengths=(70, 30), prefixes=(150, 290), heads=4,
                           kv_heads=2, page_size=64, capacity=384, padding=1,
                           causal=True, window_left=127, softcap=30.0),
    "sinks_readonly": dict(lengths=(5, 2), prefixes=(40, 129), heads=8,
                           kv_heads=1, page_size=64, capacity=192, padding=0,
                           causal=True, sinks=True, new=False),
    "mha_window_nosoftcap": dict(lengths=(9, 1), prefixes=(100, 300), heads=4,
                                 kv_heads=4, page_size=128, capacity=384,
                                 padding=0, causal=True, window_left=31),
}


def build(name):
    """Inputs of one case: dict with q, k_pages, v_pages (separate f32-exact
    bf16 page arrays), k, v (or None), cu, lengths, table and the kwargs."""
    spec = dict(head_dim=128, padding=0, window_left=None, softcap=0.0,
                sinks=False, new=True)
    spec.update(CASES[name])
    rng = np.random.default_rng(sum(map(ord, name)))
    lengths, prefixes = spec["lengths"], spec["prefixes"]
    batch = len(lengths)
    heads, kv_heads, d = spec["heads"], spec["kv_heads"], spec["head_dim"]
    page_size, capacity = spec["page_size"], spec["capacity"]
    cu = np.concatenate(([0], np.cumsum(lengths))).astype(np.int32)
    total = int(cu[-1]) + spec["padding"]

    def normal(shape):
        return rng.standard_normal(shape, dtype=np.float32).astype(BF16)

    pages_per_seq = capacity // page_size
    q = normal((total, heads, d))
    k = normal((total, kv_heads, d))
    v = normal((total, kv_heads, d))
    table = rng.permutation(batch * pages_per_seq).reshape(
        batch, pages_per_seq).astype(np.int32)
    shape = (batch * pages_per_seq, page_size, kv_heads, d)
    sinks = (rng.uniform(-2, 8, heads).astype(np.float32)
             if spec["sinks"] else None)
    if not spec["new"]:
        k = v = None
    return dict(q=q, k_pages=normal(shape), v_pages=normal(shape), k=k, v=v,
                cu=cu, lengths=np.asarray(prefixes, np.int32), table=table,
                causal=spec["causal"], window_left=spec["window_left"],
                softcap=spec["softcap"], sinks=sinks, kv_heads=kv_heads)
