"""Seeded input constructions shared by the golden-vector generator and the
tests that replay it.  Shapes follow the reference's own paged test cases
(tests/softmax_attention/test_paged.py:39-77, 359-407, 483-495, 901-942 in the
reference project); values are drawn here, not copied."""

import ml_dtypes
import numpy as np

BF16 = np.dtype(ml_dtypes.bfloat16)
E4M3 = np.dtype(ml_dtypes.float8_e4m3fn)
E5M2 = np.dtype(ml_dtypes.float8_e5m2)
KV_DTYPES = {"bf16": BF16, "e4m3": E4M3, "e5m2": E5M2}

# name -> dict(lengths, prefixes, heads, kv_heads, head_dim, page_size,
#              capacity, padding, causal, window_left, softcap, sinks, new,
#              kv_dtype, descale)
# fp8 cases follow the reference's fp8 tests (tests/softmax_attention/
# test_prefill.py:606-625 of the reference project): the cache stores x / descale
# cast to the fp8 type and the reference attends stored * descale.  descale
# "pow2" uses that test's power-of-two pair (2^-3 for K, 2^-2 for V); "amax" is
# the per-tensor amax / largest-finite scale a serving engine would pick.
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
    "fp8_e4m3_pow2_decode": dict(lengths=(1, 1, 1, 1), prefixes=(63, 64, 200, 0),
                                 heads=16, kv_heads=2, page_size=64, capacity=320,
                                 causal=True, kv_dtype="e4m3", descale="pow2"),
    "fp8_e5m2_pow2_ragged": dict(lengths=(3, 0, 5), prefixes=(100, 0, 251), heads=4,
                                 kv_heads=2, page_size=128, capacity=512,
                                 padding=2, causal=True, kv_dtype="e5m2",
                                 descale="pow2"),
    # the serving verify-window configuration in small: window 4095, softcap 50,
    # sinks, 4 query tokens per request, 64-token pages, amax descales
    "fp8_e4m3_amax_verify4": dict(lengths=(4, 4, 4, 4), prefixes=(5000, 4095, 4092, 70),
                                  heads=16, kv_heads=2, page_size=64, capacity=5120,
                                  causal=True, window_left=4095, softcap=50.0,
                                  sinks=True, kv_dtype="e4m3", descale="amax"),
    "fp8_e5m2_amax_window": dict(lengths=(70, 30), prefixes=(150, 290), heads=4,
                                 kv_heads=2, page_size=64, capacity=384, padding=1,
                                 causal=True, window_left=127, softcap=30.0,
                                 kv_dtype="e5m2", descale="amax"),
    # three KV heads: the fp8 pool carries a zero pad head
    "fp8_e4m3_odd_heads": dict(lengths=(4, 3, 9, 2), prefixes=(0, 130, 0, 5),
                               heads=6, kv_heads=3, page_size=128, capacity=256,
                               padding=2, causal=True, sinks=True, kv_dtype="e4m3",
                               descale="amax"),
    "fp8_e4m3_readonly_mqa": dict(lengths=(5, 2), prefixes=(40, 129), heads=8,
                                  kv_heads=1, page_size=64, capacity=192,
                                  causal=True, sinks=True, new=False,
                                  kv_dtype="e4m3", descale="pow2"),
}


def build(name):
    """Inputs of one case: dict with q, k_pages, v_pages (separate f32-exact
    bf16 page arrays), k, v (or None), cu, lengths, table and the kwargs."""
    spec = dict(head_dim=128, padding=0, window_left=None, softcap=0.0,
                sinks=False, new=True, kv_dtype="bf16", descale=None)
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
    k_pages, v_pages = normal(shape), normal(shape)
    kv_dtype = KV_DTYPES[spec["kv_dtype"]]
    k_descale = v_descale = 1.0
    if kv_dtype != BF16:
        # stored = x / descale cast to the cache type; the new rows use the same scales
        limit = float(ml_dtypes.finfo(kv_dtype).max)
        if spec["descale"] == "pow2":
            k_descale, v_descale = 2.0 ** -3, 2.0 ** -2
        else:
            k_descale = float(np.abs(k_pages.astype(np.float32)).max()) / limit
            v_descale = float(np.abs(v_pages.astype(np.float32)).max()) / limit

        def store(x, descale):
            scaled = x.astype(np.float32) / np.float32(descale)
            return np.clip(scaled, -limit, limit).astype(kv_dtype)

        k_pages, v_pages = store(k_pages, k_descale), store(v_pages, v_descale)
        k, v = store(k, k_descale), store(v, v_descale)
    if not spec["new"]:
        k = v = None
    return dict(q=q, k_pages=k_pages, v_pages=v_pages, k=k, v=v,
                cu=cu, lengths=np.asarray(prefixes, np.int32), table=table,
                causal=spec["causal"], window_left=spec["window_left"],
                softcap=spec["softcap"], sinks=sinks, kv_heads=kv_heads,
                kv_dtype=kv_dtype, k_descale=k_descale, v_descale=v_descale)


def dequantized(case):
    """The f32 pages and new rows the reference's NumPy oracle is handed for an
    fp8 case: stored * descale (for bf16 the values themselves)."""
    f32 = lambda x, scale: None if x is None else x.astype(np.float32) * np.float32(scale)
    return (f32(case["k_pages"], case["k_descale"]), f32(case["v_pages"], case["v_descale"]),
            f32(case["k"], case["k_descale"]), f32(case["v"], case["v_descale"]))


def stored_bits(pages_f32, case, which):
    """Bit patterns of f32 pages brought back to the cache type (pages / descale
    cast down): what the pool must hold after the append."""
    scale = np.float32(case["k_descale"] if which == "k" else case["v_descale"])
    stored = (np.asarray(pages_f32, np.float32) / scale).astype(case["kv_dtype"])
    carrier = np.uint16 if case["kv_dtype"].itemsize == 2 else np.uint8
    return np.ascontiguousarray(stored).view(carrier)
