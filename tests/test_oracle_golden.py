"""Pins the CPU oracle: (1) against golden vectors produced by executing the
reference's own NumPy test oracle (tests/golden/make_golden.py), (2) against
the deterministic known-answer constructions of the reference's tests."""

import hashlib

import numpy as np
import pytest

import cases
from oracle import paged_attention as oracle



def load(name):
    import pathlib
    path = pathlib.Path(cases.__file__).resolve().parent / f"{name}.npz"
    return np.load(path)


def digest(pages):
    carrier = np.uint16 if pages.dtype.itemsize == 2 else np.uint8
    bits = np.ascontiguousarray(pages).view(carrier)
    return np.frombuffer(hashlib.sha256(bits.tobytes()).digest(), np.uint8)


def run_oracle(case):
    pool = oracle.merge_kv_heads(case["k_pages"], case["v_pages"])
    cu, lengths = case["cu"], case["lengths"]
    if case["k"] is not None:
        out, lse, new_pool = oracle.kvcache_paged(
            case["q"], pool, case["k"], case["v"], lengths, case["table"],
            nheads_k=case["kv_heads"], cu_seqlens_q=cu, causal=case["causal"],
            window_left=case["window_left"], softcap=case["softcap"],
            sinks=case["sinks"], k_descale=case["k_descale"], v_descale=case["v_descale"])
    else:
        out, lse = oracle.ragged_paged_attention(
            case["q"], pool, cu, lengths, case["table"],
            nheads_k=case["kv_heads"], causal=case["causal"],
            window_left=case["window_left"], softcap=case["softcap"],
            sinks=case["sinks"], k_descale=case["k_descale"], v_descale=case["v_descale"])
        new_pool = pool
    return out, lse, new_pool


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_oracle_matches_reference_numpy_oracle(name):
    case = cases.build(name)
    golden = load(name)
    out, lse, new_pool = run_oracle(case)
    np.testing.assert_allclose(out, golden["out"], rtol=1e-5, atol=2e-6)
    finite = np.isfinite(golden["lse"])
    np.testing.assert_array_equal(np.isfinite(lse), finite)
    np.testing.assert_allclose(lse[finite], golden["lse"][finite],
                               rtol=1e-5, atol=1e-5)
    k_pages, v_pages = oracle.split_kv_heads(new_pool, case["kv_heads"])
    np.testing.assert_array_equal(digest(k_pages), golden["k_pages_sha256"])
    np.testing.assert_array_equal(digest(v_pages), golden["v_pages_sha256"])


def test_merge_layout_order_and_fp8_padding():
    # [k0, v0, k1, v1, ...]; an odd fp8 head count pads one zero head
    # (reference tests/softmax_attention/util.py:40-52).
    k = np.arange(3 * 4, dtype=np.float32).reshape(1, 3, 4)
    v = -k
    merged = oracle.merge_kv_heads(k.astype(oracle.BF16), v.astype(oracle.BF16))
    assert merged.shape == (1, 6, 4)
    np.testing.assert_array_equal(merged[0, 0::2].astype(np.float32), k[0])
    np.testing.assert_array_equal(merged[0, 1::2].astype(np.float32), v[0])
    merged8 = oracle.merge_kv_heads(k.astype(oracle.E4M3), v.astype(oracle.E4M3))
    assert merged8.shape == (1, 8, 4)
    assert oracle.merged_cache_heads(3, oracle.E4M3) == 8
    np.testing.assert_array_equal(merged8[0, 6:].view(np.uint8), 0)
    k2, v2 = oracle.split_kv_heads(merged8, 3)
    np.testing.assert_array_equal(k2.view(np.uint8),
                                  k.astype(oracle.E4M3).view(np.uint8))
    np.testing.assert_array_equal(v2.view(np.uint8),
                                  v.astype(oracle.E4M3).view(np.uint8))


def test_append_moves_bits_not_values():
    # NaN payloads and subnormals survive the append (kv_layout.py:98-111).
    pool = np.zeros((2, 64, 2, 128), oracle.BF16)
    bits = np.array([0x7FC1, 0xFFFF, 0x0001, 0x8000], np.uint16)
    k = np.tile(bits, 32).view(oracle.BF16).reshape(1, 1, 128)
    v = np.tile(bits[::-1], 32).view(oracle.BF16).reshape(1, 1, 128)
    out = oracle.append_to_pool(pool, k, v, [0, 1], [70], [[1, 0]], 1)
    np.testing.assert_array_equal(out[0, 6, 0].view(np.uint16), k.view(np.uint16)[0, 0])
    np.testing.assert_array_equal(out[0, 6, 1].view(np.uint16), v.view(np.uint16)[0, 0])
    changed = out.view(np.uint16) != pool.view(np.uint16)
    assert changed.sum() == changed[0, 6].sum()


def test_known_answer_two_level_keys():
    # Keys 0 then 32 (scores), values 1 then 3: the high-score keys dominate,
    # so out -> 3 (construction of test_paged.py:667-688 in the reference).
    d, n = 128, 2048
    q = np.ones((1, 1, d), np.float32)
    keys = np.zeros((n, 1, d), np.float32)
    keys[1024:] = 32.0 * np.sqrt(d) / d
    values = np.ones((n, 1, d), np.float32)
    values[1024:] = 3.0
    out, lse = oracle.attend_rows(q, keys, values, total=n, causal=True,
                                  window_left=None, softcap=0.0,
                                  scale=1 / np.sqrt(d), sinks=None)
    np.testing.assert_allclose(out, 3.0, atol=1e-5)
    np.testing.assert_allclose(lse, 32.0 + np.log(1024.0), rtol=1e-6)


def test_sink_identity():
    # out_s = out * sigmoid(lse - sink); lse_s = logaddexp(lse, sink)
    # (identity checked by test_paged.py:1190-1229 in the reference).
    rng = np.random.default_rng(3)
    q = rng.standard_normal((3, 4, 128), dtype=np.float32)
    keys = rng.standard_normal((50, 2, 128), dtype=np.float32)
    values = rng.standard_normal((50, 2, 128), dtype=np.float32)
    sinks = rng.uniform(-2, 8, 4).astype(np.float32)
    kw = dict(total=50, causal=True, window_left=None, softcap=0.0,
              scale=128 ** -0.5)
    out, lse = oracle.attend_rows(q, keys, values, sinks=None, **kw)
    out_s, lse_s = oracle.attend_rows(q, keys, values, sinks=sinks, **kw)
    gate = 1 / (1 + np.exp(-(lse - sinks[:, None])))
    np.testing.assert_allclose(out_s, out * gate.T[:, :, None], rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(lse_s, np.logaddexp(lse, sinks[:, None]), rtol=1e-5)


def test_merge_states_equals_joint_attention():
    rng = np.random.default_rng(5)
    q = rng.standard_normal((1, 8, 128), dtype=np.float32)
    keys = rng.standard_normal((96, 2, 128), dtype=np.float32)
    values = rng.standard_normal((96, 2, 128), dtype=np.float32)
    sinks = rng.standard_normal(8).astype(np.float32)
    kw = dict(causal=False, window_left=None, softcap=0.0, scale=128 ** -0.5)
    full, full_lse = oracle.attend_rows(q, keys, values, total=96, sinks=sinks, **kw)
    parts = [oracle.attend_rows(q, keys[a:b], values[a:b], total=b - a,
                                sinks=None, **kw)
             for a, b in ((0, 40), (40, 41), (41, 96))]
    empty = (np.zeros_like(full), np.full_like(full_lse, -np.inf))
    outs = np.stack([p[0] for p in parts] + [empty[0]])
    lses = np.stack([p[1].T for p in parts] + [empty[1].T])     # (parts, 1, heads)
    out, lse = oracle.merge_states(outs, lses, sinks=sinks[None, :])
    np.testing.assert_allclose(out, full, rtol=1e-4, atol=1e-6)
    np.testing.assert_allclose(lse, full_lse.T, rtol=1e-5)
    out0, lse0 = oracle.merge_states(empty[0][None], empty[1].T[None])
    assert not out0.any() and np.isneginf(lse0).all()


def test_contiguous_decode_matches_paged_view():
    rng = np.random.default_rng(11)
    b, cap, hk, hq, d = 3, 128, 2, 8, 128
    kc = rng.standard_normal((4, cap, hk, d), dtype=np.float32).astype(oracle.BF16)
    vc = rng.standard_normal((4, cap, hk, d), dtype=np.float32).astype(oracle.BF16)
    q = rng.standard_normal((b, 1, hq, d), dtype=np.float32).astype(oracle.BF16)
    k = rng.standard_normal((b, 1, hk, d), dtype=np.float32).astype(oracle.BF16)
    v = rng.standard_normal((b, 1, hk, d), dtype=np.float32).astype(oracle.BF16)
    lengths = np.array([0, 17, 127], np.int32)
    rows = np.array([2, 0, 3], np.int32)
    out, lse, kc2, vc2 = oracle.kvcache_contiguous(
        q, kc, vc, k, v, lengths, rows, causal=True)
    pool = oracle.merge_kv_heads(kc, vc)            # one page per cache row
    out_p, lse_p, pool2 = oracle.kvcache_paged(
        q, pool, k, v, lengths, rows[:, None], nheads_k=hk, causal=True)
    np.testing.assert_allclose(out, out_p, rtol=1e-6)
    np.testing.assert_allclose(lse, lse_p, rtol=1e-6)
    k2, v2 = oracle.split_kv_heads(pool2, hk)
    np.testing.assert_array_equal(k2.view(np.uint16), kc2.view(np.uint16))
    np.testing.assert_array_equal(v2.view(np.uint16), vc2.view(np.uint16))


def test_write_kv_cache_pages_oracle():
    pool = np.zeros((3, 4, 4, 8), oracle.BF16)
    k = np.arange(5 * 2 * 8, dtype=np.float32).reshape(5, 2, 8).astype(oracle.BF16)
    v = (-k.astype(np.float32)).astype(oracle.BF16)
    slices = np.array([[9, 2], [0, 3], [3, 2]], np.int32)      # two pieces
    out = oracle.write_kv_cache_pages(pool, k, v, slices, [2])
    flat = out.reshape(12, 4, 8)
    np.testing.assert_array_equal(flat[9:12, 0::2].astype(np.float32), k[0:3].astype(np.float32))
    np.testing.assert_array_equal(flat[2:4, 1::2].astype(np.float32), v[3:5].astype(np.float32))
    untouched = np.ones(12, bool)
    untouched[[9, 10, 11, 2, 3]] = False
    assert not flat[untouched].view(np.uint16).any()
    assert not oracle.write_kv_cache_pages(pool, k, v, slices, [0]).view(np.uint16).any()


def test_rotate_packed_q_positions_and_norm():
    rng = np.random.default_rng(9)
    q = rng.standard_normal((6, 2, 128), dtype=np.float32)
    angle = rng.random((40, 64)) * 2 * np.pi
    cos, sin = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    cu, seqused = np.array([0, 2, 5]), np.array([10, 3])
    for interleaved in (False, True):
        out = oracle.rotate_packed_q(q, cos, sin, cu, seqused, interleaved)
        np.testing.assert_allclose(np.linalg.norm(out[:5], axis=-1), np.linalg.norm(q[:5], axis=-1), rtol=1e-5)
        np.testing.assert_array_equal(out[5], q[5])            # row of no request
    out = oracle.rotate_packed_q(q, cos, sin, cu, seqused, False)
    pos = 8                                                    # token 0 of request 0: 10 - 2 + 0
    x1, x2 = q[0, 0, :64], q[0, 0, 64:]
    np.testing.assert_allclose(out[0, 0, :64], x1 * cos[pos] - x2 * sin[pos], rtol=1e-6)
    np.testing.assert_allclose(out[0, 0, 64:], x1 * sin[pos] + x2 * cos[pos], rtol=1e-6)
