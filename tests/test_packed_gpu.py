"""GPU parity of attention over packed (non-paged) K/V: flash_attn_func and
flash_attn_varlen_func with cu_seqlens_k, against the CPU oracle.  Shapes and
options follow the reference's dense and varlen tests
(tests/softmax_attention/test_prefill.py:504-824 of the reference): MHA / GQA /
MQA, seqlen_q != seqlen_k with bottom-right alignment, causal / local, softcap,
sinks, both layouts, fused RoPE."""

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu

OUT_TOL = dict(rtol=1e-2, atol=2e-2)
LSE_TOL = dict(rtol=2e-3, atol=4e-3)
D = 128


def draw(rng, shape):
    return rng.standard_normal(shape, dtype=np.float32).astype(oracle.BF16)


def check(out, lse, want, want_lse):
    np.testing.assert_allclose(out.astype(np.float32), want, **OUT_TOL)
    finite = np.isfinite(want_lse)
    np.testing.assert_array_equal(np.isfinite(lse), finite)
    np.testing.assert_allclose(lse[finite], want_lse[finite], **LSE_TOL)


@pytest.mark.parametrize("hq,hk", [(4, 4), (8, 2), (8, 1), (16, 1), (6, 2), (6, 1), (10, 2), (14, 2), (12, 1), (32, 1), (64, 1), (128, 1)])
@pytest.mark.parametrize("sq,sk", [(1, 239), (113, 203), (128, 128), (256, 512), (300, 77), (1, 1)])
@pytest.mark.parametrize("causal,left", [(False, None), (True, None), (True, 64), (False, 100)])
def test_flash_attn_func_head_major(hq, hk, sq, sk, causal, left):
    from flywheel_tpu import flash_attn_func
    rng = np.random.default_rng(hq * 1000 + sq + sk)
    batch = 3
    q, k, v = draw(rng, (batch, hq, sq, D)), draw(rng, (batch, hk, sk, D)), draw(rng, (batch, hk, sk, D))
    sinks = rng.standard_normal(hq).astype(np.float32) if (sq + sk) % 2 else None
    softcap = 20.0 if sk % 2 else 0.0
    out, lse = flash_attn_func(q, k, v, causal=causal, window_size=(-1 if left is None else left, -1),
                               softcap=softcap, learnable_sink=sinks, return_softmax_lse=True)
    want, want_lse = oracle.dense_attention(
        q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3), causal=causal,
        window_left=left, softcap=softcap, sinks=sinks)
    check(out.transpose(0, 2, 1, 3), lse, want, want_lse)


@pytest.mark.parametrize("hq,hk", [(8, 2), (4, 4)])
@pytest.mark.parametrize("sq,sk", [(200, 200), (64, 1000)])
def test_flash_attn_func_token_major(hq, hk, sq, sk):
    from flywheel_tpu import flash_attn_func
    rng = np.random.default_rng(sq + sk + hq)
    batch = 2
    q, k, v = draw(rng, (batch, sq, hq, D)), draw(rng, (batch, sk, hk, D)), draw(rng, (batch, sk, hk, D))
    sinks = rng.standard_normal(hq).astype(np.float32)
    out, lse = flash_attn_func(q.reshape(batch, sq, hq * D), k.reshape(batch, sk, hk * D),
                               v.reshape(batch, sk, hk * D), causal=True, learnable_sink=sinks,
                               return_softmax_lse=True, head_dim=D, token_major=True)
    want, want_lse = oracle.dense_attention(q, k, v, causal=True, sinks=sinks)
    check(out.reshape(q.shape), lse, want, want_lse)


def test_flash_attn_func_without_lse_and_scale():
    from flywheel_tpu import flash_attn_func
    rng = np.random.default_rng(3)
    q, k, v = draw(rng, (1, 8, 500, D)), draw(rng, (1, 2, 500, D)), draw(rng, (1, 2, 500, D))
    out = flash_attn_func(q, k, v, softmax_scale=0.05, causal=True)
    want, _ = oracle.dense_attention(q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3),
                                     v.transpose(0, 2, 1, 3), causal=True, softmax_scale=0.05)
    np.testing.assert_allclose(out.astype(np.float32).transpose(0, 2, 1, 3), want, **OUT_TOL)


def ragged(rng, lens_q, lens_k, hq, hk, pad_q=7, pad_k=5):
    cu_q = np.concatenate(([0], np.cumsum(lens_q))).astype(np.int32)
    cu_k = np.concatenate(([0], np.cumsum(lens_k))).astype(np.int32)
    q = draw(rng, (int(cu_q[-1]) + pad_q, hq, D))
    k, v = draw(rng, (int(cu_k[-1]) + pad_k, hk, D)), draw(rng, (int(cu_k[-1]) + pad_k, hk, D))
    return q, k, v, cu_q, cu_k


@pytest.mark.parametrize("token_major", [False, True])
@pytest.mark.parametrize("causal,left,softcap", [(True, None, 0.0), (False, None, 15.0), (True, 90, 0.0)])
def test_varlen_packed(token_major, causal, left, softcap):
    from flywheel_tpu import flash_attn_varlen_func
    rng = np.random.default_rng(41)
    hq, hk = 8, 2
    lens_q, lens_k = (5, 128, 1, 260, 0, 33), (5, 300, 64, 260, 17, 129)
    q, k, v, cu_q, cu_k = ragged(rng, lens_q, lens_k, hq, hk)
    # NaN in the padding rows past cu_seqlens_k[-1] must not reach any output
    k[int(cu_k[-1]):], v[int(cu_k[-1]):] = np.nan, np.nan
    sinks = rng.standard_normal(hq).astype(np.float32)
    if token_major:
        args = (q.reshape(len(q), hq * D), k.reshape(len(k), hk * D), v.reshape(len(v), hk * D))
        kwargs = dict(head_dim=D, token_major=True)
    else:
        args = tuple(np.ascontiguousarray(x.transpose(1, 0, 2)) for x in (q, k, v))
        kwargs = {}
    out, lse = flash_attn_varlen_func(
        *args, cu_q, cu_k, max(lens_q), max(lens_k), causal=causal,
        window_size=(-1 if left is None else left, -1), softcap=softcap, learnable_sink=sinks,
        return_softmax_lse=True, **kwargs)
    want, want_lse = oracle.packed_varlen_attention(
        q, k, v, cu_q, cu_k, causal=causal, window_left=left, softcap=softcap, sinks=sinks)
    out = out.reshape(len(q), hq, D) if token_major else out.transpose(1, 0, 2)
    end = int(cu_q[-1])
    check(out[:end], lse[:, :end], want[:end], want_lse[:, :end])
    assert not out[end:].astype(np.float32).any() and np.isneginf(lse[:, end:]).all()


@pytest.mark.parametrize("rotary_k", [True, False])
@pytest.mark.parametrize("interleaved", [False, True])
def test_varlen_packed_rotary(rotary_k, interleaved):
    from flywheel_tpu import flash_attn_varlen_func
    rng = np.random.default_rng(9)
    hq, hk = 4, 2
    lens_q, lens_k = (40, 128, 7), (100, 128, 300)
    q, k, v, cu_q, cu_k = ragged(rng, lens_q, lens_k, hq, hk, pad_q=0, pad_k=0)
    angles = rng.uniform(0, 2 * np.pi, (max(lens_k), D // 2)).astype(np.float32)
    cos, sin = np.cos(angles), np.sin(angles)
    out, lse = flash_attn_varlen_func(
        *(np.ascontiguousarray(x.transpose(1, 0, 2)) for x in (q, k, v)), cu_q, cu_k, max(lens_q),
        max(lens_k), causal=True, return_softmax_lse=True, rotary_cos=cos, rotary_sin=sin,
        rotary_interleaved=interleaved, rotary_k=rotary_k)
    len_k = np.diff(cu_k)
    q_rot = oracle.rotate_packed_q(q, cos, sin, cu_q, len_k, interleaved=interleaved)
    k_rot = oracle.rotate_packed_q(k, cos, sin, cu_k, len_k, interleaved=interleaved) if rotary_k else k
    want, want_lse = oracle.packed_varlen_attention(q_rot, k_rot, v, cu_q, cu_k, causal=True)
    check(out.transpose(1, 0, 2), lse, want, want_lse)


def test_dense_rotary_matches_varlen_rule():
    from flywheel_tpu import flash_attn_func
    rng = np.random.default_rng(10)
    batch, hq, hk, sq, sk = 2, 4, 4, 96, 160
    q, k, v = draw(rng, (batch, hq, sq, D)), draw(rng, (batch, hk, sk, D)), draw(rng, (batch, hk, sk, D))
    angles = rng.uniform(0, 2 * np.pi, (sk, D // 2)).astype(np.float32)
    cos, sin = np.cos(angles), np.sin(angles)
    out = flash_attn_func(q, k, v, causal=True, rotary_cos=cos, rotary_sin=sin)
    qt, kt, vt = (x.transpose(0, 2, 1, 3) for x in (q, k, v))
    cu_q, cu_k = np.arange(batch + 1) * sq, np.arange(batch + 1) * sk
    q_rot = oracle.rotate_packed_q(qt.reshape(-1, hq, D), cos, sin, cu_q, np.full(batch, sk))
    k_rot = oracle.rotate_packed_q(kt.reshape(-1, hk, D), cos, sin, cu_k, np.full(batch, sk))
    want, _ = oracle.packed_varlen_attention(q_rot, k_rot, vt.reshape(-1, hk, D), cu_q, cu_k, causal=True)
    np.testing.assert_allclose(out.astype(np.float32).transpose(0, 2, 1, 3).reshape(-1, hq, D), want, **OUT_TOL)


@pytest.mark.parametrize("window", [(-1, 3), (50, 20), (0, 0), (7, 300), (200, 1)])
@pytest.mark.parametrize("sq,sk", [(160, 160), (90, 400), (300, 130)])
def test_two_sided_window(window, sq, sk):
    from flywheel_tpu import flash_attn_func
    rng = np.random.default_rng(sq + window[1])
    q, k, v = draw(rng, (2, 8, sq, D)), draw(rng, (2, 2, sk, D)), draw(rng, (2, 2, sk, D))
    out, lse = flash_attn_func(q, k, v, window_size=window, return_softmax_lse=True)
    want, want_lse = oracle.dense_attention(
        q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3),
        window_left=None if window[0] < 0 else window[0], window_right=window[1])
    check(out.transpose(0, 2, 1, 3), lse, want, want_lse)


@pytest.mark.parametrize("d", [64, 256])
@pytest.mark.parametrize("hq,hk", [(4, 4), (8, 2), (6, 1)])
@pytest.mark.parametrize("sq,sk,causal", [(150, 150, True), (64, 333, True), (257, 100, False), (1, 700, True)])
def test_other_head_dims(d, hq, hk, sq, sk, causal):
    from flywheel_tpu import flash_attn_func, flash_attn_varlen_func
    rng = np.random.default_rng(hq + sq + d)
    q, k, v = draw(rng, (2, hq, sq, d)), draw(rng, (2, hk, sk, d)), draw(rng, (2, hk, sk, d))
    sinks = rng.standard_normal(hq).astype(np.float32)
    angles = rng.uniform(0, 2 * np.pi, (max(sq, sk), d // 2)).astype(np.float32)
    out, lse = flash_attn_func(q, k, v, causal=causal, softcap=12.0, learnable_sink=sinks, return_softmax_lse=True)
    want, want_lse = oracle.dense_attention(
        q.transpose(0, 2, 1, 3), k.transpose(0, 2, 1, 3), v.transpose(0, 2, 1, 3), causal=causal, softcap=12.0,
        sinks=sinks)
    check(out.transpose(0, 2, 1, 3), lse, want, want_lse)
    if sq <= sk:
        # packed varlen, token-major, with fused RoPE on q and k
        cos, sin = np.cos(angles), np.sin(angles)
        qt, kt, vt = (np.ascontiguousarray(x.transpose(0, 2, 1, 3)) for x in (q, k, v))
        cu_q, cu_k = (np.arange(3) * sq).astype(np.int32), (np.arange(3) * sk).astype(np.int32)
        out2 = flash_attn_varlen_func(
            qt.reshape(2 * sq, hq * d), kt.reshape(2 * sk, hk * d), vt.reshape(2 * sk, hk * d), cu_q, cu_k, sq, sk,
            causal=causal, head_dim=d, token_major=True, rotary_cos=cos, rotary_sin=sin)
        q_rot = oracle.rotate_packed_q(qt.reshape(-1, hq, d), cos, sin, cu_q, np.full(2, sk))
        k_rot = oracle.rotate_packed_q(kt.reshape(-1, hk, d), cos, sin, cu_k, np.full(2, sk))
        want2, _ = oracle.packed_varlen_attention(q_rot, k_rot, vt.reshape(-1, hk, d), cu_q, cu_k, causal=causal)
        np.testing.assert_allclose(out2.astype(np.float32).reshape(-1, hq, d), want2, **OUT_TOL)


def test_rejections():
    from flywheel_tpu import flash_attn_func, flash_attn_varlen_func
    rng = np.random.default_rng(0)
    q, k = draw(rng, (1, 4, 8, D)), draw(rng, (1, 4, 8, D))
    with pytest.raises(NotImplementedError, match="head_dim"):
        flash_attn_func(q[..., :32], k[..., :32], k[..., :32])
    with pytest.raises(NotImplementedError, match="up to 128"):
        flash_attn_func(draw(rng, (1, 130, 8, D)), k[:, :1], k[:, :1])
    with pytest.raises(ValueError, match="head_dim="):
        flash_attn_func(q.reshape(1, 8, 4 * D), k.reshape(1, 8, 4 * D), k.reshape(1, 8, 4 * D), token_major=True)
    with pytest.raises(ValueError, match="need block_table"):
        flash_attn_varlen_func(q[0], k[0], k[0], np.array([0, 8]), np.array([0, 8]), 8, 8, nheads_k=4)
    with pytest.raises(ValueError, match="equal-shaped"):
        flash_attn_varlen_func(q[0], k[0], k[0], np.array([0, 8]), np.array([0, 4, 8]), 8, 8)
