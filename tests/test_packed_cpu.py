"""CPU checks for the packed K/V path: the oracle's dense / packed-varlen
restatement against a naive einsum softmax (the construction of
tests/softmax_attention/util.py:181-273 of the reference, written out directly),
and the argument rejections of flash_attn_func / flash_attn_varlen_func, which
answer before any device is touched."""

import numpy as np
import pytest

from oracle import paged_attention as oracle


def naive_dense(q, k, v, causal, window, softcap, sinks):
    """q (b, sq, h, d), k / v (b, sk, hk, d) f32; window (left, right) with -1
    unbounded; masks bottom-right aligned."""
    b, sq, h, d = q.shape
    sk = k.shape[1]
    k, v = np.repeat(k, h // k.shape[2], axis=2), np.repeat(v, h // v.shape[2], axis=2)
    scores = np.einsum("bthd,bshd->bhts", q, k) / np.sqrt(d)
    if softcap:
        scores = np.tanh(scores / softcap) * softcap
    left, right = window
    if causal:
        right = 0
    row = np.arange(sq)[:, None] + sk - sq
    col = np.arange(sk)[None]
    masked = np.zeros((sq, sk), bool)
    if left >= 0:
        masked |= col < row - left
    if right >= 0:
        masked |= col > row + right
    logits = np.where(masked, -np.inf, scores)
    if sinks is not None:
        logits = np.concatenate([logits, np.broadcast_to(sinks[None, :, None, None], (b, h, sq, 1))], axis=-1)
    top = logits.max(axis=-1, keepdims=True)
    safe = np.where(np.isneginf(top), 0.0, top)
    weights = np.exp(logits - safe)
    denom = weights.sum(axis=-1, keepdims=True)
    probs = weights / np.where(denom == 0, 1.0, denom)
    out = np.einsum("bhts,bshd->bthd", probs[..., :sk], v)
    with np.errstate(divide="ignore"):
        lse = (safe + np.log(denom))[..., 0]
    return out, np.where(denom[..., 0] == 0, -np.inf, lse)


@pytest.mark.parametrize("sq,sk", [(1, 9), (7, 7), (12, 5), (5, 12)])
@pytest.mark.parametrize("causal,window", [(False, (-1, -1)), (True, (-1, -1)), (False, (3, 2)), (True, (4, -1)),
                                           (False, (-1, 0)), (False, (0, 0))])
@pytest.mark.parametrize("use_sinks", [False, True])
def test_dense_oracle_matches_naive_softmax(sq, sk, causal, window, use_sinks):
    rng = np.random.default_rng(sq * 31 + sk)
    q = rng.standard_normal((2, sq, 4, 16)).astype(np.float32)
    k = rng.standard_normal((2, sk, 2, 16)).astype(np.float32)
    v = rng.standard_normal((2, sk, 2, 16)).astype(np.float32)
    sinks = rng.standard_normal(4).astype(np.float32) if use_sinks else None
    softcap = 5.0 if sq % 2 else 0.0
    right = 0 if causal else window[1]
    got, got_lse = oracle.dense_attention(
        q, k, v, causal=causal or right == 0, window_left=None if window[0] < 0 else window[0],
        window_right=None if right <= 0 else right, softcap=softcap, sinks=sinks)
    want, want_lse = naive_dense(q, k, v, causal, window, softcap, sinks)
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(got_lse, want_lse, rtol=1e-5, atol=1e-5)


def test_packed_varlen_is_dense_per_sequence():
    rng = np.random.default_rng(4)
    lens_q, lens_k = (3, 0, 5), (6, 2, 5)
    cu_q, cu_k = np.concatenate(([0], np.cumsum(lens_q))), np.concatenate(([0], np.cumsum(lens_k)))
    q = rng.standard_normal((cu_q[-1] + 2, 4, 8)).astype(np.float32)
    k = rng.standard_normal((cu_k[-1], 2, 8)).astype(np.float32)
    v = rng.standard_normal((cu_k[-1], 2, 8)).astype(np.float32)
    out, lse = oracle.packed_varlen_attention(q, k, v, cu_q, cu_k, causal=True)
    for r in range(3):
        if lens_q[r] == 0:
            continue
        want, want_lse = naive_dense(q[None, cu_q[r]:cu_q[r + 1]], k[None, cu_k[r]:cu_k[r + 1]],
                                     v[None, cu_k[r]:cu_k[r + 1]], True, (-1, -1), 0.0, None)
        np.testing.assert_allclose(out[cu_q[r]:cu_q[r + 1]], want[0], rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(lse[:, cu_q[r]:cu_q[r + 1]], want_lse[0], rtol=1e-5, atol=1e-5)
    assert not out[cu_q[-1]:].any() and np.isneginf(lse[:, cu_q[-1]:]).all()


def test_packed_entry_points_reject_like_the_reference():
    import ml_dtypes
    from flywheel_tpu import flash_attn_func, flash_attn_varlen_func
    bf16 = np.dtype(ml_dtypes.bfloat16)
    q, k = np.zeros((1, 4, 8, 128), bf16), np.zeros((1, 4, 8, 128), bf16)
    with pytest.raises(NotImplementedError, match="dropout"):
        flash_attn_func(q, k, k, dropout_p=0.1)
    with pytest.raises(NotImplementedError, match="attention_chunk"):
        flash_attn_func(q, k, k, attention_chunk=4)
    with pytest.raises(NotImplementedError, match="bfloat16"):
        flash_attn_func(q.astype(np.float32), k, k)
    with pytest.raises(NotImplementedError, match="head_dim"):
        flash_attn_func(q[..., :32], k[..., :32], k[..., :32])
    with pytest.raises(ValueError, match="multiple of"):
        flash_attn_func(q, k[:, :3], k[:, :3])
    with pytest.raises(ValueError, match="head_dim is only meaningful"):
        flash_attn_func(q, k, k, head_dim=128)
    with pytest.raises(ValueError, match="head_dim="):
        flash_attn_func(q.reshape(1, 8, 512), k.reshape(1, 8, 512), k.reshape(1, 8, 512), token_major=True)
    with pytest.raises(ValueError, match="window_size"):
        flash_attn_func(q, k, k, window_size=(-3, 0))
    with pytest.raises(ValueError, match="rotary_k=False needs"):
        flash_attn_func(q, k, k, rotary_k=False)
    with pytest.raises(ValueError, match="provided together"):
        flash_attn_func(q, k, k, rotary_cos=np.zeros((8, 64), np.float32))
    with pytest.raises(ValueError, match="need block_table"):
        flash_attn_varlen_func(q[0], k[0], k[0], np.array([0, 8]), np.array([0, 8]), 8, 8, nheads_k=4)
    with pytest.raises(ValueError, match="need block_table"):
        flash_attn_varlen_func(q[0], k[0], k[0], np.array([0, 8]), np.array([0, 8]), 8, 8,
                               seqused_k=np.array([8]))
    with pytest.raises(ValueError, match="equal-shaped"):
        flash_attn_varlen_func(q[0], k[0], k[0], np.array([0, 8]), np.array([0, 4, 8]), 8, 8)
    with pytest.raises(ValueError, match="max_seqlen_k must be positive"):
        flash_attn_varlen_func(q[0], k[0], k[0], np.array([0, 8]), np.array([0, 8]), 8, 0)
