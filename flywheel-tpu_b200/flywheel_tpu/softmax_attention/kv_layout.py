"""Merged KV-cache layout: a token row holds each KV head's K row then its V
row, [k0, v0, k1, v1, ...], for bf16 and fp8; an fp8 pool pads an odd head
count with one zero head (flywheel_tpu/softmax_attention/kv_layout.py:39-46,
67-95 of the reference project)."""

from flywheel_tpu.softmax_attention import _arrays

MERGED_KV_DTYPES = ("bfloat16", "float8_e4m3fn", "float8_e5m2")


def check_merged_kv_dtype(dtype) -> None:
    if _arrays.dtype_name(dtype) not in MERGED_KV_DTYPES:
        raise NotImplementedError(
            "the merged KV cache holds bfloat16, float8_e4m3fn or float8_e5m2;"
            f" got {_arrays.dtype_name(dtype)}."
        )


def kv_heads_per_word(dtype) -> int:
    """KV heads whose (K, V) pair fills one 32-bit word: 1 for bf16, 2 for
    fp8."""
    return (4 // _arrays.itemsize(dtype)) // 2


def merged_cache_heads(num_kv_heads: int, dtype) -> int:
    """Head rows of one merged-cache token: 2 * num_kv_heads, padded to whole
    32-bit words."""
    per_word = kv_heads_per_word(dtype)
    return 2 * (-(-num_kv_heads // per_word) * per_word)


def resolve_merged_kv_heads(cache_heads: int, dtype, nheads_k) -> int:
    """KV heads of a merged cache whose tokens hold cache_heads head rows:
    nheads_k, else half the rows of a bf16 cache."""
    check_merged_kv_dtype(dtype)
    if nheads_k is not None:
        num_kv_heads = nheads_k
    elif kv_heads_per_word(dtype) > 1:
        raise ValueError(
            "an fp8 cache pads an odd nheads_k, so its head axis does not give"
            " the KV head count; pass nheads_k."
        )
    else:
        num_kv_heads = cache_heads // 2
    if merged_cache_heads(num_kv_heads, dtype) != cache_heads:
        raise ValueError(
            f"a merged {_arrays.dtype_name(dtype)} cache of {num_kv_heads} KV heads"
            f" holds {merged_cache_heads(num_kv_heads, dtype)} head rows per"
            f" token; got {cache_heads}."
        )
    return num_kv_heads
