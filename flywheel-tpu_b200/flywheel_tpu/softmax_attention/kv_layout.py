"""Shape rules of the merged KV pool.

A token row of the pool is `[k0, v0, k1, v1, ...]`: KV head i's K plane at head
row 2i and its V plane at 2i + 1.  The reference moves rows as 32-bit words, so
a word holds one (K, V) pair of bf16 planes or two pairs of fp8 planes, and an
fp8 pool with an odd number of KV heads carries one extra zero head to fill the
last word (flywheel_tpu/softmax_attention/kv_layout.py:39-46, 67-95 of the
reference project).  The CUDA kernels address the same rows byte for byte.
"""

from flywheel_tpu.softmax_attention import _arrays

MERGED_KV_DTYPES = ("bfloat16", "float8_e4m3fn", "float8_e5m2")
_WORD_BYTES = 4


def check_merged_kv_dtype(dtype) -> None:
    name = _arrays.dtype_name(dtype)
    if name not in MERGED_KV_DTYPES:
        raise NotImplementedError(
            f"a merged KV pool is {', '.join(MERGED_KV_DTYPES)}; {name} is not"
            " one of them.")


def kv_heads_per_word(dtype) -> int:
    """How many KV heads' (K, V) pairs one 32-bit word of a row covers."""
    planes_per_word = _WORD_BYTES // _arrays.itemsize(dtype)
    return planes_per_word // 2


def merged_cache_heads(num_kv_heads: int, dtype) -> int:
    """Length of the pool's head axis for `num_kv_heads` KV heads: two planes
    per head, the head count first rounded up to whole words."""
    step = kv_heads_per_word(dtype)
    whole_words = (num_kv_heads + step - 1) // step
    return 2 * step * whole_words


def resolve_merged_kv_heads(cache_heads: int, dtype, nheads_k) -> int:
    """The KV head count behind a pool whose head axis is `cache_heads` long.

    `nheads_k` wins when given.  Without it a bf16 pool tells by itself (half
    its head axis); an fp8 pool does not, because of the pad head, and raises.
    Either way the pool must have exactly the head axis that count implies.
    """
    check_merged_kv_dtype(dtype)
    if nheads_k is None:
        if kv_heads_per_word(dtype) != 1:
            raise ValueError(
                "nheads_k is required for an fp8 pool: its head axis may include"
                " a pad head, so the KV head count cannot be read off the shape.")
        nheads_k = cache_heads // 2
    expected = merged_cache_heads(nheads_k, dtype)
    if expected != cache_heads:
        raise ValueError(
            f"{nheads_k} KV heads in {_arrays.dtype_name(dtype)} make"
            f" {expected} head rows per token, but the pool has {cache_heads}.")
    return nheads_k
