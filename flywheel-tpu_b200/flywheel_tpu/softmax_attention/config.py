"""Static limits of the B200 kernels."""

from flywheel_tpu.core.tiling import DECODE_TILE_TOKENS

# The reference needs page_size % 128 == 0
# (flywheel_tpu/softmax_attention/config.py:40); these kernels stage 16-token
# tiles, so any multiple of 16 works (64-token pages included).
PAGE_SIZE_MULTIPLE = DECODE_TILE_TOKENS
# Query rows per KV head (seqlen_q * nheads / nheads_k) the decode kernel takes
# in one launch; the reference folds a verify window up to the same bound
# (decode.py:49-53).
MAX_FOLDED_QUERY_ROWS = 128


def max_folded_query_rows(head_dim: int) -> int:
    """The bound above at head_dim 128; half of it at 256, where a warp's
    registers hold twice the output columns."""
    return MAX_FOLDED_QUERY_ROWS if head_dim <= 128 else MAX_FOLDED_QUERY_ROWS // 2
SUPPORTED_HEAD_DIMS = (128, 256)
# The decode kernel (single token, folded verify window) also takes head_dim 64
# with a bf16 cache, like the reference's (traits.py:50, 473-477 there); the
# paged prefill kernels need head_dim % 128 == 0, as the reference's do.
DECODE_HEAD_DIMS = (64, 128, 256)
# Rows one decode launch takes; the host entry slices larger batches.
MAX_DECODE_BATCH = 2048
