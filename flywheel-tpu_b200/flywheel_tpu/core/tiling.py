"""Tile constants of the B200 kernels and integer helpers
(the reference keeps TPU lane counts here: flywheel_tpu/core/tpu.py:18-27,
core/tiling.py:18-20)."""

# Tokens one decode pipeline stage stages per TMA copy; page sizes and
# contiguous capacities are multiples of it.
DECODE_TILE_TOKENS = 16
# Kept for callers that size buffers in multiples of the reference's lane count.
NUM_LANES = 128


def round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple
