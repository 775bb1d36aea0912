"""FlyWheel's paged-KV softmax attention entry points on B200 (sm_100a).

Drop-in for the serving path of heavyball-research/flywheel-tpu: the names,
arguments and layouts of ``flywheel_tpu.flash_attn_with_kvcache`` and
``flywheel_tpu.flash_attn_varlen_func(block_table=...)`` are kept
(flywheel_tpu/__init__.py:20-32 of the reference project); the kernels behind
them are hand-written CUDA reached through a C ABI.  There is no CPU path: a
call without the compiled library or without a CUDA device raises.
"""

import importlib
import warnings

from flywheel_tpu.softmax_attention import (
    flash_attn_func,
    flash_attn_varlen_func,
    flash_attn_with_kvcache,
)

__version__ = "0.4.1+b200"

__all__ = [
    "flash_attn_func",
    "flash_attn_varlen_func",
    "flash_attn_with_kvcache",
]

# Internal names a serving backend imports from the package root
# (flywheel_tpu/__init__.py:39-45 of the reference project); each access warns.
INTERNAL_EXPORTS = {
    "PAGE_SIZE_MULTIPLE": "flywheel_tpu.softmax_attention.config",
    "NUM_LANES": "flywheel_tpu.core.tiling",
    "merged_cache_heads": "flywheel_tpu.softmax_attention.kv_layout",
    "write_kv_cache_pages": "flywheel_tpu.softmax_attention.page",
}


def __getattr__(name: str):
    module_name = INTERNAL_EXPORTS.get(name)
    if module_name is None:
        raise AttributeError(f"module 'flywheel_tpu' has no attribute {name!r}")
    warnings.warn(
        f"flywheel_tpu.{name} is internal ({module_name}.{name}): it is not"
        " public API and may move or be removed.",
        FutureWarning,
        stacklevel=2,
    )
    return getattr(importlib.import_module(module_name), name)
