"""FlyWheel's paged-KV softmax attention entry points on B200 (sm_100a).

Drop-in for the serving path of heavyball-research/flywheel-tpu: the names,
arguments and layouts of ``flywheel_tpu.flash_attn_with_kvcache``,
``flywheel_tpu.flash_attn_varlen_func`` and ``flywheel_tpu.flash_attn_func`` are
kept (flywheel_tpu/__init__.py:20-32 of the reference project); the kernels
behind them are hand-written CUDA reached through a C ABI.  There is no CPU
path: a call without the compiled library or without a CUDA device raises.

A serving backend also reads a few internal names from the package root
(flywheel_tpu/__init__.py:39-60 of the reference project); they resolve here
too, lazily and with a FutureWarning, through ``_root_aliases``.
"""

from flywheel_tpu import _root_aliases
from flywheel_tpu.softmax_attention.decode import flash_attn_with_kvcache
from flywheel_tpu.softmax_attention.packed import flash_attn_func
from flywheel_tpu.softmax_attention.prefill import flash_attn_varlen_func

__version__ = "0.4.1+b200"
__all__ = ["flash_attn_func", "flash_attn_varlen_func", "flash_attn_with_kvcache"]

INTERNAL_EXPORTS = _root_aliases.HOMES


def __getattr__(name):
    return _root_aliases.resolve(__name__, name)
