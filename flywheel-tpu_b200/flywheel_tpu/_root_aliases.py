"""Internal names that are reachable from the package root for a serving
backend's sake.  They are not public API: every access warns."""

import importlib
import warnings

# name -> module that really owns it
HOMES = {
    "merged_cache_heads": "flywheel_tpu.softmax_attention.kv_layout",
    "write_kv_cache_pages": "flywheel_tpu.softmax_attention.page",
    "PAGE_SIZE_MULTIPLE": "flywheel_tpu.softmax_attention.config",
    "NUM_LANES": "flywheel_tpu.core.tiling",
}


def resolve(package: str, name: str):
    """The object `package.name` stands for, or AttributeError."""
    try:
        home = HOMES[name]
    except KeyError:
        raise AttributeError(f"module {package!r} has no attribute {name!r}") from None
    warnings.warn(
        f"{package}.{name} is an internal name (it lives in {home}); it may move"
        " or disappear without notice.", FutureWarning, stacklevel=3)
    return getattr(importlib.import_module(home), name)
