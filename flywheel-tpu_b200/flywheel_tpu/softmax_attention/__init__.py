"""The flash-attention entry points, served by the B200 CUDA kernels."""

from flywheel_tpu.softmax_attention import decode, packed, prefill

flash_attn_with_kvcache = decode.flash_attn_with_kvcache
flash_attn_varlen_func = prefill.flash_attn_varlen_func
flash_attn_func = packed.flash_attn_func

__all__ = ["flash_attn_func", "flash_attn_varlen_func", "flash_attn_with_kvcache"]
