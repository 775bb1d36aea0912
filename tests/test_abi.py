"""The C-ABI library loads and exports every symbol include/flywheel_b200.h
declares; argument validation answers without touching a GPU."""

import ctypes
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent


def declared_symbols():
    header = (ROOT / "include" / "flywheel_b200.h").read_text()
    return sorted(set(re.findall(r"\b(fw_[a-z_0-9]+)\s*\(", header)))


def test_library_exports_every_declared_symbol():
    from flywheel_tpu.softmax_attention import _native
    lib = _native.library()
    names = declared_symbols()
    assert {"fw_decode_kvcache", "fw_append_ragged", "fw_prefill_paged",
            "fw_lse_combine", "fw_last_error", "fw_version"} <= set(names)
    for name in names:
        assert getattr(lib, name) is not None, name
    assert set(names) == set(_native.EXPORTS), set(names) ^ set(_native.EXPORTS)


def test_struct_layouts_match_the_header(tmp_path):
    """Every ctypes mirror has the size and the field offsets a C compiler gives
    the struct declared in the header."""
    import subprocess
    from flywheel_tpu.softmax_attention import _native
    structs = ["FwDecodeArgs", "FwAppendArgs", "FwWritePagesArgs", "FwPrefillArgs", "FwCombineArgs",
               "FwExchangeArgs", "FwShardStepArgs", "FwShardedDecodeArgs", "FwExtendArgs"]
    lines = ['#include <stddef.h>', '#include <stdio.h>', '#include "flywheel_b200.h"', 'int main(void) {']
    for name in structs:
        lines.append(f'  printf("{name} %zu\\n", sizeof({name}));')
        for field, _ in getattr(_native, name)._fields_:
            lines.append(f'  printf("{name}.{field} %zu\\n", offsetof({name}, {field}));')
    lines += ['  return 0;', '}']
    source = tmp_path / "layout.c"
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(ROOT / "include"), "-o", str(binary), str(source)], check=True)
    want = dict(line.split() for line in subprocess.run([str(binary)], check=True, capture_output=True,
                                                        text=True).stdout.splitlines())
    for name in structs:
        mirror = getattr(_native, name)
        assert ctypes.sizeof(mirror) == int(want[name]), name
        for field, _ in mirror._fields_:
            assert getattr(mirror, field).offset == int(want[f"{name}.{field}"]), f"{name}.{field}"


def test_argument_errors_mirror_reference_exception_types():
    from flywheel_tpu.softmax_attention import _native
    lib = _native.library()
    args = _native.FwDecodeArgs(batch=2, seqlen_q=1, nheads=6, nheads_k=4, head_dim=128,
                                block_table=1, page_size=64, pages_per_seq=2, num_pages=4)
    assert lib.fw_decode_workspace_bytes(ctypes.byref(args)) == 0
    assert "multiple of nheads_k" in _native.last_error()
    with pytest.raises(ValueError):
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), None))
    args.nheads_k, args.kv_dtype = 2, 7
    with pytest.raises(NotImplementedError):
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), None))
    args.kv_dtype, args.page_size = 0, 40
    with pytest.raises(ValueError, match="page_size"):
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), None))
    args.page_size, args.head_dim = 64, 96
    with pytest.raises(NotImplementedError, match="head_dim"):
        _native.check(lib.fw_decode_kvcache(ctypes.byref(args), None))


def test_host_api_rejections_follow_the_reference():
    import numpy as np
    import ml_dtypes
    from flywheel_tpu import flash_attn_with_kvcache, flash_attn_varlen_func
    bf16 = np.dtype(ml_dtypes.bfloat16)
    q = np.zeros((2, 1, 4, 128), bf16)
    pool = np.zeros((4, 64, 4, 128), bf16)
    table = np.zeros((2, 2), np.int32)
    with pytest.raises(ValueError, match="v_cache=None"):
        flash_attn_with_kvcache(q, pool, pool, cache_seqlens=1, block_table=table)
    with pytest.raises(ValueError, match="mutually exclusive"):
        flash_attn_with_kvcache(q, pool, None, cache_seqlens=1, block_table=table,
                                cache_batch_idx=np.zeros(2, np.int32))
    with pytest.raises(NotImplementedError, match="paged merged"):
        flash_attn_with_kvcache(np.zeros((2, 3, 4, 128), bf16), pool, pool, cache_seqlens=1)
    with pytest.raises(ValueError, match="window_size"):
        flash_attn_with_kvcache(q, pool, None, cache_seqlens=1, block_table=table,
                                window_size=(-2, 0))
    with pytest.raises(NotImplementedError, match="bfloat16"):
        flash_attn_with_kvcache(q.astype(np.float32), pool, None, cache_seqlens=1,
                                block_table=table)
    with pytest.raises(ValueError, match="passed together"):
        flash_attn_with_kvcache(q, pool, None, np.zeros((2, 1, 2, 128), bf16), None,
                                cache_seqlens=1, block_table=table)
    with pytest.raises(ValueError, match="head rows per"):
        flash_attn_with_kvcache(q, pool, None, cache_seqlens=1, block_table=table, nheads_k=3)
    with pytest.raises(ValueError, match="max_seqlen_q"):
        flash_attn_with_kvcache(np.zeros((5, 4, 128), bf16), pool, None, cache_seqlens=1,
                                block_table=table, cu_seqlens_q=np.array([0, 2, 5], np.int32))
    with pytest.raises(ValueError, match="seqused_k"):
        flash_attn_varlen_func(np.zeros((4, 5, 128), bf16), pool, None,
                               np.array([0, 2, 5], np.int32), None, 3, 64, block_table=table)
    with pytest.raises(NotImplementedError, match="right bound"):
        flash_attn_varlen_func(np.zeros((4, 5, 128), bf16), pool, None,
                               np.array([0, 2, 5], np.int32), None, 3, 64, block_table=table,
                               seqused_k=np.array([3, 4], np.int32), window_size=(-1, 5))


def test_exchange_and_packed_entry_points_validate_without_a_gpu():
    from flywheel_tpu.softmax_attention import _native
    lib = _native.library()
    # exchange buffer: header + 2 parities x world slots of rows * (d + 1) {value, epoch} pairs,
    # slots 16-byte aligned
    assert lib.fw_exchange_buffer_bytes(4, 64, 128) == 4096 + 2 * 4 * 64 * 129 * 8
    assert lib.fw_exchange_buffer_bytes(2, 5, 128) == 4096 + 2 * 2 * (5 * 129 + 1) * 8
    assert lib.fw_exchange_buffer_bytes(0, 64, 128) == 0 and "world" in _native.last_error()
    assert lib.fw_exchange_buffer_bytes(2, 64, 96) == 0
    swap = _native.FwExchangeArgs(world=2, rank=0, rows=64, nheads=64, head_dim=128)
    with pytest.raises(ValueError, match="must not be NULL"):
        _native.check(lib.fw_state_exchange_merge(ctypes.byref(swap), None))
    peers = (ctypes.c_void_p * 2)(1, 0)
    swap = _native.FwExchangeArgs(peer_buffers=ctypes.cast(peers, ctypes.c_void_p), state_out=1, state_lse=1,
                                  out=1, world=2, rank=3, rows=64, nheads=64, head_dim=128)
    with pytest.raises(ValueError, match="rank inside"):
        _native.check(lib.fw_state_exchange_merge(ctypes.byref(swap), None))
    swap.rank = 1
    with pytest.raises(ValueError, match=r"peer_buffers\[1\]"):
        _native.check(lib.fw_state_exchange_merge(ctypes.byref(swap), None))
    swap.state_lse = 0
    with pytest.raises(ValueError, match="passed together"):
        _native.check(lib.fw_state_exchange_merge(ctypes.byref(swap), None))

    # the fused sharded step validates the same way
    step = _native.FwShardedDecodeArgs(world=2, rank=0)
    with pytest.raises(ValueError, match="peer_buffers must not be NULL"):
        _native.check(lib.fw_sharded_decode_step(ctypes.byref(step), None))
    step.peer_buffers = ctypes.cast(peers, ctypes.c_void_p)
    step.decode = _native.FwDecodeArgs(batch=2, seqlen_q=2, nheads=8, nheads_k=4, head_dim=128, block_table=1,
                                       page_size=64, pages_per_seq=2, num_pages=4)
    with pytest.raises(NotImplementedError, match="one request"):
        _native.check(lib.fw_sharded_decode_step(ctypes.byref(step), None))
    step.decode.batch, step.decode.partial_out = 1, 1
    with pytest.raises(ValueError, match="partial_out / partial_lse must be NULL"):
        _native.check(lib.fw_sharded_decode_step(ctypes.byref(step), None))

    packed = _native.FwPrefillArgs(batch=1, total_q=8, total_k=8, nheads=4, nheads_k=4, head_dim=128,
                                   kv_cache=1, v_packed=1, cu_seqlens_q=1, cu_seqlens_k=1, q=1, out=1,
                                   softmax_scale=0.1)
    assert lib.fw_attention_packed_workspace_bytes(ctypes.byref(packed)) > 0
    packed.head_dim = 96
    with pytest.raises(NotImplementedError, match="head_dim"):
        _native.check(lib.fw_attention_packed(ctypes.byref(packed), None))
    packed.head_dim, packed.block_table = 128, 1
    with pytest.raises(ValueError, match="paged cache"):
        _native.check(lib.fw_attention_packed(ctypes.byref(packed), None))
    packed.block_table, packed.kv_dtype = 0, 1
    with pytest.raises(NotImplementedError, match="bfloat16"):
        _native.check(lib.fw_attention_packed(ctypes.byref(packed), None))
    packed.kv_dtype, packed.nheads = 0, 4 * 130
    with pytest.raises(NotImplementedError, match="up to 128"):
        _native.check(lib.fw_attention_packed(ctypes.byref(packed), None))
    # head_dim 64 is a packed-K/V size only
    paged = _native.FwPrefillArgs(batch=1, total_q=8, nheads=4, nheads_k=4, head_dim=64, block_table=1,
                                  page_size=64, pages_per_seq=1, num_pages=1, softmax_scale=0.1)
    assert lib.fw_prefill_workspace_bytes(ctypes.byref(paged)) == 0
    assert "head_dim 64" in _native.last_error()
