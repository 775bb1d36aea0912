"""ctypes access to the C restatement (oracle/paged_decode_ref.c).  Test
infrastructure only: the checker and the timed CPU baseline."""

import ctypes
import pathlib
import subprocess

import numpy as np

ROOT = pathlib.Path(__file__).resolve().parent
LIBRARY = ROOT / "_build" / "libpaged_decode_ref.so"


def build(force=False):
    source = ROOT / "paged_decode_ref.c"
    if force or not LIBRARY.exists() or LIBRARY.stat().st_mtime < source.stat().st_mtime:
        LIBRARY.parent.mkdir(exist_ok=True)
        # -march=native is left out: the library is built on one machine and timed on another.
        subprocess.run(["gcc", "-O3", "-mavx2", "-mfma", "-fopenmp", "-shared", "-fPIC", "-o", str(LIBRARY),
                        str(source), "-lm"], check=True)
    return LIBRARY


def paged_decode(q, pool, k_new, v_new, cache_seqlens, block_table, *, nheads_k, causal=True,
                 window_left=None, softcap=0.0, softmax_scale=None, sinks=None, threads=None,
                 in_place=False):
    """Runs the C port.  q (batch, q_len, heads, d), pool merged bf16 (copied
    unless in_place; the updated pool is returned).  threads: OpenMP team size
    for this call (None = the runtime's own default).  Returns (out f32, lse
    (batch, heads, q_len), pool)."""
    lib = ctypes.CDLL(str(build()))
    batch, q_len, heads, d = q.shape
    pool = np.ascontiguousarray(pool) if in_place else np.ascontiguousarray(pool).copy()
    out = np.zeros((batch, q_len, heads, d), np.float32)
    lse = np.zeros((batch, heads, q_len), np.float32)
    ptr = lambda a: None if a is None else np.ascontiguousarray(a).ctypes.data_as(ctypes.c_void_p)
    keep = [np.ascontiguousarray(x) if x is not None else None
            for x in (q, k_new, v_new, np.asarray(cache_seqlens, np.int32), np.asarray(block_table, np.int32),
                      None if sinks is None else np.asarray(sinks, np.float32))]
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    lib.fw_ref_paged_decode.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int] * 9 + [ctypes.c_float] * 2 + [ctypes.c_int]
    lib.fw_ref_paged_decode(
        ptr(keep[0]), pool.ctypes.data_as(ctypes.c_void_p), ptr(keep[1]), ptr(keep[2]), ptr(keep[3]),
        ptr(keep[4]), ptr(keep[5]), out.ctypes.data_as(ctypes.c_void_p), lse.ctypes.data_as(ctypes.c_void_p),
        batch, q_len, heads, nheads_k, d, pool.shape[1], keep[4].shape[1], int(causal),
        -1 if window_left is None else int(window_left), ctypes.c_float(scale), ctypes.c_float(softcap),
        int(threads or 0))
    return out, lse, pool
