"""The entry points without PyTorch: a child process in which `import torch`
fails calls them with NumPy arrays only (device memory through libcudart, see
flywheel_tpu/softmax_attention/_cuda.py) and checks the results against the CPU
oracle.  The reference takes JAX arrays; nothing in this package may depend on
one particular array library."""

import pathlib
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parent.parent

CHILD = r'''
import sys
sys.modules["torch"] = None                      # any `import torch` now raises ImportError
for path in ("{root}", "{root}/flywheel-tpu_b200", "{root}/tests", "{root}/tests/golden"):
    sys.path.insert(0, path)
import numpy as np
import cases
import paged_cases
from oracle import paged_attention as oracle
from flywheel_tpu import flash_attn_with_kvcache, flash_attn_varlen_func, flash_attn_func
from flywheel_tpu.softmax_attention.extend import paged_extend
from flywheel_tpu.softmax_attention.page import write_kv_cache_pages

# decode with the fused append: paged bf16, sinks, lse; the updated pool comes back as NumPy
case = paged_cases.host_case(71, lens=(0, 63, 64, 900, 2500), hq=32, hk=4, page_size=64)
sinks = np.linspace(-1, 3, 32).astype(np.float32)
out, lse, pool = flash_attn_with_kvcache(
    case.q, case.pool, None, case.k_new, case.v_new, cache_seqlens=case.cache_seqlens,
    block_table=case.block_table, causal=True, return_softmax_lse=True, learnable_sink=sinks)
assert isinstance(out, np.ndarray) and isinstance(pool, np.ndarray)
want, want_lse, want_pool = oracle.kvcache_paged(
    case.q, case.pool, case.k_new, case.v_new, case.cache_seqlens, case.block_table, nheads_k=4,
    causal=True, sinks=sinks)
np.testing.assert_array_equal(pool.view(np.uint16), want_pool.view(np.uint16))
np.testing.assert_allclose(out.astype(np.float32), want, rtol=1e-2, atol=2e-2)
np.testing.assert_allclose(lse, want_lse, rtol=2e-3, atol=4e-3)

# an fp8 verify window on the decode kernel and the packed (append + prefill) route, from the golden cases
for name, q_len in (("fp8_e4m3_amax_verify4", 4), ("multi_block", None)):
    c = cases.build(name)
    golden = np.load("{root}/tests/golden/" + name + ".npz")
    fp8 = c["kv_dtype"] != oracle.BF16
    extra = dict(k_descale=c["k_descale"], v_descale=c["v_descale"], nheads_k=c["kv_heads"]) if fp8 else {{}}
    pool = oracle.merge_kv_heads(c["k_pages"], c["v_pages"])
    window = (-1 if c["window_left"] is None else c["window_left"], -1)
    if q_len:
        shape = (len(c["lengths"]), q_len, -1, 128)
        out, lse, _ = flash_attn_with_kvcache(
            c["q"].reshape(shape), pool, None, c["k"].reshape(shape), c["v"].reshape(shape),
            cache_seqlens=c["lengths"], block_table=c["table"], causal=c["causal"], softcap=c["softcap"],
            window_size=window, learnable_sink=c["sinks"], return_softmax_lse=True, **extra)
        np.testing.assert_allclose(out.astype(np.float32), golden["out"].reshape(out.shape), rtol=1e-2, atol=5e-2)
    else:
        out, lse, _ = flash_attn_with_kvcache(
            c["q"], pool, None, c["k"], c["v"], cache_seqlens=c["lengths"], block_table=c["table"],
            cu_seqlens_q=c["cu"], max_seqlen_q=int(np.diff(c["cu"]).max()), causal=c["causal"],
            return_softmax_lse=True, **extra)
        np.testing.assert_allclose(out.astype(np.float32), golden["out"], rtol=1e-2, atol=2e-2)
        finite = np.isfinite(golden["lse"])
        np.testing.assert_allclose(lse[finite], golden["lse"][finite], rtol=2e-3, atol=4e-3)

# chunked prefill over the pool, read only
c = cases.build("window_softcap")
golden = np.load("{root}/tests/golden/window_softcap.npz")
pool = oracle.append_to_pool(oracle.merge_kv_heads(c["k_pages"], c["v_pages"]), c["k"], c["v"], c["cu"],
                             c["lengths"], c["table"], nheads_k=c["kv_heads"])
seqused = c["lengths"] + np.diff(c["cu"]).astype(np.int32)
out = flash_attn_varlen_func(
    np.ascontiguousarray(c["q"].transpose(1, 0, 2)), pool, None, c["cu"], None, int(np.diff(c["cu"]).max()),
    int(seqused.max()), causal=True, softcap=c["softcap"], window_size=(c["window_left"], -1),
    block_table=c["table"], seqused_k=seqused)
np.testing.assert_allclose(out.astype(np.float32).transpose(1, 0, 2), golden["out"], rtol=1e-2, atol=2e-2)

# dense attention over packed K/V
rng = np.random.default_rng(5)
q, k, v = (rng.standard_normal((2, 4, 200, 128), dtype=np.float32).astype(oracle.BF16) for _ in range(3))
out = flash_attn_func(q, k, v, causal=True)
want, _ = oracle.dense_attention(*(x.transpose(0, 2, 1, 3) for x in (q, k, v)), causal=True)   # token-major there
np.testing.assert_allclose(out.astype(np.float32), want.transpose(0, 2, 1, 3), rtol=1e-2, atol=2e-2)
assert sys.modules.get("torch") is None
print("ok without torch")
'''


def test_entry_points_run_without_torch():
    result = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT)], capture_output=True, text=True,
                            timeout=600)
    assert result.returncode == 0, result.stdout + result.stderr
    assert "ok without torch" in result.stdout
