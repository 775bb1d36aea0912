"""The C restatement (timed CPU baseline) against the NumPy oracle."""

import numpy as np
import pytest

from oracle import c_port
from oracle import paged_attention as oracle


@pytest.mark.parametrize("kwargs", [
    dict(), dict(window_left=40, softcap=30.0), dict(sinks=True), dict(q_len=4), dict(append=False)])
def test_c_port_matches_numpy_oracle(kwargs):
    import paged_cases as workloads
    q_len = kwargs.get("q_len", 1)
    case = workloads.host_case(41, lens=(0, 63, 64, 300), q_len=q_len, hq=8, hk=2)
    rng = np.random.default_rng(2)
    sinks = rng.uniform(-2, 6, 8).astype(np.float32) if kwargs.get("sinks") else None
    k, v = (case.k_new, case.v_new) if kwargs.get("append", True) else (None, None)
    common = dict(nheads_k=2, causal=True, window_left=kwargs.get("window_left"),
                  softcap=kwargs.get("softcap", 0.0), sinks=sinks)
    want, want_lse, want_pool = oracle.kvcache_paged(case.q, case.pool, k, v, case.cache_seqlens,
                                                     case.block_table, **common)
    got, got_lse, got_pool = c_port.paged_decode(case.q, case.pool, k, v, case.cache_seqlens,
                                                 case.block_table, **common)
    np.testing.assert_allclose(got, want, rtol=2e-4, atol=2e-5)
    finite = np.isfinite(want_lse)
    np.testing.assert_array_equal(np.isfinite(got_lse), finite)
    np.testing.assert_allclose(got_lse[finite], want_lse[finite], rtol=1e-4, atol=1e-4)
    np.testing.assert_array_equal(got_pool.view(np.uint16), want_pool.view(np.uint16))
