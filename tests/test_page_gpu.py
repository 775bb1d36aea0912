"""write_kv_cache_pages against the CPU oracle, bit for bit (the reference's
own check: tests/softmax_attention/test_page.py:32-69 of the reference)."""

import numpy as np
import pytest

from oracle import paged_attention as oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [oracle.BF16, oracle.E4M3, oracle.E5M2])
@pytest.mark.parametrize("nheads_k", [1, 2, 3, 8])
def test_write_kv_cache_pages(dtype, nheads_k):
    import torch
    from flywheel_tpu.softmax_attention.kv_layout import merged_cache_heads
    from flywheel_tpu.softmax_attention.page import write_kv_cache_pages
    rng = np.random.default_rng(5)
    num_pages, page_size, d = 6, 128, 128
    draw = lambda shape: rng.standard_normal(shape, dtype=np.float32).astype(dtype)
    cache = draw((num_pages, page_size, merged_cache_heads(nheads_k, dtype), d))
    k, v = draw((300, nheads_k, d)), draw((300, nheads_k, d))
    # a page tail, a whole page and a page head, out of token order; unused columns hold junk
    pieces = [(4 * page_size + 100, 0, 28), (1 * page_size, 28, 128), (3 * page_size, 156, 100)]
    slices = np.full((3, 8), 7, np.int32)
    for column, piece in enumerate(pieces):
        slices[:, column] = piece
    want = oracle.write_kv_cache_pages(cache, k, v, slices, [len(pieces)])
    carrier = np.int16 if dtype == oracle.BF16 else np.uint8
    out = write_kv_cache_pages(k, v, cache, slices, np.array([len(pieces)], np.int32))
    np.testing.assert_array_equal(out.view(carrier), want.view(carrier))
    # device-resident cache: updated in place
    torch_dtype = {oracle.BF16: torch.bfloat16, oracle.E4M3: torch.float8_e4m3fn,
                   oracle.E5M2: torch.float8_e5m2}[dtype]
    cache_t = torch.from_numpy(cache.view(carrier)).cuda().view(torch_dtype)
    assert write_kv_cache_pages(k, v, cache_t, slices, np.array([len(pieces)], np.int32)) is cache_t
    np.testing.assert_array_equal(
        cache_t.cpu().view(torch.int16 if dtype == oracle.BF16 else torch.uint8).numpy(), want.view(carrier))


def test_internal_exports_warn():
    import flywheel_tpu
    with pytest.warns(FutureWarning):
        assert flywheel_tpu.write_kv_cache_pages is not None
    with pytest.warns(FutureWarning):
        assert flywheel_tpu.PAGE_SIZE_MULTIPLE == 16
