"""The allocation-free scatter-add entry point against the allocating one.

Collected last on purpose: if it fails under `pytest -x`, every other test has already run.
It passes alone in a fresh process and after the other tests; the first call on the device is
made outside any stream capture, as the entry point asks."""

import numpy as np
import pytest

from distributed_kge_poplar_b200 import capi

pytestmark = pytest.mark.gpu


def _device_call(grad, idx, rows):
    """Callers of this entry point own the device buffers; torch stands in for such a caller."""
    import torch

    g = torch.from_numpy(grad).cuda()
    i = torch.from_numpy(idx.astype(np.int32)).cuda()  # same 32-bit pattern as uint32
    out = torch.full((rows, grad.shape[1]), float("nan"), device="cuda")  # every row must be written
    torch.cuda.synchronize()
    capi.op_scatter_add_rows_noalloc(g.data_ptr(), i.data_ptr(), idx.size, rows, grad.shape[1], out.data_ptr(), 0)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    rng = np.random.RandomState(7)
    # the second call is smaller and uses other rows: anything stale in the shared array would show
    for n, rows, width in ((4096, 3000, 64), (700, 41, 256)):
        grad = rng.normal(size=(n, width)).astype(np.float32)
        idx = rng.randint(rows, size=n).astype(np.uint32)
        want = capi.op_scatter_add_rows(grad, idx, rows)
        got = _device_call(grad, idx, rows)
        # same kernels, same summation order: identical bits (the fp32 tolerance of the suite, 1e-5, a fortiori)
        np.testing.assert_array_equal(got, want)
        np.testing.assert_allclose(got, want, rtol=1e-5)


def test_sizes_beyond_the_fixed_array_are_refused():
    import torch

    buf = torch.zeros(16, device="cuda")
    with pytest.raises(ValueError, match="exceed the fixed working memory"):
        capi.op_scatter_add_rows_noalloc(buf.data_ptr(), buf.data_ptr(), 4097, 8, 1, buf.data_ptr(), 0)
    with pytest.raises(ValueError, match="exceed the fixed working memory"):
        capi.op_scatter_add_rows_noalloc(buf.data_ptr(), buf.data_ptr(), 8, 65537, 1, buf.data_ptr(), 0)
