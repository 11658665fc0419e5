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


def test_against_numpy_and_indices_past_the_table_are_ignored():
    """The operator's own definition, np.add.at into a zeroed table (the duplicate-combining
    scatter-add of src/pag/pag.cpp:706-746), including what the header promises for indices that
    are not below `rows`: their gradient rows are dropped.  Lookups of one row are added in
    position order, which is the order np.add.at uses, so the sums agree to the last bit."""
    rng = np.random.RandomState(9)
    n, rows, width = 3000, 500, 48
    grad = rng.normal(size=(n, width)).astype(np.float32)
    idx = rng.randint(rows + 60, size=n).astype(np.uint32)   # about a tenth of them past the table
    idx[:5] = [0, rows - 1, rows, rows + 59, 2**31 + 5]
    assert np.any(idx >= rows)
    want = np.zeros((rows, width), np.float32)
    keep = idx < rows
    np.add.at(want, idx[keep], grad[keep])
    got = _device_call(grad, idx, rows)
    np.testing.assert_array_equal(got, want)
    empty = _device_call(grad[:0], idx[:0], rows)   # no lookups at all: a zeroed table
    np.testing.assert_array_equal(empty, np.zeros_like(want))


def test_sizes_beyond_the_fixed_array_are_refused():
    import torch

    buf = torch.zeros(16, device="cuda")
    with pytest.raises(ValueError, match="exceed the fixed working memory"):
        capi.op_scatter_add_rows_noalloc(buf.data_ptr(), buf.data_ptr(), 4097, 8, 1, buf.data_ptr(), 0)
    with pytest.raises(ValueError, match="exceed the fixed working memory"):
        capi.op_scatter_add_rows_noalloc(buf.data_ptr(), buf.data_ptr(), 8, 65537, 1, buf.data_ptr(), 0)
