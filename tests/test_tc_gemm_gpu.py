"""The tensor-core contraction (tcgen05, 3xTF32 split) against float64 numpy, through the C ABI.

Bound: 1e-5 relative with the tensor's rms in the denominator, the suite's fp32 tolerance: the
split leaves about 1e-6 of sum |a||b|."""

import numpy as np
import pytest

from distributed_kge_poplar_b200 import capi
from helpers import assert_close

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def _ref(a, b, a_t, b_t, m, n, k, gather=None):
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    if gather is not None:
        a64 = a64[gather]
    A = a64.T[:m, :k] if a_t else a64[:m, :k]
    B = b64.T[:n, :k] if b_t else b64[:n, :k]
    return A @ B.T, A


@pytest.mark.parametrize("tile_n", [64, 128])
@pytest.mark.parametrize("shape", [(128, 128, 32), (128, 64, 8), (512, 768, 256), (100, 70, 45), (1, 1, 1), (300, 257, 130)])
def test_plain_product(shape, tile_n):
    m, n, k = shape
    rng = np.random.RandomState(m + n + k)
    a = rng.normal(size=(m, k)).astype(np.float32)
    b = rng.normal(size=(n, k)).astype(np.float32)
    out = capi.op_tc_gemm(a, b, m, n, k, tile_n=tile_n)[0]
    assert_close(out, _ref(a, b, False, False, m, n, k)[0], RTOL, f"A.B^T {shape} tile {tile_n}")


def test_split_is_needed_and_sufficient():
    """Values with full 24-bit significands: a single TF32 product would be off by about 1e-3."""
    rng = np.random.RandomState(0)
    a = (1.0 + rng.uniform(size=(128, 256))).astype(np.float32)
    b = (1.0 + rng.uniform(size=(128, 256))).astype(np.float32)
    out = capi.op_tc_gemm(a, b, 128, 128, 256)[0]
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    assert np.max(np.abs(out / ref - 1)) < 2e-6


@pytest.mark.parametrize("a_t,b_t", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(512, 256, 768), (768, 256, 512), (130, 70, 100)])
def test_transposed_operands(shape, a_t, b_t):
    m, n, k = shape
    rng = np.random.RandomState(7)
    a = rng.normal(size=(k, m) if a_t else (m, k)).astype(np.float32)
    b = rng.normal(size=(k, n) if b_t else (n, k)).astype(np.float32)
    out = capi.op_tc_gemm(a, b, m, n, k, a_transposed=a_t, b_transposed=b_t, tile_n=64)[0]
    assert_close(out, _ref(a, b, a_t, b_t, m, n, k)[0], RTOL, f"{shape} a_t={a_t} b_t={b_t}")


def test_gathered_half_rows_and_value_epilogue():
    """The hidden-row product: fp16 feature rows picked by index, times W stored [k, n], plus x."""
    rng = np.random.RandomState(3)
    rows, f, d, r = 1000, 96, 64, 300
    table = rng.normal(size=(rows, f)).astype(np.float16)
    w = (rng.normal(size=(f, d)) / 10).astype(np.float32)
    x = rng.normal(size=(r, d)).astype(np.float32)
    idx = rng.randint(rows, size=r).astype(np.uint32)
    out = capi.op_tc_gemm(table, w, r, d, f, b_transposed=True, a_gather=idx, epilogue=1, x=x, tile_n=64)[0]
    ref = table[idx].astype(np.float64) @ w.astype(np.float64) + x
    assert_close(out, ref, RTOL, "gathered fp16 A, value epilogue")


def test_transposed_gathered_half_with_splits():
    """The projection gradient: feature^T (gathered rows are the k index) times d_hidden, k split."""
    rng = np.random.RandomState(4)
    rows, f, d, r = 500, 80, 48, 333
    table = rng.normal(size=(rows, f)).astype(np.float16)
    dh = rng.normal(size=(r, d)).astype(np.float32)
    idx = rng.randint(rows, size=r).astype(np.uint32)
    out = capi.op_tc_gemm(table, dh, f, d, r, a_transposed=True, b_transposed=True, a_gather=idx, splits=3, tile_n=64)
    ref = table[idx].astype(np.float64).T @ dh.astype(np.float64)
    assert_close(out.astype(np.float64).sum(0), ref, RTOL, "split-k projection gradient")
    # the splits partition k in order: each partial is the product over its own k range
    per = ((r + 2) // 3 + 31) // 32 * 32
    part0 = table[idx[:per]].astype(np.float64).T @ dh[:per].astype(np.float64)
    assert_close(out[0], part0, RTOL, "first split")


@pytest.mark.parametrize("a_t", [False, True])
def test_rowsum_epilogue(a_t):
    """The L2 backward form: rowsum(C)[m] * x[m, n] - (C . Y)[m, n]."""
    rng = np.random.RandomState(5)
    m, n, k = 200, 96, 150
    c = rng.normal(size=(k, m) if a_t else (m, k)).astype(np.float32)
    y = rng.normal(size=(k, n)).astype(np.float32)
    x = rng.normal(size=(m, n)).astype(np.float32)
    out = capi.op_tc_gemm(c, y, m, n, k, a_transposed=a_t, b_transposed=True, epilogue=2, x=x, tile_n=64)[0]
    C = c.astype(np.float64).T if a_t else c.astype(np.float64)
    ref = C.sum(1, keepdims=True) * x - C @ y.astype(np.float64)
    assert_close(out, ref, RTOL, f"rowsum epilogue a_t={a_t}")
