"""The plane-fed tensor-core contraction (TMA boxes under the 128-byte swizzle straight into the
UMMA layout, 3xTF32) against float64 numpy, through the C ABI.

Bound: 1e-5 relative with the tensor's rms in the denominator, the suite's fp32 tolerance."""

import numpy as np
import pytest

from distributed_kge_poplar_b200 import capi
from helpers import assert_close

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def _operands(rng, m, n, k, a_mn, b_mn, pad=0):
    """Stored matrices (row length padded to a multiple of 4 floats) and the float64 product."""
    def stored(rows, cols):
        cols_p = (cols + pad + 3) // 4 * 4
        return rng.normal(size=(rows, cols_p)).astype(np.float32)
    a = stored(k, m) if a_mn else stored(m, k)
    b = stored(k, n) if b_mn else stored(n, k)
    A = (a.T if a_mn else a)[:m, :k].astype(np.float64)
    B = (b.T if b_mn else b)[:n, :k].astype(np.float64)
    return a, b, A, B


@pytest.mark.parametrize("tile_n", [64, 128])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(128, 64, 32), (128, 128, 64), (512, 768, 256), (100, 70, 45), (1, 1, 1), (300, 257, 130)])
def test_all_operand_layouts(shape, a_mn, b_mn, tile_n):
    m, n, k = shape
    rng = np.random.RandomState(m + 3 * n + 7 * k)
    a, b, A, B = _operands(rng, m, n, k, a_mn, b_mn)
    out, _ = capi.op_tc_planes(a, b, m, n, k, a_mn_major=a_mn, b_mn_major=b_mn, tile_n=tile_n)
    assert_close(out, A @ B.T, RTOL, f"{shape} a_mn={a_mn} b_mn={b_mn} tile {tile_n}")


@pytest.mark.parametrize("tile_n", [64, 128])
@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True)])
def test_cluster_split_k(splits, a_mn, b_mn, tile_n):
    """The step's shapes: hidden (1280 x 256 x 768) and the projection gradient (768 x 256 x 1280)."""
    m, n, k = (1280, 256, 768) if not a_mn else (768, 256, 1280)
    rng = np.random.RandomState(splits)
    a, b, A, B = _operands(rng, m, n, k, a_mn, b_mn)
    out, _ = capi.op_tc_planes(a, b, m, n, k, a_mn_major=a_mn, b_mn_major=b_mn, splits=splits, tile_n=tile_n)
    assert_close(out, A @ B.T, RTOL, f"splits={splits} a_mn={a_mn} tile {tile_n}")


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_the_tensor_core_ignores_the_low_bits_of_the_upper_plane(a_mn, b_mn):
    """The stored fp32 array serves as the upper plane: a copy with the low 13 significand bits
    cleared gives the same result bit for bit, in every operand layout."""
    rng = np.random.RandomState(17)
    a, b, _, _ = _operands(rng, 256, 256, 256, a_mn, b_mn)
    raw, _ = capi.op_tc_planes(a, b, 256, 256, 256, a_mn_major=a_mn, b_mn_major=b_mn, splits=2)
    cleared, _ = capi.op_tc_planes(a, b, 256, 256, 256, a_mn_major=a_mn, b_mn_major=b_mn, splits=2, hi_is_cleared=True)
    np.testing.assert_array_equal(raw.view(np.uint32), cleared.view(np.uint32))


def test_split_is_needed_and_sufficient():
    """Values with full 24-bit significands: a single TF32 product would be off by about 1e-3."""
    rng = np.random.RandomState(0)
    a = (1.0 + rng.uniform(size=(128, 256))).astype(np.float32)
    b = (1.0 + rng.uniform(size=(128, 256))).astype(np.float32)
    out, _ = capi.op_tc_planes(a, b, 128, 128, 256)
    ref = a.astype(np.float64) @ b.astype(np.float64).T
    assert np.max(np.abs(out / ref - 1)) < 2e-6


def test_exact_operand_has_one_plane():
    """fp16 feature rows widened to fp32 are exact in TF32: the lo plane of A is skipped."""
    rng = np.random.RandomState(5)
    m, n, k = 300, 64, 96
    a = rng.normal(size=(m, k)).astype(np.float16).astype(np.float32)
    w = (rng.normal(size=(k, n)) / 10).astype(np.float32)
    x = rng.normal(size=(m, n)).astype(np.float32)
    out, _ = capi.op_tc_planes(a, w, m, n, k, b_mn_major=True, a_exact=True, epilogue=1, x=x, splits=3)
    assert_close(out, a.astype(np.float64) @ w.astype(np.float64) + x, RTOL, "exact A, value epilogue")


@pytest.mark.parametrize("tile_n", [64, 128])
@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("splits", [1, 4])
def test_rowsum_epilogue(a_mn, splits, tile_n):
    """The L2 backward in contraction form: out = rowsum(A) * x - A . B^T, for both gradients
    (A = the coefficient matrix k-major, and its transpose mn-major)."""
    rng = np.random.RandomState(11 + splits)
    m, n, k = (512, 256, 768) if not a_mn else (768, 256, 512)
    a, b, A, B = _operands(rng, m, n, k, a_mn, True)
    x = rng.normal(size=(m, n)).astype(np.float32)
    out, _ = capi.op_tc_planes(a, b, m, n, k, a_mn_major=a_mn, b_mn_major=True, epilogue=2, x=x, splits=splits, tile_n=tile_n)
    ref = A.sum(1, keepdims=True) * x.astype(np.float64) - A @ B.T
    assert_close(out, ref, RTOL, f"rowsum epilogue a_mn={a_mn} splits={splits}")


def test_argument_errors():
    a = np.zeros((8, 6), np.float32)
    with pytest.raises(ValueError):
        capi.op_tc_planes(a, a, 8, 8, 6)  # stored rows of 24 bytes
    b = np.zeros((8, 8), np.float32)
    with pytest.raises(ValueError):
        capi.op_tc_planes(b, b, 8, 8, 8, splits=9)


@pytest.mark.parametrize("tile_n", [64, 128])
@pytest.mark.parametrize("splits", [1, 2, 4])
def test_l2_distance_in_contraction_form(splits, tile_n):
    """sqrt(|a|^2 + |b|^2 - 2 a.b) with the direct form where the expansion cancels: rows of b that
    equal a row of a give an exact zero, near rows keep 1e-5 relative, and the rest agree with the
    float64 distance to 1e-5 of the matrix's scale."""
    rng = np.random.RandomState(3 + splits)
    m, n, k = 200, 300, 256
    a = rng.normal(size=(m, k)).astype(np.float32)
    b = rng.normal(size=(n, k)).astype(np.float32)
    b[5] = a[17]                                   # identical rows: distance exactly 0
    b[6] = a[18] + np.float32(1e-3) * rng.normal(size=k).astype(np.float32)   # near rows: the expansion alone would lose these
    b[7] = 10 * a[19]
    out, _ = capi.op_tc_planes(a, b, m, n, k, epilogue=3, splits=splits, tile_n=tile_n)
    ref = np.sqrt(((a.astype(np.float64)[:, None, :] - b.astype(np.float64)[None, :, :]) ** 2).sum(-1))
    assert out[17, 5] == 0.0
    np.testing.assert_allclose(out[18, 6], ref[18, 6], rtol=1e-5)
    assert_close(out, ref, RTOL, f"L2 distance splits={splits} tile {tile_n}")
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-30)


def _bf16_round(x):
    """Round-to-nearest-even to bfloat16, returned as float32."""
    bits = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return bits.astype(np.uint32).view(np.float32)


@pytest.mark.parametrize("tile_n", [64, 128])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape,splits", [((128, 128, 64), 1), ((1024, 2048, 512), 1), ((1024, 512, 2048), 4), ((300, 264, 200), 2), ((5, 3, 9), 1)])
def test_bf16_operands(shape, splits, a_mn, b_mn, tile_n):
    """bfloat16 operands, fp32 accumulation (the 2e-2 tier's contraction): products of bf16 values
    are exact in fp32, so against the float64 product of the rounded inputs only the order of the
    fp32 additions shows."""
    m, n, k = shape
    rng = np.random.RandomState(m + n + k)
    def stored(rows, cols):
        return rng.normal(size=(rows, (cols + 7) // 8 * 8)).astype(np.float32)
    a = stored(k, m) if a_mn else stored(m, k)
    b = stored(k, n) if b_mn else stored(n, k)
    A = _bf16_round(a.T if a_mn else a)[:m, :k].astype(np.float64)
    B = _bf16_round(b.T if b_mn else b)[:n, :k].astype(np.float64)
    out, _ = capi.op_tc_planes_bf16(a, b, m, n, k, a_mn_major=a_mn, b_mn_major=b_mn, splits=splits, tile_n=tile_n)
    assert_close(out, A @ B.T, RTOL, f"bf16 {shape} a_mn={a_mn} b_mn={b_mn} tile {tile_n}")
