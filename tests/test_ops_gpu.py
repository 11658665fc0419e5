"""Operator-level parity through the C ABI, modelled on the reference's operator tests.

The known-answer cases restate tests/pag/testPag.cpp (l1dist :290-319, l2dist :334-369,
l2dist-large :371-392, matMul :582-600, multiSlice :602-628, logSoftmax :775-794,
logSigmoid :817-845, allToAll :881-904) and tests/fructose/testFructose.cpp (Buffer
write/read :121-139).  The seeded cases compare with the numpy oracle; fp32 tolerance 1e-5.
"""

import numpy as np
import pytest

from distributed_kge_poplar_b200 import capi
from helpers import assert_close
from oracle import step_oracle as so

pytestmark = pytest.mark.gpu
RTOL = 1e-5


def _iota(rows, cols):
    return np.arange(rows * cols, dtype=np.float32).reshape(rows, cols)


def test_l1_distance_known_answers():
    a, b = _iota(2, 5), _iota(4, 5)
    out = capi.op_pairwise(capi.L1, a, b)
    np.testing.assert_array_equal(out, [[0, 25, 50, 75], [25, 0, 25, 50]])
    ga, gb = capi.op_pairwise_grad(capi.L1, a, b, np.ones((2, 4), np.float32))
    np.testing.assert_array_equal(ga, [[-3] * 5, [-1] * 5])
    np.testing.assert_array_equal(gb, [[-1] * 5, [1] * 5, [2] * 5, [2] * 5])


def test_l2_distance_known_answers():
    a, b = _iota(2, 5), _iota(4, 5)
    out = capi.op_pairwise(capi.L2, a, b)
    np.testing.assert_allclose(out, [[0, 11.1803, 22.3607, 33.5410], [11.1803, 0, 11.1803, 22.3607]], atol=1e-4)
    assert out[0, 0] == 0 and out[1, 1] == 0  # zero distance is exact and must not poison the gradient
    ga, gb = capi.op_pairwise_grad(capi.L2, a, b, np.ones((2, 4), np.float32))
    np.testing.assert_allclose(ga, [[-1.3416] * 5, [-0.4472] * 5], atol=1e-4)
    np.testing.assert_allclose(gb, [[-0.4472] * 5, [0.4472] * 5, [0.8944] * 5, [0.8944] * 5], atol=1e-4)
    assert np.all(np.isfinite(ga)) and np.all(np.isfinite(gb))


def test_l2_distance_large_values():
    a = np.array([[100, 200, 300, 400, 500]], np.float32)
    b = np.full((1, 5), 600, np.float32)
    np.testing.assert_allclose(capi.op_pairwise(capi.L2, a, b), [[741.62]], atol=0.5)
    ga, _ = capi.op_pairwise_grad(capi.L2, a, b, np.ones((1, 1), np.float32))
    np.testing.assert_allclose(ga, [[-0.6742, -0.5394, -0.4045, -0.2697, -0.1348]], atol=1e-3)


def test_dot_known_answers():
    a, bt = np.ones((2, 3), np.float32), np.ones((5, 3), np.float32)  # b^T of the reference's [3, 5]
    np.testing.assert_array_equal(capi.op_pairwise(capi.DOT, a, bt), np.full((2, 5), 3.0))
    ga, gbt = capi.op_pairwise_grad(capi.DOT, a, bt, np.ones((2, 5), np.float32))
    np.testing.assert_array_equal(ga, np.full((2, 3), 5.0))
    np.testing.assert_array_equal(gbt, np.full((5, 3), 2.0))


@pytest.mark.parametrize("fn,name", [(capi.L1, "l1"), (capi.L2, "l2"), (capi.DOT, "dot")])
@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 5, 7), (33, 65, 31), (64, 128, 64), (100, 257, 130), (512, 768, 256)])
def test_pairwise_matches_oracle(fn, name, shape):
    m, n, k = shape
    rng = np.random.RandomState(m * 1000 + n + k)
    a = rng.normal(size=(m, k)).astype(np.float32)
    b = rng.normal(size=(n, k)).astype(np.float32)
    b[0] = a[0]  # an exact zero distance
    if k > 2:
        b[-1, : k // 2] = a[-1, : k // 2]  # zero differences inside a row: sign(0) = 0
    g = rng.normal(size=(m, n)).astype(np.float32)
    a64, b64, g64 = a.astype(np.float64), b.astype(np.float64), g.astype(np.float64)
    if name == "l1":
        ref = so.l1_distance(a64, b64)
        ref_ga, ref_gb = so.l1_distance_grad(a64, b64, g64), so.l1_distance_grad(b64, a64, g64.T)
    elif name == "l2":
        ref = so.l2_distance(a64, b64)
        ref_ga = so.l2_distance_grad(a64, b64, ref, g64)
        ref_gb = so.l2_distance_grad(b64, a64, ref.T, g64.T)
    else:
        ref, ref_ga, ref_gb = a64 @ b64.T, g64 @ b64, g64.T @ a64
    out = capi.op_pairwise(fn, a, b)
    assert_close(out, ref, RTOL, f"{name} forward {shape}")
    if name == "l2":
        assert out[0, 0] == 0
        # the operator divides by its own fp32 distance; pairs that coincide must give exactly zero
        g[0, 0] = 1e6
    ga, gb = capi.op_pairwise_grad(fn, a, b, g)
    if name == "l2":
        g64[0, 0] = 1e6
        ref_ga = so.l2_distance_grad(a64, b64, ref, g64)
        ref_gb = so.l2_distance_grad(b64, a64, ref.T, g64.T)
    assert_close(ga, ref_ga, RTOL, f"{name} grad_a {shape}")
    assert_close(gb, ref_gb, RTOL, f"{name} grad_b {shape}")


def test_pairwise_empty_and_bad_arguments():
    a = np.zeros((0, 4), np.float32)
    b = np.ones((3, 4), np.float32)
    assert capi.op_pairwise(capi.L1, a, b).shape == (0, 3)
    with pytest.raises(ValueError):
        capi.op_pairwise(7, b, b)


def test_gather_rows_is_bit_exact():
    table = np.array([[10, 11], [20, 21], [30, 31]], np.float32)
    out = capi.op_gather_rows(table, [1, 1, 0, 1])
    np.testing.assert_array_equal(out, [[20, 21], [20, 21], [10, 11], [20, 21]])
    rng = np.random.RandomState(0)
    for width in (1, 3, 4, 256, 1152):
        big = rng.normal(size=(1000, width)).astype(np.float32)
        idx = rng.randint(1000, size=777).astype(np.uint32)
        np.testing.assert_array_equal(capi.op_gather_rows(big, idx), big[idx])
    with pytest.raises(ValueError):
        capi.op_gather_rows(table, [3])


def test_scatter_add_combines_duplicates():
    grad = np.array([[0.1, 1], [0.2, 2], [0.3, 3], [0.4, 4]], np.float32)
    out = capi.op_scatter_add_rows(grad, [1, 1, 0, 1], rows=3)
    np.testing.assert_allclose(out, [[0.3, 3], [0.7, 7], [0, 0]], rtol=1e-6)
    rng = np.random.RandomState(1)
    for n, rows, width in ((1, 1, 1), (100, 7, 5), (1280, 1280, 256), (4096, 50, 64)):
        g = rng.normal(size=(n, width)).astype(np.float32)
        idx = rng.randint(rows, size=n).astype(np.uint32)
        out = capi.op_scatter_add_rows(g, idx, rows)
        ref = so.scatter_add_rows(rows, idx.astype(np.int64), g.astype(np.float64))
        assert_close(out, ref, RTOL, f"scatter_add {n}x{width} -> {rows}")
        # fixed summation order: a second run is bit-identical
        np.testing.assert_array_equal(out, capi.op_scatter_add_rows(g, idx, rows))


def test_log_softmax_known_answers():
    x = np.array([[1, 1, 2]], np.float32)
    y, gx = capi.op_activation(1, x, np.array([[10, 15, 5]], np.float32))
    norm = np.log(np.exp(1.0) + np.exp(1.0) + np.exp(2.0))
    np.testing.assert_allclose(y, [[1 - norm, 1 - norm, 2 - norm]], rtol=1e-6)
    np.testing.assert_allclose(gx, [[10 - 30 * np.exp(1 - norm), 15 - 30 * np.exp(1 - norm), 5 - 30 * np.exp(2 - norm)]], rtol=1e-5)


def test_log_sigmoid_known_answers():
    x = np.array([-100, -12, -1, 0, 1, 12, 100], np.float32)
    y, gx = capi.op_activation(0, x, np.full(7, 10.0, np.float32))
    np.testing.assert_allclose(y, -np.log1p(np.exp(-x.astype(np.float64))), atol=1e-2)
    np.testing.assert_allclose(gx, 10.0 / (1 + np.exp(x.astype(np.float64))), atol=1e-2)
    # and the guarded form itself, tightly
    x64 = x.astype(np.float64)
    assert_close(y, so.log_sigmoid(x64), RTOL, "log_sigmoid")
    assert_close(gx, so.log_sigmoid_grad(x64, np.full(7, 10.0)), RTOL, "log_sigmoid grad")


def test_activations_match_oracle_on_wide_rows():
    rng = np.random.RandomState(2)
    x = (4 * rng.normal(size=(37, 768))).astype(np.float32)
    g = rng.normal(size=x.shape).astype(np.float32)
    y, gx = capi.op_activation(1, x, g)
    logp = so.log_softmax(x.astype(np.float64))
    assert_close(y, logp, RTOL, "log_softmax")
    assert_close(gx, so.log_softmax_grad(logp, g.astype(np.float64)), RTOL, "log_softmax grad")


def test_all_to_all_routing_is_exact():
    # payload encodes (shard, block, element) so that any misrouting is visible
    # (tests/pag/testPag.cpp:856-878): shard s holds value 1000*(1+s) + 10*(1+i) + (1+j)
    n, block = 2, 3
    data = np.zeros((n, n, block), np.float32)
    for s in range(n):
        for i in range(n):
            for j in range(block):
                data[s, i, j] = 1000 * (1 + s) + 10 * (1 + i) + (1 + j)
    out = capi.op_all_to_all(data)
    np.testing.assert_array_equal(out.reshape(-1), [1011, 1012, 1013, 2011, 2012, 2013, 1021, 1022, 1023, 2021, 2022, 2023])
    # the backward is the same exchange: applying it twice restores the input
    np.testing.assert_array_equal(capi.op_all_to_all(out), data)
    for n, block in ((1, 5), (4, 80 * 64), (8, 96 * 256), (3, 7)):
        big = np.arange(n * n * block, dtype=np.float32).reshape(n, n, block)
        np.testing.assert_array_equal(capi.op_all_to_all(big), so.all_to_all(big))
