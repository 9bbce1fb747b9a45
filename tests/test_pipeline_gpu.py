"""The row-partition scheduler (db2_vectorizedPipeline) against unpartitioned execution, in the style of the
reference's MultiThreadedKernelTest (test/runtime/local/vectorized/MultiThreadedKernelTest.cpp:41-154: X+Y and X*Y on
1234 x 10 through the scheduler equal the single call), extended to every VectorCombine and to several batch sizes."""
import numpy as np
import pytest

from tests.util import assert_bits_equal, rng_matrix

pytestmark = pytest.mark.gpu

ROWS, COLS, ADD, MIN, MAX = 1, 2, 3, 4, 5


def _k():
    import daphne_b200.kernels as k
    return k


@pytest.mark.parametrize("batch", [0, 100, 333, 1234, 5000])
def test_elementwise_bodies_rows_combine(ctx, batch):
    k = _k()
    x, y = rng_matrix(1, 1234, 10), rng_matrix(2, 1234, 10)
    X, Y = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y)
    for op, exp in ((k.BinaryOpCode.ADD, x + y), (k.BinaryOpCode.MUL, x * y)):
        (r,) = k.vectorizedPipeline(ctx, [X, Y], [1, 1], [ROWS], lambda ins, op=op: [k.ewBinaryMat(op, *ins)], batch)
        assert_bits_equal(r.to_numpy(), exp, f"op {op} batch {batch}")


@pytest.mark.parametrize("batch", [0, 7000, 100000])
def test_all_combines_with_broadcast_and_large_inputs(ctx, batch):
    k = _k()
    B, A = k.BinaryOpCode, k.AggOpCode
    x = rng_matrix(3, 70001, 32)
    mu = x.mean(axis=0, keepdims=True)
    X, MU = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, mu)

    def body(ins):
        xs, m = ins
        d = k.ewBinaryMat(B.SUB, xs, m)
        return [k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, d, 2.0)),   # ROWS
                k.aggCol(A.SUM, d),                                  # ADD
                k.aggCol(A.MIN, xs),                                 # MIN
                k.aggCol(A.MAX, xs),                                 # MAX
                k.transpose(k.aggRow(A.MAX, xs))]                    # COLS

    r, s, mn, mx, t = k.vectorizedPipeline(ctx, [X, MU], [1, 0], [ROWS, ADD, MIN, MAX, COLS], body, batch)
    d = x - mu
    assert_bits_equal(r.to_numpy(), np.array([[sum_seq(row)] for row in (d * d)]), "rowSums ROWS")
    np.testing.assert_allclose(s.to_numpy(), d.sum(axis=0, keepdims=True), rtol=1e-9, atol=1e-9)
    assert_bits_equal(mn.to_numpy(), x.min(axis=0, keepdims=True), "MIN combine")
    assert_bits_equal(mx.to_numpy(), x.max(axis=0, keepdims=True), "MAX combine")
    assert_bits_equal(t.to_numpy(), x.max(axis=1, keepdims=True).T.copy(), "COLS combine")


def sum_seq(row):
    s = 0.0
    for v in row:
        s += v
    return s


def test_single_batch_results_stay_deferred_until_used(ctx):
    k = _k()
    B = k.BinaryOpCode
    x = rng_matrix(4, 80000, 16)
    X = k.DenseMatrix.from_numpy(ctx, x)
    X.device_ptr()
    l0 = ctx.stats()["launches"]
    (z,) = k.vectorizedPipeline(ctx, [X], [1], [ROWS], lambda ins: [k.ewBinaryObjSca(B.MUL, ins[0], 3.0)])
    assert ctx.stats()["launches"] == l0, "an elementwise body of a single batch launches nothing by itself"
    assert_bits_equal(z.to_numpy(), x * 3.0, "deferred result")
