"""Parity of the aggregation CUDA kernels with the CPU oracle (AggRow / AggCol / AggAll)."""
import numpy as np
import pytest

from tests.util import RTOL_REDUCE_F32, RTOL_REDUCE_F64, assert_bits_equal, assert_close_rel, rng_matrix

pytestmark = pytest.mark.gpu

SHAPES = [(1, 1), (3, 5), (64, 32), (257, 33), (1000, 64), (4099, 50), (5, 20011), (100003, 1), (1, 100003),
          (700, 1024), (20000, 3), (33, 130)]
VALUE_OPS = ["SUM", "MIN", "MAX", "MEAN", "VAR", "STDDEV"]
IDX_OPS = ["IDXMIN", "IDXMAX"]


def _k():
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    return k, o


def _expected(f_cpu, op, a, name):
    """f32 sums: the sequential float loop of the reference is the noisy side (relative error grows with the
    number of addends), so float inputs are checked against the same loop run in double and rounded once."""
    if a.dtype == np.float32 and name not in ("MIN", "MAX"):
        return np.asarray(f_cpu(op, a.astype(np.float64))).astype(np.float32)
    return f_cpu(op, a)


def _rtol(dtype):
    return RTOL_REDUCE_F64 if np.dtype(dtype) == np.float64 else RTOL_REDUCE_F32


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("which", ["row", "col"])
def test_value_aggregates(ctx, dtype, which):
    k, o = _k()
    f_gpu = k.aggRow if which == "row" else k.aggCol
    f_cpu = o.aggRow if which == "row" else o.aggCol
    for i, (r, c) in enumerate(SHAPES):
        a = rng_matrix(100 + i, r, c, dtype)
        A = k.DenseMatrix.from_numpy(ctx, a)
        for name in VALUE_OPS:
            op = k.AggOpCode[name]
            got, exp = f_gpu(op, A).to_numpy(), _expected(f_cpu, op, a, name)
            if name in ("MIN", "MAX"):
                assert_bits_equal(got, exp, f"{which} {name} {r}x{c}")
            else:
                # variance of a single value is exactly 0 on both sides; otherwise relative to the result
                assert_close_rel(got, exp, _rtol(dtype) * (10 if name in ("VAR", "STDDEV") else 1),
                                 f"{which} {name} {dtype.__name__} {r}x{c}", scale=1e-300)


@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.int64])
@pytest.mark.parametrize("which", ["row", "col"])
def test_index_aggregates_bit_exact_with_ties(ctx, dtype, which):
    k, o = _k()
    f_gpu = k.aggRow if which == "row" else k.aggCol
    f_cpu = o.aggRow if which == "row" else o.aggCol
    for i, (r, c) in enumerate(SHAPES):
        rng = np.random.default_rng(200 + i)
        # few distinct values => many ties; the lowest index has to win (AggRow.h:71-96, AggCol.h:70-121)
        a = rng.integers(0, 4, size=(r, c)).astype(dtype)
        A = k.DenseMatrix.from_numpy(ctx, a)
        for name in IDX_OPS:
            op = k.AggOpCode[name]
            got, exp = f_gpu(op, A).to_numpy(), f_cpu(op, a)
            assert got.dtype == np.uint64
            assert_bits_equal(got, exp, f"{which} {name} {dtype.__name__} {r}x{c}")


@pytest.mark.parametrize("which", ["row", "col"])
def test_int64_sum_min_max_bit_exact(ctx, which):
    k, o = _k()
    f_gpu = k.aggRow if which == "row" else k.aggCol
    f_cpu = o.aggRow if which == "row" else o.aggCol
    for i, (r, c) in enumerate(SHAPES):
        a = rng_matrix(300 + i, r, c, np.int64)
        A = k.DenseMatrix.from_numpy(ctx, a)
        for name in ["SUM", "MIN", "MAX"]:
            op = k.AggOpCode[name]
            assert_bits_equal(f_gpu(op, A).to_numpy(), f_cpu(op, a), f"{which} {name} i64 {r}x{c}")


@pytest.mark.parametrize("which", ["row", "col"])
def test_nan_inf_and_signed_zero_follow_the_sequential_scan(ctx, which):
    """std::min/std::max and the strict comparisons of the reference only ever return a NaN when it is the first
    element scanned, and return the first of several equal extrema (so -0.0 vs +0.0 depends on order)."""
    k, o = _k()
    rows = [
        [np.nan, 1.0, 2.0, -3.0],
        [1.0, np.nan, 2.0, -3.0],
        [np.nan, np.nan, np.nan, np.nan],
        [np.inf, np.nan, np.inf, np.inf],
        [-np.inf, -np.inf, np.nan, -np.inf],
        [0.0, -0.0, 0.0, -0.0],
        [-0.0, 0.0, -0.0, 0.0],
        [5.0, 5.0, 5.0, 5.0],
        [1.0, 7.0, 7.0, -2.0],
        [-2.0, 1.0, -2.0, 7.0],
    ]
    a = np.array(rows)
    if which == "col":
        a = np.ascontiguousarray(a.T)
    f_gpu = k.aggRow if which == "row" else k.aggCol
    f_cpu = o.aggRow if which == "row" else o.aggCol
    A = k.DenseMatrix.from_numpy(ctx, a)
    for name in ["MIN", "MAX", "IDXMIN", "IDXMAX"]:
        op = k.AggOpCode[name]
        got, exp = f_gpu(op, A).to_numpy(), f_cpu(op, a)
        if got.dtype == np.float64:
            nan = np.isnan(exp)
            assert np.array_equal(np.isnan(got), nan), name
            got, exp = np.where(nan, 0.0, got), np.where(nan, 0.0, exp)
        assert_bits_equal(got, exp, f"{which} {name} specials")


@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.int64])
def test_agg_all(ctx, dtype):
    k, o = _k()
    for i, (r, c) in enumerate(SHAPES + [(3000, 1000)]):
        a = rng_matrix(400 + i, r, c, dtype)
        A = k.DenseMatrix.from_numpy(ctx, a)
        ops = ["SUM", "MIN", "MAX"] + ([] if np.dtype(dtype) == np.int64 else ["MEAN", "VAR", "STDDEV"])
        for name in ops:
            op = k.AggOpCode[name]
            got, exp = k.aggAll(op, A), _expected(o.aggAll, op, a, name)
            if name in ("MIN", "MAX") or np.dtype(dtype) == np.int64:
                assert got == exp, f"all {name} {dtype.__name__} {r}x{c}: {got} vs {exp}"
            else:
                assert_close_rel(np.array([got]), np.array([exp]),
                                 _rtol(dtype) * (10 if name in ("VAR", "STDDEV") else 1),
                                 f"all {name} {dtype.__name__} {r}x{c}", scale=1e-300)


def test_agg_on_row_views(ctx):
    k, o = _k()
    a = rng_matrix(500, 5000, 32)
    A = k.DenseMatrix.from_numpy(ctx, a)
    v = A.slice_rows(1234, 4321)
    s = a[1234:4321]
    assert_close_rel(k.aggRow(k.AggOpCode.SUM, v).to_numpy(), o.aggRow(0, s), RTOL_REDUCE_F64, "row view")
    assert_close_rel(k.aggCol(k.AggOpCode.SUM, v).to_numpy(), o.aggCol(0, s), RTOL_REDUCE_F64, "col view")
    assert_close_rel(np.array([k.aggAll(k.AggOpCode.SUM, v)]), np.array([o.aggAll(0, s)]), RTOL_REDUCE_F64, "all view")
    assert_bits_equal(k.aggRow(k.AggOpCode.IDXMAX, v).to_numpy(), o.aggRow(5, s), "idxmax view")


def test_reduction_error_is_measured_against_an_exact_sum(ctx):
    """The sequential CPU sum is itself the noisier side for long columns: both results are compared with an exactly
    rounded sum (math.fsum), and the CUDA result has to be at least as close as the tolerance."""
    import math
    k, o = _k()
    a = rng_matrix(600, 200000, 4)
    A = k.DenseMatrix.from_numpy(ctx, a)
    got = k.aggCol(k.AggOpCode.SUM, A).to_numpy()[0]
    seq = o.aggCol(0, a)[0]
    for c in range(4):
        exact = math.fsum(a[:, c].tolist())
        assert abs(got[c] - exact) <= RTOL_REDUCE_F64 * abs(exact)
        assert abs(seq[c] - exact) <= RTOL_REDUCE_F64 * abs(exact)


def test_agg_cum_against_the_sequential_loop(ctx):
    """AggCum.h:48-86: MIN / MAX and int64 are exact; f64 / f32 sums and products are blocked on the device, so they
    are held to the error bound of a sum of that length in any order.  NaN handling of MIN / MAX: a NaN in
    row 0 stays for the whole column, later NaNs are skipped; -0.0 in row 0 is copied."""
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    rng = np.random.default_rng(51)
    A = k.AggOpCode
    shapes = [(1, 1), (5, 3), (1, 40), (300, 1), (4097, 33), (20000, 7), (70001, 2), (2000, 130)]
    for dtype in (np.float64, np.int64, np.float32):
        for rows, cols in shapes:
            if dtype == np.int64:
                x = rng.integers(-3, 4, size=(rows, cols)).astype(dtype)
            else:
                x = rng.standard_normal((rows, cols)).astype(dtype)
            X = k.DenseMatrix.from_numpy(ctx, x)
            for op in (A.SUM, A.MIN, A.MAX, A.PROD):
                if op == A.PROD:
                    xp = np.where(rng.random((rows, cols)) < 0.5, 1, -1).astype(dtype) if dtype == np.int64 else \
                        (1.0 + 0.001 * x).astype(dtype)
                    got = k.aggCum(op, k.DenseMatrix.from_numpy(ctx, xp)).to_numpy()
                    exp = o.aggCum(int(op), xp)
                else:
                    got, exp = k.aggCum(op, X).to_numpy(), o.aggCum(int(op), x)
                assert got.shape == exp.shape and got.dtype == exp.dtype
                if dtype == np.int64 or op in (A.MIN, A.MAX):
                    assert np.array_equal(got, exp), (dtype, rows, cols, op)
                else:
                    # classical bound of a length-n sum / product in any order: n * eps * magnitude, against the
                    # double-precision result of the same inputs
                    src = (xp if op == A.PROD else x).astype(np.float64)
                    exact = np.cumprod(src, axis=0) if op == A.PROD else np.cumsum(src, axis=0)
                    tol = rows * np.finfo(dtype).eps * max(1.0, np.abs(src).cumsum(axis=0).max() if op == A.SUM
                                                           else np.abs(exact).max())
                    assert np.abs(got.astype(np.float64) - exact).max() <= tol, (dtype, rows, cols, op)
                    assert np.abs(exp.astype(np.float64) - exact).max() <= tol, "the sequential loop meets it too"
    x = rng.standard_normal((5000, 4))
    x[0, 1] = np.nan          # whole column NaN for MIN / MAX
    x[700, 2] = np.nan        # skipped
    x[0, 3] = -0.0
    x[1:, 3] = np.abs(x[1:, 3])
    X = k.DenseMatrix.from_numpy(ctx, x)
    for op in (A.MIN, A.MAX):
        got, exp = k.aggCum(op, X).to_numpy(), o.aggCum(int(op), x)
        assert np.array_equal(np.isnan(got), np.isnan(exp)) and np.array_equal(np.nan_to_num(got), np.nan_to_num(exp))
    got = k.aggCum(A.SUM, X).to_numpy()
    assert np.signbit(got[0, 3]) and np.isnan(got[700:, 2]).all() and not np.isnan(got[:700, 2]).any()
    v = X.slice_rows(1000, 4000)
    assert np.array_equal(k.aggCum(A.MAX, v).to_numpy()[:, 0], np.maximum.accumulate(x[1000:4000, 0]))
    with pytest.raises(k.Db2Error, match="pure binary reduction"):
        k.aggCum(A.MEAN, X)
