"""The C restatement (oracle/oracle.c) against the reference's own CPU kernels compiled from its sources
(oracle/_ref).  Bit-exact: both run the same scalar expressions in the same order.  Skipped where oracle/_ref was not
built (no DAPHNE source tree on this machine)."""
import numpy as np
import pytest

from oracle import pyoracle as o
from oracle import refkernels as ref
from tests.util import assert_bits_equal, rng_matrix

pytestmark = pytest.mark.skipif(not ref.available(), reason="oracle/_ref not built")

SHAPES = [(1, 1), (3, 5), (64, 32), (257, 33), (1, 1003), (1003, 1), (130, 70)]
DTYPES = [np.float64, np.float32, np.int64]


def _nanfix(a, b):
    if a.dtype.kind == "f":
        nan = np.isnan(b)
        assert np.array_equal(np.isnan(a), nan)
        return np.where(nan, 0, a), np.where(nan, 0, b)
    return a, b


@pytest.mark.parametrize("dtype", DTYPES)
def test_ew_binary(dtype):
    for i, (r, c) in enumerate(SHAPES):
        a, b = rng_matrix(i, r, c, dtype), rng_matrix(50 + i, r, c, dtype)
        rv, cv = rng_matrix(70 + i, 1, c, dtype), rng_matrix(90 + i, r, 1, dtype)
        for m in (b, rv, cv):
            m[m == 0] = 3
        a.reshape(-1)[::5] = b.reshape(-1)[::5]
        for op in range(17):
            if np.dtype(dtype) == np.int64 and op in (4, 5, 6):
                x, y, z, w = np.abs(a) % 7 + 1, np.abs(b) % 4 + 1, np.abs(rv) % 4 + 1, np.abs(cv) % 4 + 1
            elif op in (4, 6):
                x, y, z, w = np.abs(a) + 1, np.abs(b) % 3 + 1.5, np.abs(rv) % 3 + 1.5, np.abs(cv) % 3 + 1.5
                x, y, z, w = (t.astype(dtype) for t in (x, y, z, w))
            else:
                x, y, z, w = a, b, rv, cv
            for rhs in (y, z, w):
                assert_bits_equal(*_nanfix(o.ewBinaryMat(op, x, rhs), ref.ewBinaryMat(op, x, rhs)),
                                  f"op {op} {dtype.__name__} {x.shape} {rhs.shape}")
            s = 3 if np.dtype(dtype) == np.int64 else 2.5
            assert_bits_equal(*_nanfix(o.ewBinaryObjSca(op, x, s), ref.ewBinaryObjSca(op, x, s)), f"sca op {op}")


def _int_operands(dtype, seed, r, c):
    """Operands of the 32-bit / unsigned integer value types inside the range where C++ integer arithmetic is defined
    (no signed overflow, no out-of-range double -> integer conversion, non-zero divisors)."""
    rng = np.random.default_rng(seed)
    lo = 0 if np.dtype(dtype).kind == "u" else -30
    a = rng.integers(lo, 60, size=(r, c)).astype(dtype)
    b = rng.integers(2, 9, size=(r, c)).astype(dtype)
    rv = rng.integers(2, 9, size=(1, c)).astype(dtype)
    cv = rng.integers(2, 9, size=(r, 1)).astype(dtype)
    a.reshape(-1)[::5] = b.reshape(-1)[::5]
    return a, b, rv, cv


@pytest.mark.parametrize("dtype", [np.uint64, np.int32, np.uint32])
def test_ew_binary_other_integer_types(dtype):
    for i, (r, c) in enumerate(SHAPES):
        a, b, rv, cv = _int_operands(dtype, i, r, c)
        for op in range(17):
            x = a
            if op in (4, 5, 6) or (op == 1 and np.dtype(dtype).kind == "u"):
                x = (np.abs(a.astype(np.int64)) % 7 + 9).astype(dtype)  # pow / log / mod / unsigned sub stay in range
            if op == 4:
                x = (x % 5 + 1).astype(dtype)
            for rhs in (b, rv, cv):
                assert_bits_equal(o.ewBinaryMat(op, x, rhs), ref.ewBinaryMat(op, x, rhs),
                                  f"op {op} {np.dtype(dtype).name} {x.shape} {rhs.shape}")
            assert_bits_equal(o.ewBinaryObjSca(op, x, 3), ref.ewBinaryObjSca(op, x, 3), f"sca op {op}")


def test_ew_binary_shape_error_matches():
    with pytest.raises(o.OracleError):
        o.ewBinaryMat(0, np.ones((4, 5)), np.ones((3, 2)))
    with pytest.raises(o.OracleError):
        ref.ewBinaryMat(0, np.ones((4, 5)), np.ones((3, 2)))


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_ew_unary(dtype):
    for i, (r, c) in enumerate(SHAPES):
        a = (rng_matrix(i, r, c, dtype, kind="uniform") * 0.9 + 0.05).astype(dtype)
        for op in range(19):
            assert_bits_equal(*_nanfix(o.ewUnaryMat(op, a), ref.ewUnaryMat(op, a)), f"unary {op} {dtype.__name__}")
        neg = (a - 0.5).astype(dtype)
        for op in (0, 1, 2, 4, 6, 7, 8, 11, 12, 13, 14, 15, 16, 17, 18):
            assert_bits_equal(*_nanfix(o.ewUnaryMat(op, neg), ref.ewUnaryMat(op, neg)), f"unary {op} neg")
    bad = np.array([[1.0, -1.0]])
    for op in (3, 5):
        with pytest.raises(o.OracleError) as e1:
            o.ewUnaryMat(op, bad)
        with pytest.raises(o.OracleError) as e2:
            ref.ewUnaryMat(op, bad)
        assert e1.value.code == e2.value.code == 5


@pytest.mark.parametrize("dtype", DTYPES)
def test_aggregations(dtype):
    ops = range(9) if np.dtype(dtype) != np.int64 else (0, 1, 2, 3, 4, 5)
    for i, (r, c) in enumerate(SHAPES):
        a = rng_matrix(i, r, c, dtype)
        if np.dtype(dtype) == np.int64:
            a = a % 5
        a.reshape(-1)[::3] = a.reshape(-1)[0]
        for op in ops:
            assert_bits_equal(o.aggRow(op, a), ref.aggRow(op, a), f"aggRow {op} {dtype.__name__} {r}x{c}")
            assert_bits_equal(o.aggCol(op, a), ref.aggCol(op, a), f"aggCol {op} {dtype.__name__} {r}x{c}")
            if op not in (4, 5):
                x, y = o.aggAll(op, a), ref.aggAll(op, a)
                assert x == y or (x != x and y != y), f"aggAll {op} {dtype.__name__} {r}x{c}: {x} {y}"
    # strided input (rowSkip > numCols) takes the per-row branch of AggAll (AggAll.h:147-163)
    big = rng_matrix(7, 50, 40, np.float64)
    v = big[:, 3:30]
    for op in (0, 2, 3, 6, 7, 8):
        assert o.aggAll(op, v) == ref.aggAll(op, v)
        assert_bits_equal(o.aggRow(op, v), ref.aggRow(op, v), "strided row")
        assert_bits_equal(o.aggCol(op, v), ref.aggCol(op, v), "strided col")


def test_nan_and_signed_zero_cases():
    rows = np.array([[np.nan, 1.0, 2.0], [1.0, np.nan, 2.0], [0.0, -0.0, 0.0], [-0.0, 0.0, -0.0],
                     [np.inf, np.nan, np.inf]])
    for a in (rows, np.ascontiguousarray(rows.T)):
        for op in (2, 3, 4, 5):
            assert_bits_equal(*_nanfix(o.aggRow(op, a), ref.aggRow(op, a)), f"row {op}")
            assert_bits_equal(*_nanfix(o.aggCol(op, a), ref.aggCol(op, a)), f"col {op}")


def test_contractions_and_helpers():
    """BLAS-backed kernels fix no summation order: tolerance 1e-12 relative to the largest entry; the rest is exact."""
    rng = np.random.default_rng(5)
    a, y = rng.random((300, 40)), rng.standard_normal((300, 1))
    for ta, tb, x, z in ((0, 0, a, rng.random((40, 17))), (1, 0, a, rng.random((300, 9))),
                         (0, 1, a, rng.random((11, 40))), (1, 1, a, rng.random((7, 300)))):
        g, e = o.matMul(x, z, ta, tb), ref.matMul(x, z, ta, tb)
        assert np.abs(g - e).max() <= 1e-12 * np.abs(e).max()
    for tl in (True, False):
        g, e = o.syrk(a, tl), ref.syrk(a, tl)
        assert np.abs(g - e).max() <= 1e-12 * np.abs(e).max()
    assert np.abs(o.gemv(a, y) - ref.gemv(a, y)).max() <= 1e-12 * np.abs(ref.gemv(a, y)).max()
    s = o.syrk(a) + 0.001 * np.eye(40)
    b = o.gemv(a, y)
    assert np.abs(o.solve(s, b) - ref.solve(s, b)).max() <= 1e-9 * np.abs(ref.solve(s, b)).max()
    ints = rng.integers(-5, 6, size=(30, 12)).astype(np.float64)
    assert_bits_equal(o.syrk(ints), ref.syrk(ints), "integer syrk")
    assert_bits_equal(o.matMul(ints, ints, True, False), ref.matMul(ints, ints, True, False), "integer matMul")
    assert_bits_equal(o.transpose(a), ref.transpose(a), "transpose")
    l, r = rng.integers(0, 5, 200), rng.integers(0, 7, 200)
    assert_bits_equal(o.ctable(l, r), ref.ctable(l, r), "ctable")
    assert_bits_equal(o.ctable(l, r, 2.0, 3, 4), ref.ctable(l, r, 2.0, 3, 4), "ctable given shape")
    for args in ((1, 10, 1), (0, 1, 0.1), (10, 1, -3), (5, 5, 1), (1, 1000, 7)):
        assert_bits_equal(o.seq(*args), ref.seq(*args), f"seq {args}")
