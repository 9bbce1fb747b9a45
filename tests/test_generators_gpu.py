"""rand() with a device-resident result against the reference's own RandMatrix kernel (bit for bit: same engines, same
draw order), and row / column ranges as zero-copy views."""
import numpy as np
import pytest

from tests.util import assert_bits_equal

pytestmark = pytest.mark.gpu


def _k():
    import daphne_b200.kernels as k
    from oracle import refkernels as ref
    return k, ref


@pytest.mark.parametrize("rows,cols,lo,hi,sparsity,seed", [
    (100_000, 100, 0.0, 1.0, 1.0, 42),     # DaphneDSL rand(100000, 100, 0.0, 1.0, 1, 42): the lmDS input
    (1000, 64, -1.0, 1.0, 1.0, 5),
    (3, 7, 2.0, 9.0, 1.0, 0),
    (500, 40, 0.0, 1.0, 0.3, 7),            # mostly zeros: values placed by selection sampling
    (500, 40, -2.0, 3.0, 0.7, 8),           # mostly values: zeros placed by selection sampling
    (200, 30, 0.0, 1.0, 0.0, 9),            # all zeros
    (200, 30, 0.0, 1.0, 0.5, 10),
])
def test_rand_matrix_has_the_references_stream(ctx, rows, cols, lo, hi, sparsity, seed):
    k, ref = _k()
    if not ref.available():
        pytest.skip("the reference-built kernels are not present")
    got = k.randMatrix(ctx, rows, cols, lo, hi, sparsity, seed).to_numpy()
    assert_bits_equal(got, ref.rand(rows, cols, lo, hi, sparsity, seed), f"rand {rows}x{cols} sparsity {sparsity}")


def test_rand_matrix_other_types_and_errors(ctx):
    k, _ = _k()
    f = k.randMatrix(ctx, 300, 20, 0.0, 1.0, 1.0, 3, dtype=np.float32).to_numpy()
    assert f.dtype == np.float32 and f.min() > 0.0 and f.max() < 1.0 and abs(f.mean() - 0.5) < 0.02
    i = k.randMatrix(ctx, 300, 20, -5, 5, 1.0, 3, dtype=np.int64).to_numpy()
    assert i.dtype == np.int64 and i.min() >= -5 and i.max() <= 5 and not (i == 0).any()  # zeros are redrawn
    a, b = (k.randMatrix(ctx, 50, 5, 0.0, 1.0, 1.0, 11).to_numpy() for _ in range(2))
    assert_bits_equal(a, b, "same seed, same matrix")
    for args, msg in (((0, 5, 0.0, 1.0, 1.0, 1), "numRows must be > 0"), ((5, 0, 0.0, 1.0, 1.0, 1), "numCols must be > 0"),
                      ((5, 5, 2.0, 1.0, 1.0, 1), "min must be <= max"), ((5, 5, 0.0, 0.0, 1.0, 1), "must not both be zero"),
                      ((5, 5, 0.0, 1.0, 1.5, 1), "sparsity has to be in the interval")):
        with pytest.raises(k.Db2Error, match=msg):
            k.randMatrix(ctx, *args)


def test_slice_row_and_col_are_views_with_the_references_index_rules(ctx):
    k, _ = _k()
    B, A = k.BinaryOpCode, k.AggOpCode
    x = np.random.default_rng(1).standard_normal((4000, 37))
    X = k.DenseMatrix.from_numpy(ctx, x)
    X.device_ptr()
    for lo, hi in ((0, 37), (3, 20), (5, 6), (-10, -2), (-5, 0), (36, 37), (2, 2)):
        a = lo + 37 if lo < 0 else lo
        b = hi + 37 if (hi < 0 or (lo < 0 and hi <= 0)) else hi
        v = k.sliceCol(X, lo, hi)
        assert v.shape == (4000, b - a)
        assert v.device_ptr()[0] == X.device_ptr()[0] + 8 * a, "a column range is a view, not a copy"
        assert_bits_equal(v.to_numpy(), np.ascontiguousarray(x[:, a:b]), f"sliceCol {lo}:{hi}")
        if b > a:  # kernels honour the view's leading dimension and its (possibly unaligned) first column
            assert_bits_equal(k.aggRow(A.MAX, v).to_numpy(), x[:, a:b].max(axis=1, keepdims=True), "aggRow on a view")
            np.testing.assert_allclose(k.aggCol(A.SUM, v).to_numpy(), x[:, a:b].sum(axis=0, keepdims=True), rtol=1e-12)
            assert_bits_equal(k.ewBinaryObjSca(B.MUL, v, 3.0).to_numpy(), x[:, a:b] * 3.0, "elementwise on a view")
    r = k.sliceRow(X, -100, 0)
    assert_bits_equal(r.to_numpy(), x[-100:], "sliceRow with negative bounds")
    assert_bits_equal(k.sliceCol(k.sliceRow(X, 10, 500), 4, 9).to_numpy(), np.ascontiguousarray(x[10:500, 4:9]), "both")
    for f, lo, hi in ((k.sliceCol, 37, 38), (k.sliceCol, 5, 3), (k.sliceCol, 0, 40), (k.sliceRow, 4000, 4001)):
        with pytest.raises(k.Db2Error, match="invalid arguments"):
            f(X, lo, hi)
