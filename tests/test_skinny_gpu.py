"""Tall-skinny products (n x K) @ op(B) with at most 64 result columns: the deferred product, the chain applied to its
accumulators, the fused row minimum / maximum with positions, the one-hot forms of ctable, and the fall-back paths.

Values of the product: |got - ref| <= 1e-12 * max|ref| (the reference calls cblas_dgemm, MatMul.cpp:284-288, which
fixes no summation order).  Positions (idxMin / idxMax) must be those of a left-to-right scan with strict comparison
(AggRow.h:71-96) over the values the device itself produced: they are checked against numpy's argmin/argmax of the
device's own D, and against the oracle's on inputs whose products are exact (small integers)."""
import numpy as np
import pytest

from tests.util import assert_bits_equal

pytestmark = pytest.mark.gpu


def _k():
    import daphne_b200.kernels as k
    from daphne_b200.kernels import AggOpCode as A, BinaryOpCode as B
    return k, A, B


def _close(got, exp, what, rtol=1e-12):
    assert got.shape == exp.shape, what
    err = np.abs(got - exp).max() / max(np.abs(exp).max(), 1e-300)
    assert err <= rtol, f"{what}: {err:.3e}"


@pytest.mark.parametrize("tb", [True, False])
def test_plain_product_shapes(ctx, tb):
    k, A, B = _k()
    rng = np.random.default_rng(21)
    for n, kk, m in [(70000, 64, 50), (66000, 1, 1), (9000, 7, 9), (5000, 16, 64), (4100, 100, 33), (8200, 128, 8),
                     (131072 + 5, 64, 64), (20000, 63, 17)]:
        x = rng.standard_normal((n, kk))
        c = rng.standard_normal((m, kk) if tb else (kk, m))
        got = k.matMul(k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, c), False, tb).to_numpy()
        _close(got, x @ (c.T if tb else c), f"{n}x{kk} @ {m} tb={tb}")


def test_kmeans_distance_chain_and_idxmin(ctx):
    k, A, B = _k()
    rng = np.random.default_rng(22)
    n, d, kc = 200000, 64, 50
    x = rng.random((n, d))
    c = x[rng.choice(n, kc, replace=False)].copy()
    X, C = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, c)
    xs = k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, X, 2.0))
    cs = k.transpose(k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, C, 2.0)))
    for _ in range(2):  # second round: xs is materialised
        xc = k.matMul(X, C, False, True)
        D = k.ewBinaryMat(B.ADD, k.ewBinaryMat(B.ADD, k.ewBinaryObjSca(B.MUL, xc, -2.0), xs), cs)
        idx = k.aggRow(A.IDXMIN, D)
        mn = k.aggRow(A.MIN, D)
        got_idx, got_min, got_d = idx.to_numpy().ravel(), mn.to_numpy().ravel(), D.to_numpy()
        ref_d = (x @ c.T) * -2.0 + (x * x).sum(1, keepdims=True) + (c * c).sum(1)[None, :]
        _close(got_d, ref_d, "D", 1e-12)
        assert np.array_equal(got_idx, got_d.argmin(1)), "idxMin follows the device's own D"
        assert_bits_equal(got_min, got_d.min(1), "row minimum of the device's own D")
        # the chosen centroid is a nearest one up to rounding of D
        assert (ref_d[np.arange(n), got_idx] <= ref_d.min(1) + 1e-9).all()


def test_fused_extrema_ties_and_nan(ctx):
    k, A, B = _k()
    rng = np.random.default_rng(23)
    n, d, kc = 70000, 8, 12
    x = rng.integers(-3, 4, size=(n, d)).astype(np.float64)  # exact products, many ties
    c = rng.integers(-2, 3, size=(kc, d)).astype(np.float64)
    x[5, 0] = np.nan         # row 5: every product is NaN
    c2 = c.copy()
    X, C = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, c2)
    xc = k.matMul(X, C, False, True)
    D = k.ewBinaryObjSca(B.ADD, xc, 1.0)
    imin, imax = k.aggRow(A.IDXMIN, D), k.aggRow(A.IDXMAX, D)
    vmin, vmax = k.aggRow(A.MIN, D), k.aggRow(A.MAX, D)
    ref = x @ c.T + 1.0
    ok = np.ones(n, bool)
    ok[5] = False
    assert np.array_equal(imin.to_numpy().ravel()[ok], ref[ok].argmin(1))
    assert np.array_equal(imax.to_numpy().ravel()[ok], ref[ok].argmax(1))
    assert_bits_equal(vmin.to_numpy().ravel()[ok], ref[ok].min(1), "min")
    assert_bits_equal(vmax.to_numpy().ravel()[ok], ref[ok].max(1), "max")
    # a NaN in column 0 stays: position 0, value NaN (sequential scan of the reference)
    assert imin.to_numpy()[5, 0] == 0 and imax.to_numpy()[5, 0] == 0
    assert np.isnan(vmin.to_numpy()[5, 0]) and np.isnan(vmax.to_numpy()[5, 0])
    # NaN only in later columns: skipped by the strict comparisons
    c3 = c.copy()
    c3[4, :] = np.nan
    xc = k.matMul(k.DenseMatrix.from_numpy(ctx, x[:65536 + 8]), k.DenseMatrix.from_numpy(ctx, c3), False, True)
    got = k.aggRow(A.IDXMIN, k.ewBinaryObjSca(B.ADD, xc, 1.0)).to_numpy().ravel()
    ref3 = x[:65536 + 8] @ c3.T + 1.0
    rows = np.array([r for r in range(ref3.shape[0]) if r != 5])
    assert np.array_equal(got[rows], np.nanargmin(ref3[rows], 1))
    # NaN in column 0 only: the scan starts there and no comparison with a NaN succeeds, so it stays
    c4 = c.copy()
    c4[0, :] = np.nan
    xc = k.matMul(k.DenseMatrix.from_numpy(ctx, x[:65536 + 8]), k.DenseMatrix.from_numpy(ctx, c4), False, True)
    D4 = k.ewBinaryObjSca(B.ADD, xc, 1.0)
    assert (k.aggRow(A.IDXMIN, D4).to_numpy() == 0).all() and (k.aggRow(A.IDXMAX, D4).to_numpy() == 0).all()
    assert np.isnan(k.aggRow(A.MIN, D4).to_numpy()).all() and np.isnan(k.aggRow(A.MAX, D4).to_numpy()).all()


def test_chain_that_cannot_be_fused_falls_back(ctx):
    k, A, B = _k()
    rng = np.random.default_rng(24)
    n, d, kc = 70000, 16, 10
    x, c, m = rng.standard_normal((n, d)), rng.standard_normal((kc, d)), rng.standard_normal((n, kc))
    X, C, M = (k.DenseMatrix.from_numpy(ctx, a) for a in (x, c, m))
    xc = k.matMul(X, C, False, True)
    D = k.ewBinaryMat(B.MUL, xc, M)  # same-shape operand: the product is written out first
    s = k.aggRow(A.SUM, D)
    ref = (x @ c.T) * m
    _close(D.to_numpy(), ref, "D")
    np.testing.assert_allclose(s.to_numpy().ravel(), ref.sum(1), rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(k.aggCol(A.SUM, k.matMul(X, C, False, True)).to_numpy().ravel(), (x @ c.T).sum(0),
                               rtol=1e-9, atol=1e-8)


def test_one_hot_ctable_consumers(ctx):
    k, A, B = _k()
    rng = np.random.default_rng(25)
    n, d, kc = 150000, 64, 50
    x = rng.random((n, d))
    a = rng.integers(0, kc, size=(n, 1)).astype(np.int64)
    a[a == 7] = 8  # an empty cluster
    X, Av = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, a)
    rows = k.seq(ctx, 0, n - 1, 1, dtype=np.int64)
    P = k.ctable(rows, Av, 1.0, n, kc)
    sums = k.matMul(P, X, True, False).to_numpy()
    counts = k.aggCol(A.SUM, P).to_numpy().ravel()
    p = np.zeros((n, kc))
    p[np.arange(n), a.ravel()] = 1.0
    _close(sums, p.T @ x, "t(P) @ X")
    assert_bits_equal(counts, p.sum(0), "sum(P, 1)")
    assert counts[7] == 0 and (sums[7] == 0).all()
    assert_bits_equal(P.to_numpy(), p, "P written out on demand")
    # other shapes: narrow X (general column loop) and a wide one that needs fewer accumulator copies
    for dd in (3, 200):
        x2 = rng.random((n, dd))
        P2 = k.ctable(rows, Av, 1.0, n, kc)
        _close(k.matMul(P2, k.DenseMatrix.from_numpy(ctx, x2), True, False).to_numpy(), p.T @ x2, f"d={dd}")


def _assign_and_sums(k, A, B, ctx, x, c, bump=None):
    """One k-means step by operator calls: nearest centroid of every row, then t(P) @ X and sum(P, 1)."""
    n, kc = x.shape[0], c.shape[0]
    X, C = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, c)
    xs = k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, X, 2.0))
    cs = k.transpose(k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, C, 2.0)))
    xc = k.matMul(X, C, False, True)
    D = k.ewBinaryMat(B.ADD, k.ewBinaryMat(B.ADD, k.ewBinaryObjSca(B.MUL, xc, -2.0), xs), cs)
    a = k.castObj(k.aggRow(A.IDXMIN, D), np.int64)
    P = k.ctable(k.seq(ctx, 0, n - 1, 1, dtype=np.int64), a, 1.0, n, kc)
    Y = X if bump is None else bump(X)
    sums = k.matMul(P, Y, True, False)
    counts = k.aggCol(A.SUM, P)
    return a.to_numpy().ravel(), sums.to_numpy(), counts.to_numpy().ravel()


@pytest.mark.parametrize("n,kc", [(200003, 50), (70000, 64), (4100, 3), (148 * 256 * 3 + 17, 50)])
def test_cluster_sums_of_integer_valued_rows_are_exact(ctx, n, kc):
    """t(P) @ X and sum(P, 1) for the one-hot P of a k-means step that is never written out.  Integer-valued X: every
    order of summation gives the same bits, so the sums must equal numpy's exactly, and a second run must repeat."""
    k, A, B = _k()
    rng = np.random.default_rng(31)
    x = rng.integers(-8, 9, size=(n, 64)).astype(np.float64)
    c = x[rng.choice(n, kc, replace=False)].copy() + 0.25
    a, sums, counts = _assign_and_sums(k, A, B, ctx, x, c)
    ref = np.zeros((kc, 64))
    np.add.at(ref, a, x)
    assert_bits_equal(sums, ref, "per-cluster sums of integer-valued rows")
    assert np.array_equal(counts, np.bincount(a, minlength=kc).astype(np.float64))
    a2, sums2, _ = _assign_and_sums(k, A, B, ctx, x, c)
    assert np.array_equal(a, a2)
    assert_bits_equal(sums2, sums, "repeatable")


def test_cluster_sums_of_real_valued_rows_repeat_bit_for_bit(ctx):
    """No atomics and a fixed order of additions: the sums of real-valued rows are the same bits in every run."""
    k, A, B = _k()
    rng = np.random.default_rng(32)
    n, kc = 300000, 50
    x = rng.random((n, 64))
    c = x[rng.choice(n, kc, replace=False)].copy()
    a, sums, _ = _assign_and_sums(k, A, B, ctx, x, c)
    ref = np.zeros((kc, 64))
    np.add.at(ref, a, x)
    _close(sums, ref, "per-cluster sums", 1e-13)
    for _ in range(3):
        a2, sums2, _ = _assign_and_sums(k, A, B, ctx, x, c)
        assert np.array_equal(a, a2)
        assert_bits_equal(sums2, sums, "same order of additions in every run")


def test_cluster_sums_of_another_matrix_than_the_distances_came_from(ctx):
    """t(P) @ Y for a Y that is not the X the distances were computed from."""
    k, A, B = _k()
    rng = np.random.default_rng(33)
    n, kc = 50000, 20
    x = rng.integers(-8, 9, size=(n, 64)).astype(np.float64)
    c = x[rng.choice(n, kc, replace=False)].copy() + 0.25
    a, sums, _ = _assign_and_sums(k, A, B, ctx, x, c, bump=lambda X: k.ewBinaryObjSca(B.ADD, X, 1.0))
    ref = np.zeros((kc, 64))
    np.add.at(ref, a, x + 1.0)
    assert_bits_equal(sums, ref, "sums of the other matrix")


def test_cast_between_the_64_bit_integer_types_shares_the_buffer_but_not_later_writes(ctx):
    """castObj ui64 <-> si64 hands out a second handle on the same device buffer (no kernel, no copy); overwriting one
    of the two matrices afterwards must leave the other one as it was."""
    k, A, B = _k()
    from daphne_b200.lib import lib
    a = np.array([[0], [5], [2 ** 63 + 7], [2 ** 64 - 1]], dtype=np.uint64)
    U = k.DenseMatrix.from_numpy(ctx, a)
    U.device_ptr()
    before = lib.db2_launch_count()
    S = k.castObj(U, np.int64)
    assert lib.db2_launch_count() == before
    assert S.dtype == np.int64 and np.array_equal(S.to_numpy(), a.astype(np.int64))
    back = k.castObj(S, np.uint64)
    assert np.array_equal(back.to_numpy(), a)
    # a result written "into" U (pre-allocated result) must not show through S
    T = k.ewBinaryObjSca(B.ADD, S, 1)
    assert np.array_equal(S.to_numpy(), a.astype(np.int64))
    assert np.array_equal(T.to_numpy(), a.astype(np.int64) + 1)
