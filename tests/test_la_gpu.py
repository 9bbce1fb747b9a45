"""Contractions and helper kernels (matMul, syrk, gemv, solve, transpose, fill, seq, diagMatrix, ctable, castObj)
against the CPU oracle.

Tolerance for the contractions: |got - ref| <= 1e-12 * max|ref| per result (relative to the largest entry: the
reference computes them with OpenBLAS, which fixes no summation order, so entries that cancel to nearly zero cannot be
compared relative to themselves).  Integer-valued inputs, as in the reference's MatMulTest/SyrkTest, must match
exactly."""
import numpy as np
import pytest

from tests.util import assert_bits_equal

pytestmark = pytest.mark.gpu
RTOL = 1e-12


def _k():
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    return k, o


def _close(got, exp, what):
    assert got.shape == exp.shape, what
    scale = max(np.abs(exp).max(), 1e-300)
    err = np.abs(got - exp).max() / scale
    assert err <= RTOL, f"{what}: {err:.3e}"


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_matmul_all_transpose_combinations(ctx, ta, tb):
    k, o = _k()
    rng = np.random.default_rng(1)
    for (m, n, kk) in [(1, 1, 1), (5, 7, 3), (64, 64, 16), (130, 70, 37), (257, 50, 64), (33, 129, 1000), (8, 8, 5000),
                       (300, 200, 150), (128, 128, 64), (384, 256, 2000), (130, 258, 96)]:
        a = rng.standard_normal((kk, m) if ta else (m, kk))
        b = rng.standard_normal((n, kk) if tb else (kk, n))
        got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b), ta, tb).to_numpy()
        _close(got, o.matMul(a, b, ta, tb), f"matMul {m}x{n}x{kk} ta={ta} tb={tb}")


def test_matmul_integer_valued_inputs_are_exact(ctx):
    k, o = _k()
    rng = np.random.default_rng(2)
    a = rng.integers(-9, 10, size=(77, 130)).astype(np.float64)
    b = rng.integers(-9, 10, size=(130, 41)).astype(np.float64)
    got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
    assert_bits_equal(got, a @ b, "integer matMul")
    got = k.syrk(k.DenseMatrix.from_numpy(ctx, a)).to_numpy()
    assert_bits_equal(got, a.T @ a, "integer syrk")


def test_matmul_on_views_and_odd_leading_dimensions(ctx):
    k, o = _k()
    rng = np.random.default_rng(3)
    big = rng.standard_normal((500, 71))
    a = big[:, 3:60]           # ld 71 (odd), offset 3
    b = rng.standard_normal((57, 29))
    got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
    _close(got, o.matMul(np.ascontiguousarray(a), b), "strided lhs")
    A = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((4000, 64)))
    v = A.slice_rows(1000, 3001)
    c = rng.standard_normal((50, 64))
    got = k.matMul(v, k.DenseMatrix.from_numpy(ctx, c), False, True).to_numpy()
    _close(got, o.matMul(A.to_numpy()[1000:3001], c, False, True), "row view x t(C)")


def test_matmul_shape_mismatch_raises(ctx):
    k, o = _k()
    a, b = np.ones((4, 5)), np.ones((4, 5))
    with pytest.raises(k.Db2Error, match="#cols of lhs and #rows of rhs must be the same"):
        k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b))
    with pytest.raises(o.OracleError):
        o.matMul(a, b)


@pytest.mark.parametrize("n,d", [(1000, 1), (5000, 7), (20000, 33), (100000, 100), (40000, 512), (300, 700)])
def test_syrk_and_gemv_tall_skinny(ctx, n, d):
    k, o = _k()
    rng = np.random.default_rng(4)
    x = rng.random((n, d))
    y = rng.standard_normal((n, 1))
    X, Y = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y)
    a = k.syrk(X, True).to_numpy()
    ref = x.T @ x  # same tolerance class as the oracle's triple loop; the oracle itself is checked below for small d
    _close(a, ref, f"syrk {n}x{d}")
    assert_bits_equal(a, a.T.copy(), "syrk result is exactly symmetric")
    if n * d * d <= 4e8:
        _close(a, o.syrk(x, True), f"syrk vs oracle {n}x{d}")
    _close(k.gemv(X, Y).to_numpy(), o.gemv(x, y), f"gemv {n}x{d}")
    if n <= 5000:
        _close(k.syrk(X, False).to_numpy(), o.syrk(x, False), f"syrk X t(X) {n}x{d}")


def test_syrk_equals_transpose_then_matmul(ctx):
    """The reference's SyrkTest checks syrk against transpose followed by matMul (SyrkTest.cpp:32-58)."""
    k, o = _k()
    x = np.random.default_rng(5).integers(-5, 6, size=(300, 40)).astype(np.float64)
    X = k.DenseMatrix.from_numpy(ctx, x)
    assert_bits_equal(k.syrk(X).to_numpy(), k.matMul(k.transpose(X), X).to_numpy(), "syrk == t(X) @ X")


def test_normal_equations_solve(ctx):
    k, o = _k()
    rng = np.random.default_rng(6)
    for n, d in [(2000, 5), (20000, 100), (30000, 512)]:
        x = rng.random((n, d))
        w = rng.standard_normal((d, 1))
        y = x @ w + 0.01 * rng.standard_normal((n, 1))
        X, Y = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y)
        lam = k.fill(ctx, 0.001, d, 1)
        A = k.ewBinaryMat(k.BinaryOpCode.ADD, k.syrk(X), k.diagMatrix(lam))
        b = k.gemv(X, Y)
        beta = k.solve(A, b).to_numpy()
        a_cpu = x.T @ x + 0.001 * np.eye(d)
        ref = o.solve(a_cpu, x.T @ y)
        # the normal equations are ill-conditioned (cond ~ 1e3..1e5): compare through the residual and loosely on beta
        assert np.abs(beta - ref).max() <= 1e-7 * np.abs(ref).max(), f"beta {n}x{d}"
        res = np.abs(a_cpu @ beta - x.T @ y).max() / np.abs(x.T @ y).max()
        assert res <= 1e-12, f"residual {res:.2e}"
        assert np.abs(beta - w).max() < 0.05


def test_solve_general_and_singular(ctx):
    k, o = _k()
    rng = np.random.default_rng(7)
    for n in (1, 2, 17, 100, 300):
        a = rng.standard_normal((n, n)) + n * np.eye(n)
        a[[0, n - 1]] = a[[n - 1, 0]]  # force row exchanges
        b = rng.standard_normal((n, 1))
        got = k.solve(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
        ref = o.solve(a, b)
        assert np.abs(got - ref).max() <= 1e-10 * np.abs(ref).max(), n
    # pivots that sit below the block row of their panel, several exchanges with the same row, n not a multiple of 32
    for n in (97, 200, 512, 515):
        a = rng.standard_normal((n, n))
        a[: n // 2] *= 1e-3                           # the large entries, hence the pivots, are in the lower half
        b = rng.standard_normal((n, 1))
        got = k.solve(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
        ref = o.solve(a, b)
        assert np.abs(got - ref).max() <= 1e-7 * np.abs(ref).max(), n
        assert np.abs(a @ got - b).max() <= 1e-9 * max(1.0, np.abs(got).max()) * np.abs(a).max() * n, n
    a32 = (rng.standard_normal((150, 150)) + 150 * np.eye(150)).astype(np.float32)
    b32 = rng.standard_normal((150, 1)).astype(np.float32)
    got = k.solve(k.DenseMatrix.from_numpy(ctx, a32), k.DenseMatrix.from_numpy(ctx, b32)).to_numpy()
    exact = np.linalg.solve(a32.astype(np.float64), b32.astype(np.float64))
    assert got.dtype == np.float32 and np.abs(got - exact).max() <= 2.0 ** -22 * np.abs(exact).max()
    sing = np.zeros((3, 3))
    sing[0, 0] = 1.0
    with pytest.raises(k.Db2Error, match="exactly singular"):
        k.solve(k.DenseMatrix.from_numpy(ctx, sing), k.DenseMatrix.from_numpy(ctx, np.ones((3, 1))))
    with pytest.raises(o.OracleError):
        o.solve(sing, np.ones((3, 1)))
    with pytest.raises(k.Db2Error, match="#rows and #cols of lhs must be the same"):
        k.solve(k.DenseMatrix.from_numpy(ctx, np.ones((3, 2))), k.DenseMatrix.from_numpy(ctx, np.ones((3, 1))))


@pytest.mark.parametrize("n", [600, 1024])
def test_solve_with_a_nan_column_stays_inside_its_buffers(ctx, n):
    """A column of NaNs (what one NaN in X makes of t(X) X after the first update) leaves the pivot search without a
    candidate.  The factorisation must report the singular / NaN pivot and must not touch memory outside the n x n work
    matrix and the n-element right-hand side: both are laid out here with guard words around them."""
    import ctypes as C
    from daphne_b200.lib import check, lib
    rng = np.random.default_rng(n)
    a = rng.standard_normal((n, n)) + n * np.eye(n)
    a[:, 5] = np.nan
    a[5, :] = np.nan
    b = rng.standard_normal((n, 1))
    guard = 512
    host = np.full(guard + n * n + guard + n + guard, 7.25)
    host[guard:guard + n * n] = a.ravel()
    host[guard + n * n + guard:guard + n * n + guard + n] = b.ravel()
    dev, scr, st = C.c_void_p(), C.c_void_p(), C.c_void_p()
    check(lib.db2_malloc(C.byref(dev), host.nbytes))
    sbytes = lib.db2k_solve_scratch_bytes(n)
    check(lib.db2_malloc(C.byref(scr), sbytes))
    check(lib.db2_malloc(C.byref(st), 4))
    check(lib.db2_memcpy_h2d(dev, host.ctypes.data, host.nbytes, None))
    a_ptr = C.c_void_p(dev.value + guard * 8)
    x_ptr = C.c_void_p(dev.value + (guard + n * n + guard) * 8)
    check(lib.db2k_solve(0, a_ptr, n, x_ptr, st, scr, sbytes, None))
    check(lib.db2_device_sync())
    back = np.empty_like(host)
    status = np.zeros(1, dtype=np.int32)
    check(lib.db2_memcpy_d2h(back.ctypes.data, dev, host.nbytes, None))
    check(lib.db2_memcpy_d2h(status.ctypes.data, st, 4, None))
    check(lib.db2_device_sync())
    for p in (dev, scr, st):
        check(lib.db2_free(p))
    assert status[0] != 0, "a NaN pivot column must be reported"
    assert np.all(back[:guard] == 7.25) and np.all(back[-guard:] == 7.25)
    assert np.all(back[guard + n * n:guard + n * n + guard] == 7.25)
    k, _ = _k()
    with pytest.raises(k.Db2Error, match="exactly singular"):
        k.solve(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b))


def test_transpose_fill_seq_diag_cast(ctx):
    k, o = _k()
    rng = np.random.default_rng(8)
    for r, c in [(1, 1), (3, 5), (33, 65), (1000, 50), (70, 1)]:
        a = rng.standard_normal((r, c))
        assert_bits_equal(k.transpose(k.DenseMatrix.from_numpy(ctx, a)).to_numpy(), o.transpose(a), f"t {r}x{c}")
    vec = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((1000, 1)))
    t = k.transpose(vec)
    assert t.shape == (1, 1000) and t.device_ptr()[0] == vec.device_ptr()[0], "vectors are reshaped in place"
    assert_bits_equal(k.fill(ctx, 2.5, 7, 9).to_numpy(), np.full((7, 9), 2.5), "fill")
    for s, e, i in [(1.0, 100000.0, 1.0), (0.0, 9.0, 3.0), (10.0, 1.0, -3.0), (5.0, 5.0, 1.0), (1.0, 10.0, -1.0)]:
        assert_bits_equal(k.seq(ctx, s, e, i).to_numpy(), o.seq(s, e, i), f"seq {s} {e} {i}")
    with pytest.raises(k.Db2Error, match="inc should not be zero"):
        k.seq(ctx, 1.0, 2.0, 0.0)
    d = rng.standard_normal((37, 1))
    assert_bits_equal(k.diagMatrix(k.DenseMatrix.from_numpy(ctx, d)).to_numpy(), np.diag(d[:, 0]), "diagMatrix")
    u = np.arange(50, dtype=np.uint64).reshape(-1, 1)
    assert_bits_equal(k.castObj(k.DenseMatrix.from_numpy(ctx, u), np.int64).to_numpy(), u.astype(np.int64), "cast")


def test_fill_shapes_and_values_of_the_reference_test(ctx):
    """FillTest.cpp:41-92: empty, vector and rectangular shapes, a zero and a non-zero value, several value types."""
    k, o = _k()
    shapes = [(0, 0), (0, 1), (0, 5), (1, 0), (5, 0), (1, 1), (1, 5), (1, 1000), (5, 1), (1000, 1), (3, 4), (1000, 1000)]
    for dtype in (np.float64, np.int64, np.float32):
        for rows, cols in shapes:
            for value in (0, 2.5):
                got = k.fill(ctx, value, rows, cols, dtype=dtype).to_numpy()
                exp = np.full((rows, cols), np.array([value]).astype(dtype)[0], dtype=dtype)
                assert got.shape == exp.shape and got.dtype == exp.dtype and np.array_equal(got, exp), (dtype, rows, cols)


def test_col_bind_and_extract_col(ctx):
    """ColBind.h:54-88 and ExtractCol.h:64-105 against their restatements, incl. views, empty operands, negative
    positions and the reference's errors."""
    k, o = _k()
    rng = np.random.default_rng(12)
    for dtype in (np.float64, np.float32, np.int64):
        for rows, cl, cr in [(1, 1, 1), (5, 3, 2), (1000, 32, 1), (70001, 7, 33), (300, 0, 5), (300, 5, 0), (0, 3, 2)]:
            a = (rng.standard_normal((rows, cl)) * 100).astype(dtype)
            b = (rng.standard_normal((rows, cr)) * 100).astype(dtype)
            got = k.colBind(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
            exp = o.colBind(a, b) if rows and cl + cr else np.empty((rows, cl + cr), dtype)
            assert got.shape == exp.shape and got.dtype == exp.dtype and np.array_equal(got, exp), (dtype, rows, cl, cr)
        x = (rng.standard_normal((40000, 37)) * 100).astype(dtype)
        X = k.DenseMatrix.from_numpy(ctx, x)
        for sel in ([0], [36, 0, 5], [-1, -37, 3, 3, 3], list(range(37)), list(range(36, -1, -1)) * 3, []):
            s = np.array(sel, dtype=np.int64).reshape(-1, 1)
            got = k.extractCol(X, k.DenseMatrix.from_numpy(ctx, s)).to_numpy()
            exp = o.extractCol(x, s)
            assert got.shape == exp.shape and got.dtype == exp.dtype and np.array_equal(got, exp), (dtype, sel)
    # row views keep their offset; a deferred elementwise result is a valid operand
    big = rng.standard_normal((5000, 16))
    B_ = k.DenseMatrix.from_numpy(ctx, big)
    v = B_.slice_rows(100, 4100)
    w = k.ewBinaryObjSca(k.BinaryOpCode.MUL, k.DenseMatrix.from_numpy(ctx, rng.standard_normal((4000, 20))), 2.0)
    got = k.colBind(v, w).to_numpy()
    assert np.array_equal(got, np.hstack([big[100:4100], w.to_numpy()]))
    s = np.array([[15], [0], [-2]], dtype=np.int64)
    assert np.array_equal(k.extractCol(v, k.DenseMatrix.from_numpy(ctx, s)).to_numpy(), big[100:4100][:, [15, 0, 14]])
    with pytest.raises(k.Db2Error, match="must have the same number of rows, but lhs has 4000 and rhs has 5000"):
        k.colBind(v, B_)
    for bad in ([16], [-17], [3, 99]):
        with pytest.raises(k.Db2Error, match="out of bounds for dense matrix with column boundaries"):
            k.extractCol(B_, k.DenseMatrix.from_numpy(ctx, np.array(bad, dtype=np.int64).reshape(-1, 1)))
    with pytest.raises(k.Db2Error, match="must be given as column matrix"):
        k.extractCol(B_, k.DenseMatrix.from_numpy(ctx, np.zeros((2, 2), dtype=np.int64)))


def test_one_hot(ctx):
    """OneHot.h:54-110 against its restatement: keep / drop / expand, f64 and int64, fractional values cut to their
    integer part, views, and the reference's errors (bad info, values outside their block)."""
    k, o = _k()
    rng = np.random.default_rng(14)
    for dtype in (np.float64, np.int64):
        for rows in (1, 7, 4000, 70001):
            x = np.empty((rows, 5), dtype=dtype)
            x[:, 0] = rng.integers(-50, 50, size=rows)
            x[:, 1] = rng.integers(0, 4, size=rows)
            x[:, 2] = rng.integers(0, 40, size=rows)
            x[:, 3] = rng.integers(0, 2, size=rows)
            x[:, 4] = rng.integers(-5, 5, size=rows)
            if dtype == np.float64:
                x[:, 1] += 0.75  # cut to the integer part
            for info in ([-1, 4, 40, 2, -1], [0, 4, 0, 0, 0], [-1, 0, 0, 0, -1], [0, 0, 40, 2, 0]):
                inf = np.array([info], dtype=np.int64)
                got = k.oneHot(k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, inf)).to_numpy()
                exp = o.oneHot(x, inf) if rows <= 4000 else None
                if exp is None:  # the restatement is a Python loop: large cases against numpy
                    cols = []
                    for c, n in enumerate(info):
                        if n == -1:
                            cols.append(x[:, c:c + 1])
                        elif n > 0:
                            cols.append((np.trunc(x[:, c:c + 1]) == np.arange(n)[None, :]).astype(dtype))
                    exp = np.hstack(cols)
                assert got.shape == exp.shape and got.dtype == exp.dtype and np.array_equal(got, exp), (dtype, rows, info)
    x = rng.integers(0, 3, size=(3000, 2)).astype(np.float64)
    X = k.DenseMatrix.from_numpy(ctx, x)
    v = X.slice_rows(500, 2500)
    inf = k.DenseMatrix.from_numpy(ctx, np.array([[3, -1]], dtype=np.int64))
    assert np.array_equal(k.oneHot(v, inf).to_numpy(), o.oneHot(x[500:2500], np.array([[3, -1]])))
    for bad, msg in (([[2, -1]], "must be positive and smaller"), ([[-2, 1]], "greater or equal than -1"),
                     ([[0, 0]], "at least one non-zero entry"), ([[3]], "information for each column"),
                     ([[3], [3]], "must be a row matrix")):
        with pytest.raises(k.Db2Error, match=msg):
            k.oneHot(X, k.DenseMatrix.from_numpy(ctx, np.array(bad, dtype=np.int64)))
    neg = x.copy()
    neg[17, 0] = -1.0
    with pytest.raises(k.Db2Error, match="must be positive and smaller"):
        k.oneHot(k.DenseMatrix.from_numpy(ctx, neg), inf)


def test_ctable(ctx):
    k, o = _k()
    rng = np.random.default_rng(9)
    n = 100000
    lhs = np.arange(n, dtype=np.int64).reshape(-1, 1)
    rhs = rng.integers(0, 50, size=(n, 1), dtype=np.int64)
    L, R = k.DenseMatrix.from_numpy(ctx, lhs), k.DenseMatrix.from_numpy(ctx, rhs)
    assert_bits_equal(k.ctable(L, R, 1.0, n, 50).to_numpy(), o.ctable(lhs, rhs, 1.0, n, 50), "one-hot ctable")
    a = rng.integers(0, 9, size=(5000, 1), dtype=np.int64)
    b = rng.integers(0, 13, size=(5000, 1), dtype=np.int64)
    A, B = k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)
    assert_bits_equal(k.ctable(A, B).to_numpy(), o.ctable(a, b), "ctable, derived shape")
    assert_bits_equal(k.ctable(A, B, 3.0, 5, 20).to_numpy(), o.ctable(a, b, 3.0, 5, 20), "ctable, given shape")
    with pytest.raises(k.Db2Error, match="same number of rows"):
        k.ctable(A, R)


@pytest.mark.parametrize("dtype", [np.int64, np.int32])
def test_integer_matmul_bit_exact(ctx, dtype):
    """MatMul for the integer value types (the reference's Eigen path): wrapping arithmetic, so bit-exact against the
    triple loop for every transpose combination, ragged tile edges and values that overflow."""
    k, o = _k()
    rng = np.random.default_rng(17)
    info = np.iinfo(dtype)
    for (m, n, kk) in [(1, 1, 1), (3, 5, 7), (64, 64, 16), (65, 130, 33), (200, 1, 300), (1, 257, 129)]:
        for ta in (False, True):
            for tb in (False, True):
                a = rng.integers(-50, 50, size=(kk, m) if ta else (m, kk)).astype(dtype)
                b = rng.integers(-50, 50, size=(n, kk) if tb else (kk, n)).astype(dtype)
                got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b), ta, tb).to_numpy()
                exp = o.matMul(a, b, ta, tb)
                assert got.dtype == dtype and np.array_equal(got, exp), (m, n, kk, ta, tb)
                la, lb = (a.T if ta else a), (b.T if tb else b)
                assert np.array_equal(got, (la.astype(np.int64) @ lb.astype(np.int64)).astype(dtype))
    a = rng.integers(info.min, info.max, size=(70, 90), dtype=dtype)      # products and sums wrap
    b = rng.integers(info.min, info.max, size=(90, 40), dtype=dtype)
    got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
    assert np.array_equal(got, o.matMul(a, b))
    A = k.DenseMatrix.from_numpy(ctx, rng.integers(-9, 9, size=(500, 20)).astype(dtype))
    v = k.sliceRow(A, 100, 300)                                            # a row view keeps its offset
    c = rng.integers(-9, 9, size=(20, 6)).astype(dtype)
    assert np.array_equal(k.matMul(v, k.DenseMatrix.from_numpy(ctx, c)).to_numpy(), o.matMul(A.to_numpy()[100:300], c))


def test_syrk_followed_by_gemv_is_one_pass(ctx):
    """t(X) X is deferred for a large X; a gemv on the same X that follows is computed by the same kernel (the idle
    warps of the diagonal tiles form t(X) y from the stages in shared memory).  The syrk part is the unchanged
    arithmetic (bit-identical to the product computed alone); t(X) y within the reduction tolerance."""
    k, o = _k()
    rng = np.random.default_rng(23)
    for n, d in [(40000, 128), (9000, 512), (50000, 100), (33000, 130)]:
        x = rng.random((n, d)) * 2.0 - 1.0
        y = rng.standard_normal((n, 1))
        X, Y = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y)
        X.device_ptr()
        alone = k.syrk(X, True).to_numpy()                 # looked at right away: the product alone
        b_alone = k.gemv(X, Y).to_numpy()                  # no t(X) X waiting: the ordinary column pass
        s0 = ctx.stats()["launches"]
        A = k.syrk(X, True)
        assert ctx.stats()["launches"] == s0               # nothing has run yet
        b = k.gemv(X, Y)
        fused_launches = ctx.stats()["launches"] - s0
        assert fused_launches <= 3                         # product kernel, reduce of the splits, fold of t(X) y
        assert_bits_equal(A.to_numpy(), alone, f"t(X) X with t(X) y folded in, {n} x {d}")
        exact = x.T @ y
        scale = np.abs(x).T @ np.abs(y)
        assert np.all(np.abs(b.to_numpy() - exact) <= 1e-12 * scale), (n, d)
        assert np.all(np.abs(b_alone - exact) <= 1e-12 * scale)
    # the deferred product is computed alone when something else needs it first, or never when it is dropped
    x = rng.random((40000, 128))
    X = k.DenseMatrix.from_numpy(ctx, x)
    X.device_ptr()
    A1 = k.syrk(X, True)
    A2 = k.syrk(X, True)                                   # one waits at a time: A1 is computed here
    yv = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((40000, 3)))
    col = k.sliceCol(yv, 1, 2)                             # a strided column: the ordinary gemv, A2 keeps waiting
    b = k.gemv(X, col).to_numpy()
    assert np.all(np.abs(b - x.T @ yv.to_numpy()[:, 1:2]) <= 1e-11 * (np.abs(x).T @ np.abs(yv.to_numpy()[:, 1:2])))
    assert_bits_equal(A1.to_numpy(), A2.to_numpy(), "both deferred products")
    A3 = k.syrk(X, True)
    del A3                                                 # dropped: never computed, and nothing left behind
    other = k.DenseMatrix.from_numpy(ctx, rng.random((40000, 128)))
    b2 = k.gemv(other, k.DenseMatrix.from_numpy(ctx, np.ones((40000, 1)))).to_numpy()
    assert np.allclose(b2[:, 0], other.to_numpy().sum(0), rtol=1e-12)
