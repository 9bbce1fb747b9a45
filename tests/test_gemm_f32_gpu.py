"""f32 matMul / syrk (tensor-core path: tcgen05 kind::tf32 with split operands) against the exact product of the
same f32 inputs.

The reference computes these with cblas_sgemm / cblas_ssyrk (MatMul.cpp:31-36, Syrk.h:80-92), whose result is not
pinned to a summation order.  Tolerance: the classical sgemm bound  |got - exact| <= (k * 2^-24 + 2^-19) * (|A| |B|)
per entry (k = contraction length; 2^-19 covers the split-operand products), and, as a sharper practical check, the
largest error must stay within 4x of what OpenBLAS' sgemm (numpy's f32 matmul) makes on the same inputs plus 2^-19 of
the largest entry (the tensor core adds into its accumulator with truncation: sums of same-sign products drift by a
few ulp per 64 k before they are promoted to a round-to-nearest register accumulator).
Integer-valued inputs, as in the reference's MatMulTest / SyrkTest, must be exact."""
import numpy as np
import pytest

from tests.util import assert_bits_equal

pytestmark = pytest.mark.gpu


def _k():
    import daphne_b200.kernels as k
    return k


def _check(got, a, b, what):
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    exact = a64 @ b64
    kk = a.shape[1]
    bound = (kk * 2.0 ** -24 + 2.0 ** -19) * (np.abs(a64) @ np.abs(b64)) + 1e-30
    assert got.dtype == np.float32 and got.shape == exact.shape, what
    err = np.abs(got.astype(np.float64) - exact)
    assert (err <= bound).all(), f"{what}: worst err/bound {np.max(err / bound):.3e}"
    blas_err = np.abs((a @ b).astype(np.float64) - exact).max()
    assert err.max() <= 4.0 * blas_err + 2.0 ** -19 * np.abs(exact).max(), \
        f"{what}: max err {err.max():.3e} vs sgemm's {blas_err:.3e}"


def test_f32_matmul_one_tile(ctx):
    k = _k()
    rng = np.random.default_rng(11)
    a = rng.standard_normal((128, 64)).astype(np.float32)
    b = rng.standard_normal((64, 128)).astype(np.float32)
    got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
    _check(got, a, b, "128x128x64")


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_f32_matmul_all_transpose_combinations(ctx, ta, tb):
    k = _k()
    rng = np.random.default_rng(12)
    for (m, n, kk) in [(1, 1, 1), (5, 7, 3), (64, 64, 16), (130, 70, 37), (257, 50, 64), (33, 129, 1000),
                       (8, 8, 5000), (300, 200, 150), (1000, 50, 64), (50, 64, 100000), (512, 512, 4096)]:
        a = rng.standard_normal((m, kk)).astype(np.float32)
        b = rng.standard_normal((kk, n)).astype(np.float32)
        A = k.DenseMatrix.from_numpy(ctx, np.ascontiguousarray(a.T) if ta else a)
        B = k.DenseMatrix.from_numpy(ctx, np.ascontiguousarray(b.T) if tb else b)
        got = k.matMul(A, B, ta, tb).to_numpy()
        _check(got, a, b, f"matMul f32 {m}x{n}x{kk} ta={ta} tb={tb}")


def test_f32_integer_valued_inputs_are_exact(ctx):
    k = _k()
    rng = np.random.default_rng(13)
    a = rng.integers(-9, 10, size=(77, 130)).astype(np.float32)
    b = rng.integers(-9, 10, size=(130, 41)).astype(np.float32)
    got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
    assert_bits_equal(got, a @ b, "integer f32 matMul")
    x = rng.integers(-5, 6, size=(3000, 40)).astype(np.float32)
    X = k.DenseMatrix.from_numpy(ctx, x)
    s = k.syrk(X).to_numpy()
    assert_bits_equal(s, x.T @ x, "integer f32 syrk")
    assert_bits_equal(s, k.matMul(k.transpose(X), X).to_numpy(), "syrk == t(X) @ X (SyrkTest.cpp:32-58)")


def test_f32_views_and_odd_leading_dimensions(ctx):
    k = _k()
    rng = np.random.default_rng(14)
    big = rng.standard_normal((500, 71)).astype(np.float32)
    a = big[:, 3:60]  # ld 71, offset 3: no 16-byte alignment
    b = rng.standard_normal((57, 29)).astype(np.float32)
    got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
    _check(got, np.ascontiguousarray(a), b, "strided lhs")
    A = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((4000, 64)).astype(np.float32))
    c = rng.standard_normal((50, 64)).astype(np.float32)
    got = k.matMul(A.slice_rows(1000, 3001), k.DenseMatrix.from_numpy(ctx, c), False, True).to_numpy()
    _check(got, A.to_numpy()[1000:3001], np.ascontiguousarray(c.T), "row view x t(C)")


@pytest.mark.parametrize("n,d", [(1000, 1), (5000, 7), (20000, 33), (100000, 100), (40000, 512), (300, 700)])
def test_f32_syrk(ctx, n, d):
    k = _k()
    x = np.random.default_rng(15).random((n, d)).astype(np.float32)
    X = k.DenseMatrix.from_numpy(ctx, x)
    s = k.syrk(X, True).to_numpy()
    _check(s, np.ascontiguousarray(x.T), x, f"syrk f32 {n}x{d}")
    assert_bits_equal(s, s.T.copy(), "syrk result is exactly symmetric")
    if n <= 5000:
        _check(k.syrk(X, False).to_numpy(), x, np.ascontiguousarray(x.T), f"syrk X t(X) f32 {n}x{d}")


def test_f32_non_finite_operands_propagate(ctx):
    k = _k()
    a = np.ones((4, 8), np.float32)
    b = np.ones((8, 4), np.float32)
    a[1, 2] = np.inf
    a[2, 3] = np.nan
    got = k.matMul(k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
    assert np.isinf(got[1]).all() and np.isnan(got[2]).all() and (got[0] == 8).all() and (got[3] == 8).all()


def test_f32_gemv(ctx):
    k = _k()
    rng = np.random.default_rng(16)
    for n, d in [(1000, 1), (20000, 33), (100000, 100)]:
        x = rng.random((n, d)).astype(np.float32)
        y = rng.standard_normal((n, 1)).astype(np.float32)
        got = k.gemv(k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y)).to_numpy()
        _check(got, np.ascontiguousarray(x.T), y, f"gemv f32 {n}x{d}")
