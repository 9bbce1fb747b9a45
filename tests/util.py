"""Shared helpers of the parity tests."""
import numpy as np

# Tolerance contract.  Elementwise +,-,*,/,min,max, comparisons, sqrt, rounding: bit-exact.  f64 reductions: 1e-12
# relative (the summation order differs from the sequential CPU loops).  pow/log/exp/trig: a few ulp (CUDA's libm
# documents up to 2 ulp for double pow; glibc is below 1 ulp).
RTOL_REDUCE_F64 = 1e-12
RTOL_REDUCE_F32 = 1e-5
RTOL_TRANSCENDENTAL_F64 = 1e-15 * 8
RTOL_TRANSCENDENTAL_F32 = 1e-6


def assert_bits_equal(a: np.ndarray, b: np.ndarray, what=""):
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    assert a.dtype == b.dtype, f"{what}: dtype {a.dtype} vs {b.dtype}"
    av = a.view(np.uint8).reshape(-1) if a.size else a
    bv = b.view(np.uint8).reshape(-1) if b.size else b
    if not np.array_equal(av, bv):
        bad = np.argwhere(~((a == b) | ((a != a) & (b != b))))
        # distinguish NaN-payload / signed-zero differences from value differences
        raise AssertionError(f"{what}: bit mismatch; first value mismatches at {bad[:5].tolist()} "
                             f"a={a[tuple(bad[0])] if len(bad) else 'bits only'} "
                             f"b={b[tuple(bad[0])] if len(bad) else 'bits only'}")


def assert_close_rel(a: np.ndarray, b: np.ndarray, rtol: float, what="", scale=None):
    """|a-b| <= rtol * max(|b|, scale) elementwise; NaNs must coincide."""
    assert a.shape == b.shape, f"{what}: shape {a.shape} vs {b.shape}"
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    nan_a, nan_b = np.isnan(a), np.isnan(b)
    assert np.array_equal(nan_a, nan_b), f"{what}: NaN pattern differs"
    inf = np.isinf(b)
    assert np.array_equal(a[inf], b[inf]), f"{what}: infinities differ"
    ok = ~(nan_b | inf)
    ref = np.abs(b[ok])
    if scale is not None:
        ref = np.maximum(ref, scale)
    err = np.abs(a[ok] - b[ok])
    bad = err > rtol * ref
    assert not bad.any(), f"{what}: max rel err {np.max(err / np.maximum(ref, 1e-300)):.3e} > {rtol:g}"


def rng_matrix(seed, rows, cols, dtype=np.float64, kind="normal"):
    rng = np.random.default_rng(seed)
    if np.dtype(dtype) == np.int64:
        return rng.integers(-1000, 1000, size=(rows, cols), dtype=np.int64)
    if kind == "normal":
        return (5.0 + 2.0 * rng.standard_normal((rows, cols))).astype(dtype)
    return rng.random((rows, cols)).astype(dtype)
