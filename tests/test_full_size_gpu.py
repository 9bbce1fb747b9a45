"""The five benchmark workloads at the sizes the benchmark configurations name, CUDA against the reference's CPU
kernels (oracle/_ref when it was built, else the C restatement).

Contract: integer, index and connected-components output bit-exact; f64 reductions within 1e-12 relative.  Where a
pipeline feeds a reduction (column mean / standard deviation, centroid) into an index result (idxMax, idxMin), the
1e-12 of the reduction can turn a near-tie between two columns the other way.  These tests do not budget such rows:
they collect every row whose index differs and assert, on the ORACLE's own values, that the two candidates are within
1e-10 relative of each other -- and they show separately that with identical statistics the index output is
bit-identical at full size."""
import numpy as np
import pytest
import scipy.sparse as sp

from tests.test_pipelines_gpu import _graph
from tests.util import assert_bits_equal

pytestmark = pytest.mark.gpu

EPS_REDUCE = 1e-12   # the contract for f64 reductions
NEAR_TIE = 1e-10     # two candidates of an index result count as tied below this relative distance


def _k():
    import daphne_b200.kernels as k
    from daphne_b200 import pipelines
    from oracle import cpu_pipelines as cpu
    return k, pipelines, cpu


def _uniform(rows, cols, lo, hi, seed, cpu):
    """DaphneDSL rand(rows, cols, lo, hi, 1, seed) through the reference's own RandMatrix kernel when it was built."""
    k, kind = cpu.backend()
    if kind == "reference":
        return k.rand(rows, cols, lo, hi, 1.0, seed)
    return lo + (hi - lo) * np.random.default_rng(seed).random((rows, cols))


def test_cfg2_standardise_aggregate_16777216x32(ctx):
    k, p, cpu = _k()
    n, c = 16_777_216, 32
    rng = np.random.default_rng(2)
    x = np.empty((n, c))
    for lo in range(0, n, 1 << 20):
        x[lo:lo + (1 << 20)] = 5.0 + 2.0 * rng.standard_normal((min(1 << 20, n - lo), c))
    threads = cpu.host_threads()
    res = p.standardise_aggregate(ctx, k.DenseMatrix.from_numpy(ctx, x))
    g_mu, g_sd = res.mu.to_numpy(), res.sd.to_numpy()
    g_r, g_m, g_i = res.r.to_numpy(), res.row_max.to_numpy(), res.row_idx_max.to_numpy()
    mu, sd, r, s, m, idx = cpu.standardise_aggregate(x, threads=threads)

    # (1) the reductions
    np.testing.assert_allclose(g_mu, mu, rtol=EPS_REDUCE)
    np.testing.assert_allclose(g_sd, sd, rtol=EPS_REDUCE)
    assert abs(res.s - s) <= 1e-11 * abs(s)          # sum over 16.7 M rows of values that carry (2) below
    assert abs(res.s - x.size) <= 1e-9 * x.size      # the sum of squared z-scores is rows * cols

    # (2) what a relative error e in mu and sd does to one entry of Z = (x - mu) / sd:
    #     |dZ| <= e |mu| / sd + e |Z|  (first order) <= e (max|mu/sd| + |Z|), plus one rounding of the division;
    #     a row maximum moves by at most that; r = sum(Z^2) moves by at most sum(2 |Z| |dZ|) <= 2 e (b sum|Z| + r),
    #     and the 32-term sums add 32 roundings.  e is the 1e-12 of (1).
    b = float(np.max(np.abs(mu / sd)))
    e = EPS_REDUCE + 4 * np.finfo(np.float64).eps
    assert np.all(np.abs(g_m - m) <= e * (b + np.abs(m)))
    # sum|Z| <= sqrt(c * r) (Cauchy-Schwarz), so the bound needs no second pass over Z
    assert np.all(np.abs(g_r - r) <= 2 * e * (b * np.sqrt(c * r) + r) + 40 * np.finfo(np.float64).eps * r)

    # (3) every row whose idxMax differs is a near-tie in the oracle's own Z
    bad = np.flatnonzero(g_i[:, 0] != idx[:, 0])
    print(f"cfg2 16777216x32: {bad.size} rows with a different idxMax (statistics differ in the last bits)")
    if bad.size:
        zb = (x[bad] - mu) / sd
        za = zb[np.arange(bad.size), idx[bad, 0].astype(np.int64)]
        zg = zb[np.arange(bad.size), g_i[bad, 0].astype(np.int64)]
        assert np.all(np.abs(za - zg) <= NEAR_TIE * np.abs(za)), "an idxMax mismatch that is not a near-tie"

    # (4) with IDENTICAL statistics (the device's) the row results are bit-identical: maxima and positions always, the
    #     row sums against the sequential sum of the exactly rounded squares (glibc's pow(z, 2) is within 1 ulp of it)
    r2, m2, i2 = cpu.standardise_tail(x, g_mu, g_sd, threads=threads, exact_squares=True)
    assert_bits_equal(g_m, m2, "rowMaxs(Z) with the device's statistics")
    assert_bits_equal(g_i, i2, "idxMax(Z) with the device's statistics")
    assert_bits_equal(g_r, r2, "rowSums(Z^2) with the device's statistics")


def test_cfg3_kmeans_1000000x64_k50_10_iterations(ctx):
    k, p, cpu = _k()
    n, d, kk, iters = 1_000_000, 64, 50, 10
    x = _uniform(n, d, 0.0, 1.0, 3, cpu)
    c0 = x[np.random.default_rng(33).choice(n, kk, replace=False)].copy()
    X = k.DenseMatrix.from_numpy(ctx, x)
    xs = (x * x).sum(axis=1, keepdims=True)
    full = p.kmeans(ctx, X, k.DenseMatrix.from_numpy(ctx, c0), iters)
    # lock step: every iteration starts from the ORACLE's centroids on both sides, so an iteration is compared on
    # identical inputs; the oracle's sequence C_0 .. C_10 is its 10-iteration run
    C, flips_total = c0, 0
    for it in range(iters):
        C_cpu, a_cpu = cpu.kmeans(x, C, 1)
        one = p.kmeans(ctx, X, k.DenseMatrix.from_numpy(ctx, np.ascontiguousarray(C)), 1)
        a_gpu, C_gpu = one.assign.to_numpy(), one.C.to_numpy()
        bad = np.flatnonzero(a_gpu[:, 0] != a_cpu[:, 0])
        flips_total += bad.size
        if bad.size:  # near-ties in the oracle's distances  D = -2 x.c + |x|^2 + |c|^2
            cs = (C * C).sum(axis=1)
            D = -2.0 * (x[bad] @ C.T) + xs[bad] + cs[None, :]
            da = D[np.arange(bad.size), a_cpu[bad, 0]]
            dg = D[np.arange(bad.size), a_gpu[bad, 0]]
            assert np.all(np.abs(da - dg) <= NEAR_TIE * np.abs(da)), f"iteration {it}: a flip that is not a near-tie"
            # a flipped point moves two centroids by x / count: bound the centroid difference by that
            counts = np.bincount(a_cpu[:, 0], minlength=kk).astype(np.float64)
            tol = (bad.size + 1) / counts.min() + EPS_REDUCE
            assert np.abs(C_gpu - C_cpu).max() <= tol
        else:
            assert np.abs(C_gpu - C_cpu).max() <= EPS_REDUCE * np.abs(C_cpu).max()
        C = C_cpu
    print(f"cfg3 1000000x64 k=50: {flips_total} assignment flips over {iters} lock-step iterations (all near-ties)")
    # the device's own 10-iteration run: identical when nothing flipped, else within what the flips explain
    got_c, got_a = full.C.to_numpy(), full.assign.to_numpy()
    if flips_total == 0 and np.array_equal(got_a[:, 0], a_cpu[:, 0]):
        assert np.abs(got_c - C).max() <= 1e-11 * np.abs(C).max()
    else:
        assert (got_a[:, 0] != a_cpu[:, 0]).mean() < 1e-3
        assert np.abs(got_c - C).max() <= 1e-4


def test_cfg4_connected_components_1000000_vertices(ctx):
    k, p, cpu = _k()
    n = 1_000_000
    g = _graph(n, 8, 4)
    assert g.nnz == 8_000_000
    res = p.connected_components(ctx, k.CSRMatrix.from_scipy(ctx, g))
    c, iters = cpu.connected_components(g)
    assert res.iterations == iters
    got = res.c.to_numpy()
    assert_bits_equal(got, c, "component labels, 1 M vertices")
    ncomp, labels = sp.csgraph.connected_components(g, directed=False)
    assert len(np.unique(got)) == ncomp
    # every vertex carries the largest (1-based) vertex id of its component
    top = np.zeros(ncomp)
    np.maximum.at(top, labels, np.arange(1, n + 1, dtype=np.float64))
    assert np.array_equal(got[:, 0], top[labels])


def test_cfg1_normal_equations_100000x100_rand_matrix(ctx):
    k, p, cpu = _k()
    n, d = 100_000, 100
    x = _uniform(n, d, 0.0, 1.0, 42, cpu)
    w = np.random.default_rng(43).standard_normal((d, 1))
    y = x @ w + 0.01 * np.random.default_rng(44).standard_normal((n, 1))
    res = p.normal_equations(ctx, k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y), 0.001)
    A, b, beta = cpu.normal_equations(x, y, 0.001)
    got_a, got_b, got_beta = res.A.to_numpy(), res.b.to_numpy(), res.beta.to_numpy()
    assert np.abs(got_a - A).max() <= EPS_REDUCE * np.abs(A).max()
    assert np.abs(got_b - b).max() <= EPS_REDUCE * np.abs(b).max()
    assert np.array_equal(got_a, got_a.T)
    # the solution inherits cond(A) ~ 1e4 .. 1e5 times the 1e-12 of A and b; the residual does not
    assert np.abs(got_beta - beta).max() <= 1e-7 * np.abs(beta).max()
    assert np.abs(A @ got_beta - b).max() <= 1e-11 * np.abs(b).max()
    assert np.abs(got_beta - w).max() < 0.01


@pytest.mark.parametrize("n", [131_072, 1_048_576])
def test_cfg5_normal_equations_shard_x512(ctx, n):
    """131 072 x 512 is 1/64 of the configuration; 1 048 576 x 512 (4 GiB) is the row shard one of eight GPUs holds."""
    k, p, cpu = _k()
    d = 512
    rng = np.random.default_rng(5)
    x = np.empty((n, d))
    for lo in range(0, n, 1 << 16):
        x[lo:lo + (1 << 16)] = 2.0 * rng.random((min(1 << 16, n - lo), d)) - 1.0
    w = np.random.default_rng(55).standard_normal((d, 1))
    y = x @ w + 0.01 * np.random.default_rng(56).standard_normal((n, 1))
    res = p.normal_equations(ctx, k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y), 0.001)
    ref, kind = cpu.backend()
    if kind == "reference":
        ref.set_blas_threads(cpu.host_threads())
    A, b, beta = cpu.normal_equations(x, y, 0.001)
    got_a, got_b, got_beta = res.A.to_numpy(), res.b.to_numpy(), res.beta.to_numpy()
    assert np.abs(got_a - A).max() <= EPS_REDUCE * np.abs(A).max()
    assert np.abs(got_b - b).max() <= EPS_REDUCE * np.abs(b).max()
    assert np.array_equal(got_a, got_a.T)
    assert np.abs(got_beta - beta).max() <= 1e-9 * np.abs(beta).max()   # cond(A) ~ 1 for uniform[-1, 1) columns
    assert np.abs(A @ got_beta - b).max() <= 1e-11 * np.abs(b).max()
    assert np.abs(got_beta - w).max() < 0.01
