"""The five benchmark workloads at sizes the CPU oracle finishes in seconds, CUDA against oracle, plus the
size-independent properties that are checked at full size by the benchmark (checksums, idempotence, fixed points)."""
import numpy as np
import pytest
import scipy.sparse as sp

from tests.util import assert_bits_equal

pytestmark = pytest.mark.gpu


def _k():
    import daphne_b200.kernels as k
    from daphne_b200 import pipelines
    from oracle import cpu_pipelines as cpu
    return k, pipelines, cpu


def _graph(n, deg, seed):
    """Symmetric 0/1 adjacency matrix: n * deg / 2 distinct undirected edges, no self loops."""
    rng = np.random.default_rng(seed)
    m = n * deg // 2
    i = rng.integers(0, n, size=3 * m)
    j = rng.integers(0, n, size=3 * m)
    keep = i != j
    lo, hi = np.minimum(i[keep], j[keep]), np.maximum(i[keep], j[keep])
    edges = np.unique(np.stack([lo, hi], axis=1), axis=0)[:m]
    rows = np.concatenate([edges[:, 0], edges[:, 1]])
    cols = np.concatenate([edges[:, 1], edges[:, 0]])
    g = sp.csr_matrix((np.ones(rows.size), (rows, cols)), shape=(n, n))
    g.sort_indices()
    return g


def test_cfg1_linear_regression_normal_equations(ctx):
    k, p, cpu = _k()
    rng = np.random.default_rng(42)
    n, d = 100000, 100
    x = rng.random((n, d))
    w = np.random.default_rng(43).standard_normal((d, 1))
    y = x @ w + 0.01 * np.random.default_rng(44).standard_normal((n, 1))
    res = p.normal_equations(ctx, k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, y), 0.001)
    A, b, beta = cpu.normal_equations(x, y, 0.001)
    got_a, got_b, got_beta = res.A.to_numpy(), res.b.to_numpy(), res.beta.to_numpy()
    assert np.abs(got_a - A).max() <= 1e-12 * np.abs(A).max()
    assert np.abs(got_b - b).max() <= 1e-12 * np.abs(b).max()
    assert np.abs(got_beta - beta).max() <= 1e-8 * np.abs(beta).max()  # cond(A) ~ 1e4
    assert np.abs(A @ got_beta - b).max() <= 1e-12 * np.abs(b).max()    # backward error of the solve
    assert np.abs(got_beta - w).max() < 0.01


def test_cfg2_standardise_and_aggregate(ctx):
    k, p, cpu = _k()
    x = 5.0 + 2.0 * np.random.default_rng(2).standard_normal((300000, 32))
    res = p.standardise_aggregate(ctx, k.DenseMatrix.from_numpy(ctx, x))
    mu, sd, r, s, m, idx = cpu.standardise_aggregate(x, threads=8)
    np.testing.assert_allclose(res.mu.to_numpy(), mu, rtol=1e-12)
    np.testing.assert_allclose(res.sd.to_numpy(), sd, rtol=1e-12)
    # Z inherits the 1e-12 of mu/sd relative to |x - mu|, so entries of Z near 0 are compared absolutely
    np.testing.assert_allclose(res.r.to_numpy(), r, rtol=1e-9)
    np.testing.assert_allclose(res.row_max.to_numpy(), m, rtol=1e-9, atol=1e-9)
    assert (res.row_idx_max.to_numpy() != idx).mean() < 1e-5  # only exact ties between two columns could differ
    assert abs(res.s - s) <= 1e-10 * abs(s)
    assert abs(res.s - x.size) <= 1e-9 * x.size  # sum of squared z-scores is rows * cols


def test_cfg3_kmeans(ctx):
    k, p, cpu = _k()
    n, d, kk = 200000, 64, 50
    x = np.random.default_rng(3).random((n, d))
    c0 = x[np.random.default_rng(33).choice(n, kk, replace=False)].copy()
    res = p.kmeans(ctx, k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, c0), 10)
    C, a = cpu.kmeans(x, c0, 10)
    got_c, got_a = res.C.to_numpy(), res.assign.to_numpy()
    # assignments: points whose two nearest centroids are at (nearly) equal distance may flip with the summation order
    assert (got_a != a).mean() < 1e-4
    assert np.abs(got_c - C).max() <= 1e-6
    # a single iteration from identical centroids is tighter: centroid sums are sums of the same points
    r1 = p.kmeans(ctx, k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, c0), 1)
    C1, a1 = cpu.kmeans(x, c0, 1)
    same = r1.assign.to_numpy() == a1
    assert same.mean() > 1 - 1e-5
    if same.all():
        assert np.abs(r1.C.to_numpy() - C1).max() <= 1e-12


def test_cfg4_connected_components_bit_exact(ctx):
    k, p, cpu = _k()
    for n, deg, seed in [(2000, 2, 1), (50000, 8, 4), (100000, 3, 5)]:
        g = _graph(n, deg, seed)
        res = p.connected_components(ctx, k.CSRMatrix.from_scipy(ctx, g))
        c, iters = cpu.connected_components(g)
        assert res.iterations == iters
        assert_bits_equal(res.c.to_numpy(), c, f"components n={n}")
        ncomp, labels = sp.csgraph.connected_components(g, directed=False)
        assert len(np.unique(c)) == ncomp
        # fixed point: every vertex carries the largest vertex id (1-based) of its component
        for comp in range(min(ncomp, 50)):
            members = np.where(labels == comp)[0]
            assert np.all(c[members, 0] == members.max() + 1)


def test_csr_row_aggregation_with_hub_rows(ctx):
    """Rows far longer than the others (hubs of a power-law graph) are finished by whole thread blocks at the end of the
    kernel; more hubs than a block's list holds fall back to the ordinary path.  Values, implicit zeros and views."""
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    rng = np.random.default_rng(5)
    n, m = 20000, 60000
    rr, cc = [rng.integers(0, n, size=240000)], [rng.integers(0, m, size=240000)]  # the ordinary short rows
    hubs = list(range(0, 3000, 75)) + [n - 1]
    for h in hubs:
        cols = rng.choice(m, size=int(rng.integers(2000, 9000)), replace=False)
        rr.append(np.full(cols.size, h))
        cc.append(cols)
    rr.append(np.full(m, 7))                            # a full row: no implicit zero takes part
    cc.append(np.arange(m))
    rr, cc = np.concatenate(rr), np.concatenate(cc)
    g = sp.csr_matrix((np.ones(rr.size), (rr, cc)), shape=(n, m))
    g.sum_duplicates()
    g.data[:] = rng.standard_normal(g.nnz)
    g.sort_indices()
    G = k.CSRMatrix.from_scipy(ctx, g)
    rv = rng.standard_normal((1, m))
    rv[0, ::9] = 0
    prod = k.ewMulCsrDense(G, k.DenseMatrix.from_numpy(ctx, rv))
    exp = o.ewMulCsrDense(g, rv)
    for op in (0, 2, 3):
        got, e = k.aggRowCsr(op, prod).to_numpy(), o.aggRowCsr(op, exp)
        if op == 0:
            np.testing.assert_allclose(got, e, rtol=1e-11, atol=1e-300)
        else:
            assert_bits_equal(got, e, f"hub rows agg {op}")
    for op in (2, 3):
        assert_bits_equal(k.aggRowCsr(op, G).to_numpy(), o.aggRowCsr(op, g), f"plain hub rows agg {op}")
    v = G.slice_rows(5, 2500)
    assert_bits_equal(k.aggRowCsr(3, v).to_numpy(), o.aggRowCsr(3, g)[5:2500], "view with hubs")
    # adjacency matrix (every value 1.0: the value array is not read)
    a = g.copy()
    a.data[:] = 1.0
    A_ = k.CSRMatrix.from_scipy(ctx, a)
    c = rng.integers(1, 1000, size=(1, m)).astype(np.float64)
    got = k.aggRowCsr(3, k.ewMulCsrDense(A_, k.DenseMatrix.from_numpy(ctx, c))).to_numpy()
    assert_bits_equal(got, o.aggRowCsr(3, o.ewMulCsrDense(a, c)), "unit values with hubs")
    # every row long, few blocks: more long rows than a block's list holds (the rest is processed in place)
    d = sp.random(300, 5000, 0.15, format="csr", random_state=3)
    d.data[:] = rng.standard_normal(d.nnz)
    d.sort_indices()
    D = k.CSRMatrix.from_scipy(ctx, d)
    for op in (2, 3):
        assert_bits_equal(k.aggRowCsr(op, D).to_numpy(), o.aggRowCsr(op, d), f"all rows long, agg {op}")
    np.testing.assert_allclose(k.aggRowCsr(0, D).to_numpy(), o.aggRowCsr(0, d), rtol=1e-11, atol=1e-11)  # sums near 0


def test_csr_kernels_against_oracle(ctx):
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    rng = np.random.default_rng(0)
    g = sp.random(3000, 2500, 0.004, format="csr", random_state=1)
    g.data[:] = rng.standard_normal(g.nnz)
    g.sort_indices()
    G = k.CSRMatrix.from_scipy(ctx, g)
    rv = rng.standard_normal((1, 2500))
    rv[0, ::7] = 0
    cv = rng.standard_normal((3000, 1))
    cv[::5] = 0
    full = rng.standard_normal((3000, 2500))
    full[::3] = 0
    for rhs in (rv, cv, full):
        R = k.DenseMatrix.from_numpy(ctx, rhs)
        prod = k.ewMulCsrDense(G, R)
        exp = o.ewMulCsrDense(g, rhs)
        for op in (0, 2, 3):  # SUM (order differs: tolerance), MIN, MAX (exact)
            got, e = k.aggRowCsr(op, prod).to_numpy(), o.aggRowCsr(op, exp)
            if op == 0:
                np.testing.assert_allclose(got, e, rtol=1e-12, atol=1e-300)
            else:
                assert_bits_equal(got, e, f"csr agg {op}")
        vals, cols, offs = prod.to_arrays()
        assert_bits_equal(vals, exp[0], "product values")
        assert_bits_equal(cols, exp[1], "product column indices")
        assert_bits_equal(offs, exp[2], "product row offsets")
        # aggregation of the materialised product and of a row view of it
        assert_bits_equal(k.aggRowCsr(3, prod).to_numpy(), o.aggRowCsr(3, exp), "materialised")
        v = prod.slice_rows(100, 1700)
        assert_bits_equal(k.aggRowCsr(3, v).to_numpy(), o.aggRowCsr(3, exp)[100:1700], "view")
    dense = rng.standard_normal((2500, 3))
    assert_bits_equal(k.matMulCsrDense(G, k.DenseMatrix.from_numpy(ctx, dense)).to_numpy(),
                      o.matMulCsrDense(g, dense), "csr @ dense")
    # empty rows, empty matrix
    e = sp.csr_matrix((5, 7))
    E = k.CSRMatrix.from_scipy(ctx, e)
    assert_bits_equal(k.aggRowCsr(3, E).to_numpy(), o.aggRowCsr(3, e), "all-empty rows max = implicit zero")
    assert_bits_equal(k.aggRowCsr(0, E).to_numpy(), o.aggRowCsr(0, e), "all-empty rows sum")
