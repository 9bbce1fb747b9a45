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


def test_chains_on_a_csr_row_aggregation_are_evaluated_in_its_pass(ctx):
    """A row aggregation of a large CSR matrix is deferred; elementwise operators on its rows x 1 result, the sum of
    the chain and live intermediate results come out of ONE pass over the CSR arrays (what connected components
    needs: u = max(aggMax(G * t(c), 0), c); diff = sum(u != c)).  Checked against the operator-by-operator oracle."""
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    B, A = k.BinaryOpCode, k.AggOpCode
    n = 150000
    g = _graph(n, 6, 11)
    rng = np.random.default_rng(12)
    c = rng.integers(1, n, size=(n, 1)).astype(np.float64)
    G, Cv = k.CSRMatrix.from_scipy(ctx, g), k.DenseMatrix.from_numpy(ctx, c)
    exp_mx = o.aggRowCsr(A.MAX, o.ewMulCsrDense(g, c.T.copy()))
    exp_u = np.maximum(exp_mx, c)
    exp_diff = float((exp_u != c).sum())
    # (1) the connected-components step: one kernel launch for four operator calls
    l0 = ctx.stats()["launches"]
    mx = k.aggRowCsr(A.MAX, k.ewMulCsrDense(G, k.transpose(Cv)))
    u = k.ewBinaryMat(B.MAX, mx, Cv)
    diff = k.aggAll(A.SUM, k.ewBinaryMat(B.NEQ, u, Cv))
    launches = ctx.stats()["launches"] - l0
    assert diff == exp_diff
    assert_bits_equal(u.to_numpy(), exp_u, "u = max(rowMaxs(G * t(c)), c)")
    assert launches <= 2, f"expected the fused pass (plus at most the upload helper), got {launches} launches"
    assert_bits_equal(mx.to_numpy(), exp_mx, "the aggregation itself, asked for afterwards")
    # (2) other aggregations, scalar / unary steps, reversed operands, the chain materialised without a sum
    w = rng.standard_normal((n, 1))
    W = k.DenseMatrix.from_numpy(ctx, w)
    gv = g.copy()
    gv.data[:] = rng.standard_normal(gv.nnz)
    GV = k.CSRMatrix.from_scipy(ctx, gv)
    for op in (A.SUM, A.MIN, A.MAX):
        base = o.aggRowCsr(op, gv)
        r = k.aggRowCsr(op, GV)
        z = k.ewBinaryMat(B.SUB, W, k.ewBinaryObjSca(B.MUL, r, 2.0))          # w - 2 r  (reversed operand)
        z = k.ewUnaryMat(k.UnaryOpCode.ABS, z)
        exp = np.abs(w - base * 2.0)
        if op == A.SUM:
            np.testing.assert_allclose(z.to_numpy(), exp, rtol=1e-12, atol=1e-12)
        else:
            assert_bits_equal(z.to_numpy(), exp, f"chain on csr agg {op}")
        s = k.aggCol(A.SUM, k.ewBinaryMat(B.GT, k.aggRowCsr(op, GV), W))           # the sum stays on the device
        assert float(s.to_numpy()[0, 0]) == float((base > w).sum())


def test_native_call_sequences_equal_the_python_ones(ctx):
    """db2w_* issue the same operator calls from C++ (what a JIT-compiled caller does): identical results."""
    k, p, cpu = _k()
    g = _graph(120000, 6, 21)
    G = k.CSRMatrix.from_scipy(ctx, g)
    a, b = p.connected_components(ctx, G), p.connected_components_native(ctx, G)
    assert a.iterations == b.iterations
    assert_bits_equal(a.c.to_numpy(), b.c.to_numpy(), "components")
    for maxi in (0, 1, 3):  # the loop's other exit: the trip limit
        a, b = p.connected_components(ctx, G, maxi=maxi), p.connected_components_native(ctx, G, maxi=maxi)
        assert a.iterations == b.iterations == maxi
        assert_bits_equal(a.c.to_numpy(), b.c.to_numpy(), f"components, at most {maxi} trips")
    xs = 5.0 + 2.0 * np.random.default_rng(4).standard_normal((300000, 32))
    Xs = k.DenseMatrix.from_numpy(ctx, xs)
    sa, sb = p.standardise_aggregate(ctx, Xs), p.standardise_aggregate_native(ctx, Xs)
    for u, v in ((sa.mu, sb.mu), (sa.sd, sb.sd), (sa.r, sb.r), (sa.row_max, sb.row_max), (sa.row_idx_max, sb.row_idx_max)):
        assert_bits_equal(u.to_numpy(), v.to_numpy(), "standardise")
    assert abs(sa.s - sb.s) <= 1e-12 * abs(sa.s)          # one is a full aggregation, the other a column sum of r
    x = np.random.default_rng(3).random((150000, 64))
    c0 = x[:50].copy()
    X, C0 = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, c0)
    ka, kb = p.kmeans(ctx, X, C0, 3), p.kmeans_native(ctx, X, C0, 3)
    assert_bits_equal(ka.C.to_numpy(), kb.C.to_numpy(), "centroids")
    assert_bits_equal(ka.assign.to_numpy(), kb.assign.to_numpy(), "assignments")
    y = x @ np.arange(64.0).reshape(-1, 1)
    Y = k.DenseMatrix.from_numpy(ctx, y)
    na, nb = p.normal_equations(ctx, X, Y, 0.001), p.normal_equations_native(ctx, X, Y, 0.001)
    for u, v in ((na.A, nb.A), (na.b, nb.b), (na.beta, nb.beta)):
        assert_bits_equal(u.to_numpy(), v.to_numpy(), "normal equations")


def test_agg_all_in_two_halves(ctx):
    """db2_aggAllStart / db2_scalarStart / db2_scalarWait: the value of the one-call form, two values outstanding."""
    k, p, cpu = _k()
    A, B = k.AggOpCode, k.BinaryOpCode
    rng = np.random.default_rng(8)
    x = rng.standard_normal((70000, 3))
    X = k.DenseMatrix.from_numpy(ctx, x)
    g = _graph(90000, 5, 9)
    G = k.CSRMatrix.from_scipy(ctx, g)
    w = rng.random((90000, 1)) * 90000
    W = k.DenseMatrix.from_numpy(ctx, w)
    ne = k.ewBinaryMat(B.GT, k.aggRowCsr(A.MAX, k.ewMulCsrDense(G, k.transpose(W))), W)   # deferred CSR chain
    expect_csr = k.aggAll(A.SUM, k.ewBinaryMat(B.GT, k.aggRowCsr(A.MAX, k.ewMulCsrDense(G, k.transpose(W))), W))
    k.aggAllStart(A.SUM, ne, 1)
    k.aggAllStart(A.MAX, X, 0)                      # any other argument: same value, already there
    one = k.aggCol(A.SUM, k.aggRow(A.SUM, k.ewBinaryObjSca(B.MUL, X, 2.0)))
    assert k.aggAllWait(ctx, 0) == x.max()
    assert k.aggAllWait(ctx, 1) == expect_csr
    k.scalarStart(one, 0)
    assert k.aggAllWait(ctx, 0) == float(one.to_numpy()[0, 0])
    with pytest.raises(Exception):
        k.aggAllStart(A.SUM, X, 2)


def test_results_copied_to_the_host_beside_the_next_run(ctx):
    """db2_matrix_to_host_async: the copy runs on the context's second stream; the matrix may be released and the next
    run queued before db2_context_side_sync, and the bytes are those of the synchronous copy."""
    import ctypes as C
    from daphne_b200.lib import lib, check
    k, p, cpu = _k()
    rng = np.random.default_rng(91)
    dsts, refs = [], []
    for i in range(4):
        x = rng.standard_normal((200000, 32)) * (i + 1)
        X = k.DenseMatrix.from_numpy(ctx, x)
        z = k.ewBinaryObjSca(k.BinaryOpCode.MUL, X, 1.5)       # a deferred chain: forced by the copy
        r = k.aggRow(k.AggOpCode.SUM, z)
        dz, dr = np.empty((200000, 40)), np.empty((200000, 1))   # a destination with a larger leading dimension
        check(lib.db2_matrix_to_host_async(z.handle, C.c_void_p(dz.ctypes.data), 40))
        check(lib.db2_matrix_to_host_async(r.handle, C.c_void_p(dr.ctypes.data), 1))
        dsts.append((dz, dr))
        refs.append((z.to_numpy(), r.to_numpy()))
        del z, r, X                                               # released while the copies may still be running
    check(lib.db2_context_side_sync(ctx.handle))
    for (dz, dr), (z, r) in zip(dsts, refs):
        assert_bits_equal(dz[:, :32], z, "values copied on the second stream")
        assert_bits_equal(dr, r, "row sums copied on the second stream")
