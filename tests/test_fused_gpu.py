"""Deferred elementwise chains and fused consumers (row pass, column pass, materialisation) against the CPU oracle.

Every case is also run with fusion disabled (a context created under DB2_EAGER=1 runs one kernel per operator call),
and the two device results have to agree bit for bit where the arithmetic is order-independent."""
import os

import numpy as np
import pytest

from tests.util import RTOL_REDUCE_F64, assert_bits_equal, assert_close_rel, rng_matrix

pytestmark = pytest.mark.gpu

SHAPES = [(70000, 32), (4099, 50), (3000, 33), (2049, 128), (1500, 1000), (66000, 7), (300, 400), (70001, 34),
          (40000, 6), (50000, 2), (3001, 70), (2500, 62)]


def _k():
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    return k, o


@pytest.fixture(scope="module")
def eager_ctx():
    import daphne_b200.kernels as k
    os.environ["DB2_EAGER"] = "1"
    try:
        c = k.Context(0)
    finally:
        del os.environ["DB2_EAGER"]
    yield c
    c.close()


def _standardise(k, M, mu, sd):
    B = k.BinaryOpCode
    return k.ewBinaryMat(B.DIV, k.ewBinaryMat(B.SUB, M, mu), sd)


@pytest.mark.parametrize("shape", SHAPES)
def test_standardise_chain_with_three_row_aggregations_in_one_pass(ctx, eager_ctx, shape):
    k, o = _k()
    B, A = k.BinaryOpCode, k.AggOpCode
    r, c = shape
    x = rng_matrix(1, r, c)
    mu = x.mean(axis=0, keepdims=True)
    sd = x.std(axis=0, keepdims=True)
    z_cpu = o.ewBinaryMat(B.DIV, o.ewBinaryMat(B.SUB, x, mu), sd)
    exp_r = o.aggRow(A.SUM, o.ewBinaryObjSca(B.POW, z_cpu, 2.0))
    # the device squares exactly; libm's pow(x, 2) may differ from x*x by one ulp, so the expected row sums are
    # recomputed from the exact squares for the bit comparison
    exp_r_exact = o.aggRow(A.SUM, z_cpu * z_cpu)
    exp_m, exp_i = o.aggRow(A.MAX, z_cpu), o.aggRow(A.IDXMAX, z_cpu)
    results = {}
    for name, cx in (("fused", ctx), ("eager", eager_ctx)):
        X = k.DenseMatrix.from_numpy(cx, x)
        MU, SD = k.DenseMatrix.from_numpy(cx, mu), k.DenseMatrix.from_numpy(cx, sd)
        launches0 = cx.stats()["launches"]
        Z = _standardise(k, X, MU, SD)
        R = k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, Z, 2.0))
        M = k.aggRow(A.MAX, Z)
        I = k.aggRow(A.IDXMAX, Z)
        got = (R.to_numpy(), M.to_numpy(), I.to_numpy(), Z.to_numpy())
        results[name] = got
        launches = cx.stats()["launches"] - launches0
        if name == "fused" and r * c >= 65536:
            assert launches == 2, f"expected one fused pass for the aggregations + one for Z, got {launches}"
        assert_bits_equal(got[3], z_cpu, f"{name} Z")
        assert_bits_equal(got[1], exp_m, f"{name} rowMax")
        assert_bits_equal(got[2], exp_i, f"{name} idxMax")
        assert_close_rel(got[0], exp_r, RTOL_REDUCE_F64, f"{name} rowSums")
    # the fused row pass adds left to right like the reference's loop: bit-identical row sums
    assert_bits_equal(results["fused"][0], exp_r_exact, "fused rowSums are the sequential sums")


@pytest.mark.parametrize("shape", SHAPES[:5])
def test_column_pass_over_a_chain(ctx, shape):
    k, o = _k()
    B, A = k.BinaryOpCode, k.AggOpCode
    r, c = shape
    x = rng_matrix(2, r, c)
    mu = x.mean(axis=0, keepdims=True)
    X, MU = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, mu)
    d = o.ewBinaryMat(B.SUB, x, mu)
    d2 = d * d
    D2 = k.ewBinaryObjSca(B.POW, k.ewBinaryMat(B.SUB, X, MU), 2.0)
    for name in ("SUM", "MEAN", "MIN", "MAX", "IDXMIN", "IDXMAX"):
        got, exp = k.aggCol(A[name], D2).to_numpy(), o.aggCol(A[name], d2)
        if name in ("SUM", "MEAN"):
            assert_close_rel(got, exp, RTOL_REDUCE_F64, f"col {name} {shape}")
        else:
            assert_bits_equal(got, exp, f"col {name} {shape}")
    # VAR/STDDEV of a chain: the chain is materialised and the two-pass kernels run
    assert_close_rel(k.aggCol(A.VAR, D2).to_numpy(), o.aggCol(A.VAR, d2), 10 * RTOL_REDUCE_F64, "col VAR")
    assert_close_rel(np.array([k.aggAll(A.SUM, D2)]), np.array([o.aggAll(A.SUM, d2)]), RTOL_REDUCE_F64, "all SUM")


def test_every_fusable_step_kind_and_operand_kind(ctx, eager_ctx):
    k, o = _k()
    B, U, A = k.BinaryOpCode, k.UnaryOpCode, k.AggOpCode
    r, c = 3001, 45
    x, y = rng_matrix(3, r, c) - 5.0, rng_matrix(4, r, c) - 5.0
    rv, cv = rng_matrix(5, 1, c) - 4.0, rng_matrix(6, r, 1) - 4.0
    y[::7] = x[::7]

    def run(kk, mk):
        X, Y, RV, CV = mk(x), mk(y), mk(rv), mk(cv)
        t = kk.ewBinaryMat(B.ADD, X, Y)             # matrix operand
        t = kk.ewBinaryMat(B.MUL, t, RV)            # row vector
        t = kk.ewBinaryMat(B.SUB, t, CV)            # column vector
        t = kk.ewBinaryObjSca(B.DIV, t, 3.7)        # scalar
        t = kk.ewUnaryMat(U.ABS, t)
        t = kk.ewBinaryMat(B.MAX, t, Y)
        t = kk.ewBinaryMat(B.DIV, t, RV)
        t = kk.ewUnaryMat(U.MINUS, t)
        t = kk.ewBinaryMat(B.MIN, t, CV)
        u = kk.ewBinaryMat(B.LE, t, X)
        v = kk.ewUnaryMat(U.FLOOR, kk.ewBinaryObjSca(B.MUL, t, 0.37))
        w = kk.ewBinaryMat(B.SUB, Y, t)             # deferred operand on the right: reversed step
        w = kk.ewBinaryMat(B.DIV, X, w)             # reversed division
        return t, u, v, w

    cpu = run(type("O", (), {"ewBinaryMat": staticmethod(o.ewBinaryMat), "ewBinaryObjSca": staticmethod(o.ewBinaryObjSca),
                             "ewUnaryMat": staticmethod(o.ewUnaryMat)}), lambda a: a)
    for name, cx in (("fused", ctx), ("eager", eager_ctx)):
        dev = run(k, lambda a: k.DenseMatrix.from_numpy(cx, a))
        for i, (g, e) in enumerate(zip(dev, cpu)):
            assert_bits_equal(g.to_numpy(), e, f"{name} result {i}")
        for g, e in zip(dev, cpu):
            assert_bits_equal(k.aggRow(A.MIN, g).to_numpy(), o.aggRow(A.MIN, e), f"{name} rowMin")
            assert_bits_equal(k.aggRow(A.IDXMIN, g).to_numpy(), o.aggRow(A.IDXMIN, e), f"{name} idxMin")
            assert_close_rel(k.aggRow(A.MEAN, g).to_numpy(), o.aggRow(A.MEAN, e), RTOL_REDUCE_F64, f"{name} rowMean",
                             scale=1e-9)


def test_chain_longer_than_the_step_limit_is_split(ctx):
    k, o = _k()
    B = k.BinaryOpCode
    x = rng_matrix(7, 5000, 20)
    X = k.DenseMatrix.from_numpy(ctx, x)
    t, e = X, x
    for i in range(25):
        s = 1.0 + i * 0.01
        op = [B.ADD, B.MUL, B.SUB][i % 3]
        t, e = k.ewBinaryObjSca(op, t, s), o.ewBinaryObjSca(op, e, s)
    assert_bits_equal(t.to_numpy(), e, "25-step chain")


def test_division_by_broadcast_divisor_is_ieee_exact(ctx):
    """The reciprocal-based division of the fused kernels must return the bits of a/d for every operand class."""
    k, o = _k()
    B = k.BinaryOpCode
    rng = np.random.default_rng(8)
    r, c = 40000, 64
    mant = rng.random((r, c)) + 1.0
    expo = rng.integers(-1000, 1000, size=(r, c))
    a = np.ldexp(mant, expo) * rng.choice([-1.0, 1.0], size=(r, c))
    specials = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 5e-324, -5e-324, 2.2250738585072014e-308,
                         1.7976931348623157e308, 1.0, -1.0, 3.0, 1e-310])
    a[:, 0] = np.resize(specials, r)
    d = np.ldexp(rng.random((1, c)) + 1.0, rng.integers(-120, 120, size=(1, c))) * rng.choice([-1.0, 1.0], size=(1, c))
    d[0, :12] = [1.0, -1.0, 3.0, 1.9999999999999998, 0.1, 1e-320, 1e300, 1e-300, np.inf, 0.0, -0.0, np.nan]
    A_, D_ = k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, d)
    got = k.ewBinaryMat(B.DIV, A_, D_).to_numpy()
    with np.errstate(all="ignore"):
        exp = a / d
    nan = np.isnan(exp)
    assert np.array_equal(np.isnan(got), nan)
    assert_bits_equal(np.where(nan, 0.0, got), np.where(nan, 0.0, exp), "broadcast division")
    for s in (3.0, 0.1, -7.25, 1.9999999999999998, 1e-200, 1e200):
        got = k.ewBinaryObjSca(B.DIV, A_, s).to_numpy()
        with np.errstate(all="ignore"):
            exp = a / s
        nan = np.isnan(exp)
        assert np.array_equal(np.isnan(got), nan)
        assert_bits_equal(np.where(nan, 0.0, got), np.where(nan, 0.0, exp), f"division by {s}")


def test_nan_rows_and_signed_zeros_in_the_fused_row_pass(ctx):
    k, o = _k()
    A, B = k.AggOpCode, k.BinaryOpCode
    r, c = 2100, 40
    x = rng_matrix(9, r, c)
    x[5, 0] = np.nan
    x[6, 3] = np.nan
    x[7, :] = np.nan
    x[8, :] = 0.0
    x[8, ::2] = -0.0
    x[9, :] = -0.0
    x[9, 1::2] = 0.0
    x[10, :] = 7.0
    X = k.DenseMatrix.from_numpy(ctx, x)
    one = k.ewBinaryObjSca(B.MUL, X, 1.0)  # a chain that leaves the values unchanged
    e = o.ewBinaryObjSca(B.MUL, x, 1.0)
    for name in ("MIN", "MAX", "IDXMIN", "IDXMAX"):
        got, exp = k.aggRow(A[name], one).to_numpy(), o.aggRow(A[name], e)
        if got.dtype == np.float64:
            nan = np.isnan(exp)
            assert np.array_equal(np.isnan(got), nan), name
            got, exp = np.where(nan, 0.0, got), np.where(nan, 0.0, exp)
        assert_bits_equal(got, exp, f"fused {name} specials")
    xt = np.ascontiguousarray(x[:64].T.repeat(40, axis=0))  # specials in row 0 of some columns
    XT = k.DenseMatrix.from_numpy(ctx, xt)
    onet, et = k.ewBinaryObjSca(B.MUL, XT, 1.0), o.ewBinaryObjSca(B.MUL, xt, 1.0)
    for name in ("MIN", "MAX", "IDXMIN", "IDXMAX"):
        got, exp = k.aggCol(A[name], onet).to_numpy(), o.aggCol(A[name], et)
        if got.dtype == np.float64:
            nan = np.isnan(exp)
            assert np.array_equal(np.isnan(got), nan), name
            got, exp = np.where(nan, 0.0, got), np.where(nan, 0.0, exp)
        assert_bits_equal(got, exp, f"fused col {name} specials")


def test_dropped_results_are_never_computed_and_views_of_chains_work(ctx):
    k, o = _k()
    A, B = k.AggOpCode, k.BinaryOpCode
    x = rng_matrix(10, 70000, 32)
    X = k.DenseMatrix.from_numpy(ctx, x)
    X.device_ptr()
    l0 = ctx.stats()["launches"]
    t = k.ewBinaryObjSca(B.ADD, X, 1.0)
    dead = k.aggRow(A.SUM, t)
    dead.free()
    t2 = k.ewBinaryObjSca(B.MUL, t, 2.0)
    t.free()
    ctx.sync()
    assert ctx.stats()["launches"] == l0, "nothing was needed, nothing may run"
    v = t2.slice_rows(1000, 2500)  # a view forces the chain once
    assert_bits_equal(v.to_numpy(), ((x + 1.0) * 2.0)[1000:2500], "view of a chain")
    assert_bits_equal(k.aggRow(A.MAX, v).to_numpy(), o.aggRow(A.MAX, ((x + 1.0) * 2.0)[1000:2500]), "agg of view")


def test_preallocated_result_does_not_clobber_a_chain_operand(ctx):
    import ctypes as C
    from daphne_b200.lib import check, lib
    k, o = _k()
    B = k.BinaryOpCode
    x = rng_matrix(11, 70000, 16)
    X = k.DenseMatrix.from_numpy(ctx, x)
    T = k.DenseMatrix.empty(ctx, 70000, 16)
    h = C.c_void_p(T.handle.value)
    check(lib.db2_ewBinaryObjSca(ctx.handle, int(B.ADD), C.byref(h), X.handle, C.c_void_p(np.array([1.0]).ctypes.data)))
    chain = k.ewBinaryObjSca(B.MUL, T, 3.0)      # deferred, reads T's buffer
    check(lib.db2_ewBinaryObjSca(ctx.handle, int(B.SUB), C.byref(h), X.handle, C.c_void_p(np.array([9.0]).ctypes.data)))
    assert_bits_equal(chain.to_numpy(), (x + 1.0) * 3.0, "chain still sees the old values")
    assert_bits_equal(T.to_numpy(), x - 9.0, "the pre-allocated result was rewritten")
