"""One-pass column statistics: the pass that produces the column sums / means of a large f64 matrix also keeps shifted
first and second moments, from which var / stddev and the deferred sum((X - mu)^2) are answered without reading the
matrix again.  Against the reference's two-pass arithmetic (AggCol.h:146-173, restated in the oracle): 1e-12 relative,
the tolerance of f64 reductions -- plus the oracle's own distance from the exactly rounded result where that is larger
(for data around 1e9 the reference's sequentially summed mean is off by 5e-5, which moves ITS variance by 1e-9; the
device value must then be within 1e-12 of the extended-precision result instead).  The cases include data far from
zero (a naive sum of squares would lose everything), a pivot row that is an outlier (the answer kernel must refuse and the two-pass kernels run), and buffers that are
released or rewritten between the two calls (stale statistics must not be used)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
RTOL = 1e-12


def _k():
    import daphne_b200.kernels as k
    from daphne_b200.kernels import AggOpCode as A, BinaryOpCode as B
    from oracle import pyoracle as o
    return k, A, B, o


def _rel(got, exp):
    return float(np.abs(got - exp).max() / np.abs(exp).max())


def _truth(op_name, x):
    xl = x.astype(np.longdouble)
    m = xl.mean(0, keepdims=True)
    v = ((xl - m) ** 2).mean(0, keepdims=True)
    return {"MEAN": m, "VAR": v, "STDDEV": np.sqrt(v), "SUM": xl.sum(0, keepdims=True)}[op_name]


def _check(got, op, x, o, what=""):
    """1e-12 from the extended-precision result, and from the oracle as far as the oracle itself is that close"""
    truth = _truth(op.name, x)
    ref = o.aggCol(op, x)
    assert _rel(got.astype(np.longdouble), truth) <= RTOL, f"{op.name} {what}"
    assert _rel(got, ref) <= RTOL + 2.0 * _rel(ref.astype(np.longdouble), truth), f"{op.name} {what} vs oracle"


@pytest.mark.parametrize("offset,scale", [(5.0, 2.0), (1e9, 1.0), (-3e6, 1e-3), (0.0, 1e8)])
def test_mean_var_stddev_after_one_pass(ctx, offset, scale):
    k, A, B, o = _k()
    x = offset + scale * np.random.default_rng(31).standard_normal((300000, 16))
    X = k.DenseMatrix.from_numpy(ctx, x)
    s0 = ctx.stats()["launches"]
    mean = k.aggCol(A.MEAN, X).to_numpy()
    var = k.aggCol(A.VAR, X).to_numpy()
    sd = k.aggCol(A.STDDEV, X).to_numpy()
    launches = ctx.stats()["launches"] - s0
    _check(mean, A.MEAN, x, o)
    _check(var, A.VAR, x, o)
    _check(sd, A.STDDEV, x, o)
    assert launches <= 4, "var and stddev are answered from the statistics of the mean pass"
    _check(k.aggCol(A.SUM, X).to_numpy(), A.SUM, x, o)


def test_var_alone_and_odd_shapes(ctx):
    k, A, B, o = _k()
    rng = np.random.default_rng(32)
    for rows, cols in [(1 << 22, 1), (600000, 7), (70000, 64), (40000, 129), (5000, 1000)]:
        x = 3.0 + rng.standard_normal((rows, cols))
        X = k.DenseMatrix.from_numpy(ctx, x)
        _check(k.aggCol(A.VAR, X).to_numpy(), A.VAR, x, o, (rows, cols))
        _check(k.aggCol(A.SUM, X).to_numpy(), A.SUM, x, o, (rows, cols))
    # a view with a leading dimension and an odd offset
    big = 2.0 + rng.standard_normal((200000, 40))
    v = big[:, 3:36]
    V = k.DenseMatrix.from_numpy(ctx, v)
    _check(k.aggCol(A.VAR, V).to_numpy(), A.VAR, np.ascontiguousarray(v), o, "view")


def test_outlier_pivot_falls_back_to_two_passes(ctx):
    k, A, B, o = _k()
    x = np.random.default_rng(33).standard_normal((300000, 16))
    x[0, :] = 1e9   # the pivot row: 1e9 standard deviations away in every column
    x[0, 3] = 0.5   # ... except one
    X = k.DenseMatrix.from_numpy(ctx, x)
    k.aggCol(A.MEAN, X)
    _check(k.aggCol(A.VAR, X).to_numpy(), A.VAR, x, o)
    _check(k.aggCol(A.STDDEV, X).to_numpy(), A.STDDEV, x, o)


def test_deferred_sum_of_squared_deviations(ctx):
    k, A, B, o = _k()
    rng = np.random.default_rng(34)
    x = 5.0 + 2.0 * rng.standard_normal((400000, 32))
    n = x.shape[0]
    X = k.DenseMatrix.from_numpy(ctx, x)
    s1 = k.aggCol(A.SUM, X)
    mu = k.ewBinaryObjSca(B.DIV, s1, float(n))
    s0 = ctx.stats()["launches"]
    v = k.aggCol(A.SUM, k.ewBinaryObjSca(B.POW, k.ewBinaryMat(B.SUB, X, mu), 2.0)).to_numpy()
    # the answer from the statistics, and behind it the two kernels of the ordinary pass, which look at the device
    # flag and return at once: no pass over X, no wait for the host
    assert ctx.stats()["launches"] - s0 <= 4
    mu_h = mu.to_numpy()
    assert _rel(v, ((x - mu_h) ** 2).sum(0, keepdims=True)) <= RTOL
    # any other row vector (the global mean of a sharded run differs from the shard's own)
    other = k.DenseMatrix.from_numpy(ctx, mu_h + 0.37)
    v2 = k.aggCol(A.SUM, k.ewBinaryObjSca(B.POW, k.ewBinaryMat(B.SUB, X, other), 2.0)).to_numpy()
    assert _rel(v2, ((x - (mu_h + 0.37)) ** 2).sum(0, keepdims=True)) <= RTOL
    # a row vector far from the data: ill-conditioned for the identity, the ordinary pass must answer
    far = k.DenseMatrix.from_numpy(ctx, mu_h + 1e7)
    v3 = k.aggCol(A.SUM, k.ewBinaryObjSca(B.POW, k.ewBinaryMat(B.SUB, X, far), 2.0)).to_numpy()
    assert _rel(v3, ((x - (mu_h + 1e7)) ** 2).sum(0, keepdims=True)) <= RTOL


def test_statistics_do_not_survive_their_buffer(ctx):
    k, A, B, o = _k()
    rng = np.random.default_rng(35)
    x = rng.standard_normal((300000, 16))
    X = k.DenseMatrix.from_numpy(ctx, x)
    k.aggCol(A.MEAN, X).to_numpy()
    X.free()
    y = 10.0 + 3.0 * rng.standard_normal((300000, 16))  # same size: the allocator hands the same block out again
    Y = k.DenseMatrix.from_numpy(ctx, y)
    _check(k.aggCol(A.VAR, Y).to_numpy(), A.VAR, y, o)
    # a different matrix aggregated in between replaces the statistics
    Z = k.DenseMatrix.from_numpy(ctx, x)
    k.aggCol(A.MEAN, Y)
    k.aggCol(A.MEAN, Z)
    _check(k.aggCol(A.VAR, Y).to_numpy(), A.VAR, y, o)
    _check(k.aggCol(A.VAR, Z).to_numpy(), A.VAR, x, o)
