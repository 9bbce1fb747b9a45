"""Several GPUs in one process: device groups, row-distributed matrices and the scheduler that splits a pipeline's row
range over the devices (db2_vectorizedPipelineGroup) against the single-device scheduler.

Every test runs on a group of two contexts that share device 0 (partials are then combined with copies and the fold
kernel, no NCCL), so the multi-device code path is exercised on a one-GPU machine; with two or more GPUs the same
tests also run over all devices with the NCCL combine."""
import numpy as np
import pytest

from tests.util import assert_bits_equal, rng_matrix

pytestmark = pytest.mark.gpu

ROWS, COLS, ADD, MIN, MAX = 1, 2, 3, 4, 5


def _k():
    import daphne_b200.kernels as k
    return k


def _device_lists():
    from daphne_b200 import lib
    n = lib.device_count()
    lists = [[0, 0], [0, 0, 0]]
    if n >= 2:
        lists.append(list(range(n)))
    return lists


@pytest.fixture(params=_device_lists(), ids=lambda d: "dev" + "".join(map(str, d)))
def group(request):
    k = _k()
    g = k.Group(request.param)
    yield g
    g.close()


def _body(k):
    B, A = k.BinaryOpCode, k.AggOpCode

    def body(ins, ctx=None):
        xs, m = ins
        d = k.ewBinaryMat(B.SUB, xs, m)
        return [k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, d, 2.0)),   # ROWS
                k.aggRow(A.IDXMAX, d),                               # ROWS (uint64)
                k.aggCol(A.SUM, d),                                  # ADD
                k.aggCol(A.MIN, xs),                                 # MIN
                k.aggCol(A.MAX, xs),                                 # MAX
                k.transpose(k.aggRow(A.MAX, xs))]                    # COLS
    return body


@pytest.mark.parametrize("rows", [70001, 1234])
def test_group_scheduler_equals_the_single_device_scheduler(ctx, group, rows):
    k = _k()
    x = rng_matrix(3, rows, 32)
    mu = x.mean(axis=0, keepdims=True)
    combines = [ROWS, ROWS, ADD, MIN, MAX, COLS]
    one = k.vectorizedPipeline(ctx, [k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, mu)], [1, 0],
                               combines, lambda ins: _body(k)(ins))
    X = k.DistMatrix.from_numpy(group, x)
    MU = k.DistMatrix.from_matrix(group, k.DenseMatrix.from_numpy(group.contexts[0], mu), replicate=True)
    outs = k.vectorizedPipelineGroup(group, [X, MU], [1, 0], combines, _body(k))
    assert [o.axis for o in outs] == [0, 0, -1, -1, -1, 1]
    r, i, s, mn, mx, t = outs
    assert_bits_equal(r.to_numpy(), one[0].to_numpy(), "ROWS result")
    assert_bits_equal(i.to_numpy(), one[1].to_numpy(), "ROWS index result")
    np.testing.assert_allclose(s.to_numpy(), one[2].to_numpy(), rtol=1e-12, atol=1e-9)
    assert_bits_equal(mn.to_numpy(), one[3].to_numpy(), "MIN combine")
    assert_bits_equal(mx.to_numpy(), one[4].to_numpy(), "MAX combine")
    assert_bits_equal(t.to_numpy(), one[5].to_numpy(), "COLS result")
    # every device holds the same combined value, bit for bit
    first = s.shard(0)[0].to_numpy()
    for d in range(1, group.size):
        assert_bits_equal(s.shard(d)[0].to_numpy(), first, f"combined ADD result on device index {d}")
    # the row partition: contiguous blocks, the first rows % n devices one row taller
    offs = [r.shard(d)[1] for d in range(group.size)] + [rows]
    sizes = np.diff(offs)
    assert sizes.sum() == rows and sizes.max() - sizes.min() <= 1 and list(sizes) == sorted(sizes, reverse=True)
    # gathered onto one device, and fed to the next pipeline while still distributed
    assert_bits_equal(r.gather(group.size - 1).to_numpy(), one[0].to_numpy(), "gather")
    (r2,) = k.vectorizedPipelineGroup(group, [r], [1], [ADD], lambda ins, c: [k.aggCol(k.AggOpCode.SUM, ins[0])])
    np.testing.assert_allclose(r2.to_numpy(), one[0].to_numpy().sum(keepdims=True), rtol=1e-12)


def test_device_resident_input_is_split_with_peer_copies(ctx, group):
    k = _k()
    x = rng_matrix(5, 4099, 7)
    Xd = k.DenseMatrix.from_numpy(group.contexts[0], x)
    Xd.device_ptr()  # the latest copy is on device index 0
    X = k.DistMatrix.from_matrix(group, Xd)
    assert_bits_equal(X.to_numpy(), x, "distributed copy")
    (z,) = k.vectorizedPipelineGroup(group, [X], [1], [ROWS],
                                     lambda ins, c: [k.ewBinaryObjSca(k.BinaryOpCode.MUL, ins[0], 3.0)])
    assert_bits_equal(z.to_numpy(), x * 3.0, "elementwise body over peer-copied shards")


def test_group_errors(ctx, group):
    k = _k()
    x = rng_matrix(6, 5000, 4)
    X = k.DistMatrix.from_numpy(group, x)
    with pytest.raises(k.Db2Error, match="must be replicated"):
        k.vectorizedPipelineGroup(group, [X, X], [1, 0], [ROWS], lambda ins, c: [ins[0]])
    if group.size >= 3:  # (a single row would be a broadcast input)
        few = k.DistMatrix.from_numpy(group, np.ones((group.size - 1, 4)))
        with pytest.raises(k.Db2Error, match="cannot be split over"):
            k.vectorizedPipelineGroup(group, [few], [1], [ROWS], lambda ins, c: [ins[0]])

    def bad(ins, c):
        raise RuntimeError("body failed")
    with pytest.raises(RuntimeError, match="body failed"):
        k.vectorizedPipelineGroup(group, [X], [1], [ROWS], bad)
    other = k.Group([0])
    try:
        with pytest.raises(k.Db2Error, match="does not belong to this device group"):
            k.vectorizedPipelineGroup(other, [X], [1], [ROWS], lambda ins, c: [ins[0]])
    finally:
        other.close()


def test_standardisation_over_a_group(ctx, group):
    """The column standardisation workload as three pipelines over the group: column sums (ADD), squared deviations
    (ADD), row results (ROWS) -- equal to the single-device pipeline."""
    k = _k()
    from daphne_b200 import pipelines
    B, A, U = k.BinaryOpCode, k.AggOpCode, k.UnaryOpCode
    n, c = 300007, 32
    x = 5.0 + 2.0 * np.random.default_rng(2).standard_normal((n, c))
    one = pipelines.standardise_aggregate(ctx, k.DenseMatrix.from_numpy(ctx, x))
    X = k.DistMatrix.from_numpy(group, x)
    (s1,) = k.vectorizedPipelineGroup(group, [X], [1], [ADD], lambda ins, cx: [k.aggCol(A.SUM, ins[0])])

    def per_device(dist, f):  # small replicated follow-up arithmetic on every device
        hs = []
        for d in range(group.size):
            m, _ = dist.shard(d)
            hs.append(f(m))
        return hs

    mus = per_device(s1, lambda m: k.ewBinaryObjSca(B.DIV, m, float(n)))
    MU = k.DistMatrix.from_matrix(group, mus[0], replicate=True)
    (v,) = k.vectorizedPipelineGroup(
        group, [X, MU], [1, 0], [ADD],
        lambda ins, cx: [k.aggCol(A.SUM, k.ewBinaryObjSca(B.POW, k.ewBinaryMat(B.SUB, ins[0], ins[1]), 2.0))])
    sds = per_device(v, lambda m: k.ewUnaryMat(U.SQRT, k.ewBinaryObjSca(B.DIV, m, float(n))))
    SD = k.DistMatrix.from_matrix(group, sds[0], replicate=True)

    def tail(ins, cx):
        xs, mu, sd = ins
        Z = k.ewBinaryMat(B.DIV, k.ewBinaryMat(B.SUB, xs, mu), sd)
        r = k.aggRow(A.SUM, k.ewBinaryObjSca(B.POW, Z, 2.0))
        return [r, k.aggRow(A.MAX, Z), k.aggRow(A.IDXMAX, Z), k.aggCol(A.SUM, r)]
    r, m, i, s = k.vectorizedPipelineGroup(group, [X, MU, SD], [1, 0, 0], [ROWS, ROWS, ROWS, ADD], tail)
    np.testing.assert_allclose(mus[0].to_numpy(), one.mu.to_numpy(), rtol=1e-13)
    np.testing.assert_allclose(sds[0].to_numpy(), one.sd.to_numpy(), rtol=1e-12)
    np.testing.assert_allclose(r.to_numpy(), one.r.to_numpy(), rtol=1e-10)
    np.testing.assert_allclose(m.to_numpy(), one.row_max.to_numpy(), rtol=1e-10, atol=1e-10)
    assert (i.to_numpy() != one.row_idx_max.to_numpy()).mean() < 1e-5
    assert abs(float(s.to_numpy()[0, 0]) - one.s) <= 1e-10 * one.s
