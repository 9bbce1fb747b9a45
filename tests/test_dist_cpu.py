"""Row sharding and cross-rank combination on CPU ranks (torch.distributed, gloo, world size 2 and 3).

The kernels are replaced by the CPU oracle (tests/cpu_shim.py); what is under test is the host logic that the
multi-GPU runs share: contiguous row blocks, ADD-combination of partial statistics / t(X)X / centroid sums, the
all-gather of the label vector, and that the sharded result equals the unsharded one (bit-identical for integer,
index and connected-components output; within 1e-12 for floating-point sums, whose grouping changes with the number
of shards)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import scipy.sparse as sp
    import torch.distributed as dist

    from daphne_b200 import pipelines
    from daphne_b200.dist import Comm, row_block
    from tests import cpu_shim as K
    from tests.test_pipelines_gpu import _graph

    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm = Comm(rank, world, "gloo")
    res = {}
    # standardisation: every rank owns a row block, the statistics are global
    x = 5.0 + 2.0 * np.random.default_rng(2).standard_normal((3001, 8))
    lo, hi = row_block(x.shape[0], rank, world)
    r = pipelines.standardise_aggregate(None, K.DenseMatrix(x[lo:hi]), x.shape[0], comm, kernels=K)
    res["mu"], res["sd"], res["s"] = r.mu.a, r.sd.a, r.s
    res["r"], res["m"], res["i"] = (comm.allgather_ragged(v.a) for v in (r.r, r.row_max, r.row_idx_max))
    # normal equations
    xx = np.random.default_rng(5).random((2000, 12))
    yy = xx @ np.arange(12.0).reshape(-1, 1)
    lo, hi = row_block(2000, rank, world)
    ne = pipelines.normal_equations(None, K.DenseMatrix(xx[lo:hi]), K.DenseMatrix(yy[lo:hi]), 0.001, comm, kernels=K)
    res["A"], res["beta"] = ne.A.a, ne.beta.a
    # k-means
    xk = np.random.default_rng(3).random((1200, 6))
    c0 = xk[:5].copy()
    lo, hi = row_block(1200, rank, world)
    km = pipelines.kmeans(None, K.DenseMatrix(xk[lo:hi]), K.DenseMatrix(c0), 4, comm, kernels=K)
    res["C"], res["assign"] = km.C.a, comm.allgather_ragged(km.assign.a)
    # connected components (the label vector is all-gathered every iteration; 601 vertices: ragged shards)
    g = _graph(601, 3, 9)
    lo, hi = row_block(601, rank, world)
    cc = pipelines.connected_components(None, K.CSRMatrix(g[lo:hi]), 1000, comm, (lo, hi), kernels=K)
    res["c"], res["iters"] = comm.allgather_ragged(cc.c.a), cc.iterations
    # a shard that is not the rank's block is refused before anything is exchanged
    try:
        comm.allgather_rows(None, K.DenseMatrix(np.zeros((hi - lo + 1, 1))), 601, k=K)
        res["refused"] = 0
    except ValueError:
        res["refused"] = 1
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **res)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_pipelines_equal_the_unsharded_ones(tmp_path, world):
    from daphne_b200 import pipelines
    from tests import cpu_shim as K
    from tests.test_pipelines_gpu import _graph

    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    ranks = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    # single-process results
    x = 5.0 + 2.0 * np.random.default_rng(2).standard_normal((3001, 8))
    one = pipelines.standardise_aggregate(None, K.DenseMatrix(x), kernels=K)
    xx = np.random.default_rng(5).random((2000, 12))
    yy = xx @ np.arange(12.0).reshape(-1, 1)
    ne = pipelines.normal_equations(None, K.DenseMatrix(xx), K.DenseMatrix(yy), 0.001, kernels=K)
    xk = np.random.default_rng(3).random((1200, 6))
    km = pipelines.kmeans(None, K.DenseMatrix(xk), K.DenseMatrix(xk[:5].copy()), 4, kernels=K)
    cc = pipelines.connected_components(None, K.CSRMatrix(_graph(601, 3, 9)), kernels=K)
    for r in ranks:
        np.testing.assert_allclose(r["mu"], one.mu.a, rtol=1e-12)
        np.testing.assert_allclose(r["sd"], one.sd.a, rtol=1e-12)
        assert abs(float(r["s"]) - one.s) <= 1e-10 * abs(one.s)
        np.testing.assert_allclose(r["r"], one.r.a, rtol=1e-9)
        np.testing.assert_allclose(r["m"], one.row_max.a, rtol=1e-9, atol=1e-9)
        assert np.array_equal(r["i"], one.row_idx_max.a)
        assert np.abs(r["A"] - ne.A.a).max() <= 1e-12 * np.abs(ne.A.a).max()
        np.testing.assert_allclose(r["beta"], ne.beta.a, rtol=1e-6)
        np.testing.assert_allclose(r["C"], km.C.a, rtol=1e-12)
        assert np.array_equal(r["assign"], km.assign.a)
        assert np.array_equal(r["c"], cc.c.a), "connected components must be bit-identical for every shard count"
        assert int(r["iters"]) == cc.iterations
        assert int(r["refused"]) == 1
    for r in ranks[1:]:  # every rank ends with the same global values
        for key in ("mu", "sd", "A", "beta", "C"):
            assert np.array_equal(r[key], ranks[0][key])


def test_row_blocks_partition_the_rows():
    from daphne_b200.dist import row_block
    for n in (0, 1, 7, 100, 16_777_216):
        for world in (1, 2, 3, 4, 8):
            blocks = [row_block(n, r, world) for r in range(world)]
            assert blocks[0][0] == 0 and blocks[-1][1] == n
            assert all(blocks[i][1] == blocks[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in blocks]
            assert max(sizes) - min(sizes) <= 1
