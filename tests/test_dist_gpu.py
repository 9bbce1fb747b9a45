"""Row-sharded runs on two GPUs, one process per GPU (NCCL), against the same workloads on one GPU: the statistics
exchange of the standardisation workload (one all-gather that carries every rank's column statistics, after which the
squared deviations from the global mean need no second exchange), the device-side change count and the ragged
all-gather of connected components, the ADD-combines of k-means and of the normal equations.  Skipped with fewer than
two GPUs."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
pytestmark = pytest.mark.gpu


def _two_gpus() -> bool:
    try:
        from daphne_b200 import lib
        return lib.device_count() >= 2
    except Exception:
        return False


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


N2, N4 = 4_200_001, 200_001   # odd sizes: the two ranks hold blocks of different heights


def _inputs():
    x = 5.0 + 2.0 * np.random.default_rng(2).standard_normal((N2, 16))
    from tests.test_pipelines_gpu import _graph
    g = _graph(N4, 6, 9)
    xk = np.random.default_rng(3).random((300_001, 64))
    return x, g, xk


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    import torch
    import torch.distributed as dist

    import daphne_b200.kernels as K
    from daphne_b200 import pipelines
    from daphne_b200.dist import Comm, row_block

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    comm = Comm(rank, world, "nccl")
    ctx = K.Context(rank)
    comm.init_device(ctx)
    x, g, xk = _inputs()
    res = {}
    lo, hi = row_block(x.shape[0], rank, world)
    c0 = ctx.stats()["collectives"]
    r = pipelines.standardise_aggregate(ctx, K.DenseMatrix.from_numpy(ctx, np.ascontiguousarray(x[lo:hi])),
                                        x.shape[0], comm)
    res["collectives"] = ctx.stats()["collectives"] - c0
    res["mu"], res["sd"], res["s"] = r.mu.to_numpy(), r.sd.to_numpy(), r.s
    res["r"], res["m"], res["i"] = (comm.allgather_ragged(v.to_numpy()) for v in (r.r, r.row_max, r.row_idx_max))
    lo, hi = row_block(x.shape[0], rank, world)
    c0 = ctx.stats()["collectives"]
    rn = pipelines.standardise_aggregate_native(ctx, K.DenseMatrix.from_numpy(ctx, np.ascontiguousarray(x[lo:hi])),
                                                x.shape[0])
    res["collectives_native"] = ctx.stats()["collectives"] - c0
    res["native_equal"] = all(np.array_equal(a.to_numpy(), b.to_numpy()) for a, b in
                              ((r.mu, rn.mu), (r.sd, rn.sd), (r.r, rn.r), (r.row_max, rn.row_max),
                               (r.row_idx_max, rn.row_idx_max))) and rn.s == r.s
    lo, hi = row_block(g.shape[0], rank, world)
    G = K.CSRMatrix.from_scipy(ctx, g[lo:hi])
    cc = pipelines.connected_components_native(ctx, G, 1000, (lo, hi))
    res["c"], res["iters"] = comm.allgather_ragged(cc.c.to_numpy()), cc.iterations
    cc2 = pipelines.connected_components(ctx, G, 1000, comm, (lo, hi))
    res["c_py"] = comm.allgather_ragged(cc2.c.to_numpy())
    lo, hi = row_block(xk.shape[0], rank, world)
    km = pipelines.kmeans_native(ctx, K.DenseMatrix.from_numpy(ctx, np.ascontiguousarray(xk[lo:hi])),
                                 K.DenseMatrix.from_numpy(ctx, xk[:50].copy()), 3)
    res["C"], res["assign"] = km.C.to_numpy(), comm.allgather_ragged(km.assign.to_numpy())
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **res)
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.skipif(not _two_gpus(), reason="needs two GPUs")
def test_two_gpus_equal_one_gpu(tmp_path, ctx):
    import torch.multiprocessing as mp

    import daphne_b200.kernels as K
    from daphne_b200 import pipelines
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    ranks = [np.load(tmp_path / f"rank{r}.npz") for r in range(2)]
    x, g, xk = _inputs()
    one = pipelines.standardise_aggregate(ctx, K.DenseMatrix.from_numpy(ctx, x))
    cc = pipelines.connected_components(ctx, K.CSRMatrix.from_scipy(ctx, g))
    km = pipelines.kmeans(ctx, K.DenseMatrix.from_numpy(ctx, xk), K.DenseMatrix.from_numpy(ctx, xk[:50].copy()), 3)
    for r in ranks:
        # one exchange for the statistics and one for the final scalar
        assert int(r["collectives"]) == 2, f"collectives per standardisation pipeline: {int(r['collectives'])}"
        assert int(r["collectives_native"]) == 2 and bool(r["native_equal"])  # the same calls, made from C++
        np.testing.assert_allclose(r["mu"], one.mu.to_numpy(), rtol=1e-13)
        np.testing.assert_allclose(r["sd"], one.sd.to_numpy(), rtol=1e-12)
        assert abs(float(r["s"]) - one.s) <= 1e-10 * abs(one.s)
        np.testing.assert_allclose(r["r"], one.r.to_numpy(), rtol=1e-9)
        np.testing.assert_allclose(r["m"], one.row_max.to_numpy(), rtol=1e-9, atol=1e-9)
        assert (r["i"] != one.row_idx_max.to_numpy()).mean() < 1e-5
        assert np.array_equal(r["c"], cc.c.to_numpy()) and np.array_equal(r["c_py"], cc.c.to_numpy())
        assert int(r["iters"]) == cc.iterations
        np.testing.assert_allclose(r["C"], km.C.to_numpy(), rtol=1e-12)
        assert np.array_equal(r["assign"], km.assign.to_numpy())
    for key in ("mu", "sd", "C"):  # both ranks end with the same bits
        assert np.array_equal(ranks[0][key], ranks[1][key])
