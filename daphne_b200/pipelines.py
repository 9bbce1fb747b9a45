"""The kernel-call sequences that the benchmark workloads lower to, written against the host-side kernel interface.

Each function issues exactly the operator calls DAPHNE's compiler emits for the corresponding DaphneDSL script
(PhyOperatorSelection: t(X)@X -> syrk, t(X)@y -> gemv; one kernel call per op), in row-sharded form: every rank runs
the same calls on its row block and ADD partials are combined across ranks (VectorCombine::ADD,
src/ir/daphneir/DaphneVectorizableOpInterface.cpp:313-350,407-430)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

from . import kernels as K
from .dist import COMBINE_ADD, Comm
from .kernels import AggOpCode as A
from .kernels import BinaryOpCode as B
from .kernels import UnaryOpCode as U


class Probe:
    """CUDA-event timing of named kernel launches inside a pipeline (events are recorded on the stream the kernels are
    launched on).  Used by the measurement harness to time the dominant kernel live inside the timed region."""

    def __init__(self, lib, stream):
        self._lib, self._stream = lib, stream
        self._pairs = {}

    def reset(self):
        self._pairs = {}

    def section(self, name: str, nbytes: int):
        probe = self

        class _S:
            def __enter__(self_inner):
                import ctypes as C
                self_inner.e0, self_inner.e1 = C.c_void_p(), C.c_void_p()
                probe._lib.db2_event_create(C.byref(self_inner.e0))
                probe._lib.db2_event_create(C.byref(self_inner.e1))
                probe._lib.db2_event_record(self_inner.e0, probe._stream)

            def __exit__(self_inner, *exc):
                probe._lib.db2_event_record(self_inner.e1, probe._stream)
                probe._pairs.setdefault(name, []).append((self_inner.e0, self_inner.e1, nbytes))

        return _S()

    def summary(self):
        """The section with the largest total time: name, launches, average ms, algorithmic GB/s."""
        import ctypes as C
        best = None
        for name, pairs in self._pairs.items():
            tot, nbytes = 0.0, 0
            for e0, e1, nb in pairs:
                ms = C.c_float()
                self._lib.db2_event_elapsed_ms(e0, e1, C.byref(ms))
                tot += ms.value
                nbytes = nb
                self._lib.db2_event_destroy(e0)
                self._lib.db2_event_destroy(e1)
            avg = tot / max(1, len(pairs))
            if best is None or tot > best["total_ms"]:
                best = {"name": name, "launches": len(pairs), "avg_ms": avg, "total_ms": tot, "bytes": nbytes,
                        "gbs": nbytes / (avg * 1e-3) / 1e9 if avg > 0 else 0.0}
        self._pairs = {}
        return best


class _NoProbe:
    def section(self, name, nbytes):
        import contextlib
        return contextlib.nullcontext()


def _allreduce_matrix(ctx: K.Context, m: K.DenseMatrix, comm: Optional[Comm], combine=COMBINE_ADD) -> K.DenseMatrix:
    """Combines a small ADD/MIN/MAX partial (1 x c, c x c, 1 x 1) across the row shards."""
    if comm is None or comm.world == 1:
        return m
    host = comm.allreduce_numpy(m.to_numpy(), combine)
    return K.DenseMatrix.from_numpy(ctx, host)


@dataclass
class StandardiseResult:
    mu: K.DenseMatrix        # 1 x c   column means
    sd: K.DenseMatrix        # 1 x c   column standard deviations (population)
    r: K.DenseMatrix         # n x 1   rowSums(Z^2)
    s: float                 #         sum(r) over ALL shards
    row_max: K.DenseMatrix   # n x 1   rowMaxs(Z)
    row_idx_max: K.DenseMatrix  # n x 1 (uint64) idxMax per row of Z


def standardise_aggregate(ctx: K.Context, X: K.DenseMatrix, n_total: Optional[int] = None,
                          comm: Optional[Comm] = None, probe=None) -> StandardiseResult:
    """Column standardisation and aggregation:

        mu = mean(X, 1); sd = sqrt(var(X, 1)); Z = (X - mu) / sd;
        r = sum(Z ^ 2, 0); s = sum(r); m = aggMax(Z, 0); i = idxMax(Z, 0);

    mean/var are issued as their ADD-combinable forms (column sums divided by the global row count, then column sums
    of squared deviations from the global mean) so that row shards on several GPUs produce the global statistics;
    on one GPU this is the arithmetic of AggCol's MEAN/VAR (src/runtime/local/kernels/AggCol.h:146-173)."""
    n = X.rows if n_total is None else n_total
    probe = probe or _NoProbe()
    s1 = _allreduce_matrix(ctx, K.aggCol(A.SUM, X), comm)
    mu = K.ewBinaryObjSca(B.DIV, s1, float(n))
    d = K.ewBinaryMat(B.SUB, X, mu)
    d2 = K.ewBinaryObjSca(B.POW, d, 2.0)
    d.free()
    v = _allreduce_matrix(ctx, K.aggCol(A.SUM, d2), comm)
    d2.free()
    var = K.ewBinaryObjSca(B.DIV, v, float(n))
    sd = K.ewUnaryMat(U.SQRT, var)
    xc = K.ewBinaryMat(B.SUB, X, mu)
    Z = K.ewBinaryMat(B.DIV, xc, sd)
    xc.free()
    z2 = K.ewBinaryObjSca(B.POW, Z, 2.0)
    r = K.aggRow(A.SUM, z2)
    z2.free()
    m = K.aggRow(A.MAX, Z)
    i = K.aggRow(A.IDXMAX, Z)
    Z.free()
    with probe.section("fused_row_kernel (Z=(X-mu)/sd; rowSums(Z^2), rowMaxs(Z), idxMax(Z))",
                       X.rows * (X.cols * 8 + 24)):
        r.device_ptr()  # the three row aggregations are produced by one pass over X
    s_local = K.aggAll(A.SUM, r)
    s = float(s_local) if comm is None or comm.world == 1 else float(
        comm.allreduce_numpy(np.array([s_local], dtype=np.float64))[0])
    return StandardiseResult(mu, sd, r, s, m, i)
