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

    def pair(self, name: str, nbytes: int):
        """Two fresh events for a caller that records them itself (native code): (begin, end)."""
        import ctypes as C
        e0, e1 = C.c_void_p(), C.c_void_p()
        self._lib.db2_event_create(C.byref(e0))
        self._lib.db2_event_create(C.byref(e1))
        self._pairs.setdefault(name, []).append((e0, e1, nbytes))
        return e0, e1

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


def _allreduce_matrix(ctx, m, comm: Optional[Comm], combine=COMBINE_ADD, k=None):
    """Combines a small ADD/MIN/MAX partial (1 x c, c x c, 1 x 1) across the row shards: in place on the device with
    NCCL when the context has a communicator, through the host otherwise (CPU tests of the sharding logic)."""
    if comm is None or comm.world == 1:
        return m
    if comm.device_collectives(ctx):
        comm.allreduce_device(ctx, m, combine)
        return m
    host = comm.allreduce_numpy(m.to_numpy(), combine)
    return (k or K).DenseMatrix.from_numpy(ctx, host)


def _allreduce_scalar(ctx, x: float, comm: Optional[Comm], combine=COMBINE_ADD) -> float:
    if comm is None or comm.world == 1:
        return float(x)
    return float(comm.allreduce_numpy(np.array([x], dtype=np.float64), combine)[0])


def _sum_over_shards(ctx, K, vec, comm: Optional[Comm]):
    """sum(vec) over all row shards for an n x 1 vector.  With a device communicator the shard's sum stays on the
    device as a 1 x 1 matrix and is combined there (one NCCL call on the compute stream, nothing is read: the caller
    gets the device matrix); the generic route reads the shard's scalar and combines it through the host."""
    if comm is not None and comm.world > 1 and comm.device_collectives(ctx) and vec.cols == 1:
        part = K.aggCol(A.SUM, vec)
        comm.allreduce_device(ctx, part, COMBINE_ADD)
        return part
    return _allreduce_scalar(ctx, K.aggAll(A.SUM, vec), comm)


class StandardiseResult:
    """mu, sd: 1 x c column means / population standard deviations; r: n x 1 rowSums(Z^2); row_max: n x 1 rowMaxs(Z);
    row_idx_max: n x 1 (uint64) idxMax per row of Z; s: sum(r) over ALL shards.  On the device path the sum stays a
    1 x 1 device matrix (already combined over the ranks) and is read when `s` is first asked for."""

    def __init__(self, mu, sd, r, s, row_max, row_idx_max):
        self.mu, self.sd, self.r, self.row_max, self.row_idx_max = mu, sd, r, row_max, row_idx_max
        self._s = s

    @property
    def s(self) -> float:
        if not isinstance(self._s, float):
            self._s = float(self._s.to_numpy()[0, 0])
        return self._s


def standardise_aggregate(ctx, X, n_total: Optional[int] = None, comm: Optional[Comm] = None, probe=None,
                          kernels=None) -> StandardiseResult:
    """Column standardisation and aggregation:

        mu = mean(X, 1); sd = sqrt(var(X, 1)); Z = (X - mu) / sd;
        r = sum(Z ^ 2, 0); s = sum(r); m = aggMax(Z, 0); i = idxMax(Z, 0);

    mean/var are issued as their ADD-combinable forms (column sums divided by the global row count, then column sums
    of squared deviations from the global mean) so that row shards on several GPUs produce the global statistics;
    on one GPU this is the arithmetic of AggCol's MEAN/VAR (src/runtime/local/kernels/AggCol.h:146-173)."""
    K = kernels or globals()["K"]
    n = X.rows if n_total is None else n_total
    probe = probe or _NoProbe()
    s1 = _allreduce_matrix(ctx, K.aggCol(A.SUM, X), comm, k=K)
    mu = K.ewBinaryObjSca(B.DIV, s1, float(n))
    d = K.ewBinaryMat(B.SUB, X, mu)
    d2 = K.ewBinaryObjSca(B.POW, d, 2.0)
    d.free()
    v = _allreduce_matrix(ctx, K.aggCol(A.SUM, d2), comm, k=K)
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
    s = _sum_over_shards(ctx, K, r, comm)
    return StandardiseResult(mu, sd, r, s, m, i)


@dataclass
class NormalEquationsResult:
    A: object      # d x d   t(X) X + lambda I (global)
    b: object      # d x 1   t(X) y (global)
    beta: object   # d x 1   solve(A, b)


def normal_equations(ctx, X, y, lam: float = 0.001, comm: Optional[Comm] = None, probe=None,
                     kernels=None) -> NormalEquationsResult:
    """Linear regression by the normal equations (lmDS, scripts/algorithms/lmDS_.daph:98-112):

        A = t(X) @ X + diagMatrix(fill(lambda, ncol(X), 1));  b = t(X) @ y;  beta = solve(A, b);

    t(X) @ X lowers to syrk and t(X) @ y to gemv (PhyOperatorSelectionPass.cpp:54-71); both are ADD-combined over the
    row shards."""
    K = kernels or globals()["K"]
    probe = probe or _NoProbe()
    d = X.cols
    # t(X) X is deferred until t(X) y arrives: both come out of one pass over X (the fold into the syrk kernel)
    with probe.section("gemm_f64_kernel syrk t(X)X with t(X)y folded in", X.rows * (d + 1) * 8):
        xtx = K.syrk(X, True)
        xty = K.gemv(X, y)
    xtx = _allreduce_matrix(ctx, xtx, comm, k=K)
    xty = _allreduce_matrix(ctx, xty, comm, k=K)
    A = K.ewBinaryMat(B.ADD, xtx, K.diagMatrix(K.fill(ctx, lam, d, 1)))
    beta = K.solve(A, xty)
    return NormalEquationsResult(A, xty, beta)


@dataclass
class KMeansResult:
    C: object        # k x d centroids after the last update (global)
    assign: object   # n x 1 (int64) cluster of every local row in the last iteration


def kmeans(ctx, X, C0, iterations: int = 10, comm: Optional[Comm] = None, kernels=None) -> KMeansResult:
    """K-means assignment + update:

        xs = sum(X ^ 2, 0);
        for i: D = (X @ t(C)) * -2.0 + xs + t(sum(C ^ 2, 0));  a = idxMin(D, 0);
               P = ctable(seq(0, n - 1), a, 1.0, n, k);  C = (t(P) @ X) / t(sum(P, 1));

    Ties in idxMin go to the lowest index (AggRow.h:71-83).  The centroid sums t(P) @ X and the counts sum(P, 1) are
    ADD-combined over the row shards."""
    K = kernels or globals()["K"]
    n, k = X.rows, C0.rows
    xs = K.aggRow(A.SUM, K.ewBinaryObjSca(B.POW, X, 2.0))
    rows = K.seq(ctx, 0, n - 1, 1, dtype=np.int64)
    Cm, assign = C0, None
    for _ in range(iterations):
        cs = K.transpose(K.aggRow(A.SUM, K.ewBinaryObjSca(B.POW, Cm, 2.0)))
        xc = K.matMul(X, Cm, False, True)
        D = K.ewBinaryMat(B.ADD, K.ewBinaryMat(B.ADD, K.ewBinaryObjSca(B.MUL, xc, -2.0), xs), cs)
        assign = K.castObj(K.aggRow(A.IDXMIN, D), np.int64)
        D.free()
        xc.free()
        P = K.ctable(rows, assign, 1.0, n, k)
        sums = _allreduce_matrix(ctx, K.matMul(P, X, True, False), comm, k=K)
        counts = _allreduce_matrix(ctx, K.aggCol(A.SUM, P), comm, k=K)
        P.free()
        Cm = K.ewBinaryMat(B.DIV, sums, K.transpose(counts))
    return KMeansResult(Cm, assign)


@dataclass
class ComponentsResult:
    c: object    # n_local x 1 component label of every local vertex
    iterations: int


def connected_components(ctx, G, maxi: int = 1000, comm: Optional[Comm] = None, row_block: Optional[tuple] = None,
                         kernels=None) -> ComponentsResult:
    """Connected components by label propagation (test/api/cli/algorithms/components.daphne:14-26):

        c = seq(1, n, 1);  while (diff > 0 && iter <= maxi):
            u = max(aggMax(G * t(c), 0), c);  diff = sum(u != c);  c = u;

    G is the row shard [row_block) of the symmetric 0/1 adjacency matrix (all n columns); every rank needs the whole
    label vector for the gather G * t(c), so the updated shard is all-gathered each iteration and the change count is
    ADD-combined."""
    K = kernels or globals()["K"]
    n = G.cols
    lo, hi = row_block if row_block is not None else (0, G.rows)
    sharded = comm is not None and comm.world > 1
    on_device = sharded and comm.device_collectives(ctx)
    c_full = K.seq(ctx, 1.0, float(n), 1.0)
    it, diff = 1, 1.0
    c_loc = c_full.slice_rows(lo, hi)
    while diff > 0.0 and it <= maxi:
        prod = K.ewMulCsrDense(G, K.transpose(c_full))
        u = K.ewBinaryMat(B.MAX, K.aggRowCsr(A.MAX, prod), c_loc)
        changed = K.ewBinaryMat(B.NEQ, u, c_loc)
        if on_device:
            # the shard's change count stays on the device and is combined there; the all-gather of the labels is
            # issued behind it on the same stream, so the one host read below waits for both
            cnt = K.aggCol(A.SUM, changed)
            comm.allreduce_device(ctx, cnt, COMBINE_ADD)
            c_full = comm.allgather_rows(ctx, u, n, k=K)
            c_loc = c_full.slice_rows(lo, hi)
            diff = float(cnt.to_numpy()[0, 0])
        else:
            diff = _allreduce_scalar(ctx, K.aggAll(A.SUM, changed), comm)
            if sharded:
                c_full = comm.allgather_rows(ctx, u, n, k=K)
                c_loc = c_full.slice_rows(lo, hi)
            else:
                c_full = u
                c_loc = u
        it += 1
    return ComponentsResult(c_loc, it - 1)


# ---- the same sequences issued from native code (csrc/workloads.cu): what a JIT-compiled caller costs on the host ----

def connected_components_native(ctx, G, maxi: int = 1000, row_block: Optional[tuple] = None) -> ComponentsResult:
    """connected_components through db2w_connected_components: the same operator calls, made from C++."""
    import ctypes as C

    from .lib import check, lib
    lo = row_block[0] if row_block is not None else 0
    h, it = C.c_void_p(), C.c_int64()
    check(lib.db2w_connected_components(ctx.handle, G.handle, int(lo), int(maxi), C.byref(h), C.byref(it)))
    return ComponentsResult(K.DenseMatrix(ctx, h), it.value)


def standardise_aggregate_native(ctx, X, n_total: Optional[int] = None, probe=None) -> StandardiseResult:
    """standardise_aggregate through db2w_standardise: the same operator calls, made from C++.  Row shards are
    combined through the communicator of the context; s stays a 1 x 1 device matrix until it is read."""
    import ctypes as C

    from .lib import check, lib
    e0 = e1 = None
    if probe is not None:
        e0, e1 = probe.pair("fused_row_kernel (Z=(X-mu)/sd; rowSums(Z^2), rowMaxs(Z), idxMax(Z))",
                            X.rows * (X.cols * 8 + 24))
    h = [C.c_void_p() for _ in range(6)]
    check(lib.db2w_standardise(ctx.handle, X.handle, int(X.rows if n_total is None else n_total),
                               *[C.byref(x) for x in h], e0, e1))
    mu, sd, r, m, i, s = (K.DenseMatrix(ctx, x) for x in h)
    return StandardiseResult(mu, sd, r, s, m, i)


def kmeans_native(ctx, X, C0, iterations: int = 10) -> KMeansResult:
    import ctypes as C

    from .lib import check, lib
    c, a = C.c_void_p(), C.c_void_p()
    check(lib.db2w_kmeans(ctx.handle, X.handle, C0.handle, int(iterations), C.byref(c), C.byref(a)))
    return KMeansResult(K.DenseMatrix(ctx, c), K.DenseMatrix(ctx, a))


def normal_equations_native(ctx, X, y, lam: float = 0.001) -> NormalEquationsResult:
    import ctypes as C

    from .lib import check, lib
    a, b, beta = C.c_void_p(), C.c_void_p(), C.c_void_p()
    check(lib.db2w_normal_equations(ctx.handle, X.handle, y.handle, float(lam), C.byref(a), C.byref(b), C.byref(beta)))
    return NormalEquationsResult(K.DenseMatrix(ctx, a), K.DenseMatrix(ctx, b), K.DenseMatrix(ctx, beta))
