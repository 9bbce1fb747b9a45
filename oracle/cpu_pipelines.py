"""TEST INFRASTRUCTURE / CPU BASELINE: the benchmark workloads run on host cores through the reference's CPU kernels
(oracle/_ref when built, else the restatement in oracle.c).

Row partitioning follows the reference's vectorized engine with its default STATIC scheme
(src/runtime/local/vectorized/LoadPartitioning.h:84-86, MTWrapper_dense.cpp:24-120): the row range is cut into one
contiguous block per worker thread, every worker runs the whole kernel chain on its block, ROWS outputs are written in
place and ADD partials are summed afterwards (Tasks.cpp:51-82).  The kernels release the GIL (ctypes), so the workers
run in parallel."""
from __future__ import annotations

import os
from concurrent.futures import ThreadPoolExecutor

import numpy as np

from . import pyoracle, refkernels

SUM, MAX, IDXMAX = 0, 3, 5
SUB, DIV, POW = 1, 3, 4
SQRT = 3


def backend(prefer_reference: bool = True):
    """(module, kind): kind is "reference" for the reference's own kernels, "port" for the restatement."""
    if prefer_reference and refkernels.available():
        return refkernels, "reference"
    return pyoracle, "port"


def _blocks(n: int, parts: int):
    base, extra = divmod(n, parts)
    out, lo = [], 0
    for p in range(parts):
        hi = lo + base + (1 if p < extra else 0)
        if hi > lo:
            out.append((lo, hi))
        lo = hi
    return out


def host_threads() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


def standardise_aggregate(X: np.ndarray, threads: int = 1, k=None):
    """CPU twin of daphne_b200.pipelines.standardise_aggregate.  Returns (mu, sd, r, s, row_max, row_idx_max)."""
    k = k or backend()[0]
    n, c = X.shape
    blocks = _blocks(n, max(1, threads))
    with ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
        def run(f):
            return list(ex.map(f, blocks))

        parts = run(lambda b: k.aggCol(SUM, X[b[0]:b[1]]))
        s1 = parts[0].copy()
        for p in parts[1:]:
            s1 = k.ewBinaryMat(0, s1, p)
        mu = k.ewBinaryObjSca(DIV, s1, float(n))
        parts = run(lambda b: k.aggCol(SUM, k.ewBinaryObjSca(POW, k.ewBinaryMat(SUB, X[b[0]:b[1]], mu), 2.0)))
        v = parts[0].copy()
        for p in parts[1:]:
            v = k.ewBinaryMat(0, v, p)
        sd = k.ewUnaryMat(SQRT, k.ewBinaryObjSca(DIV, v, float(n)))
        r = np.empty((n, 1), dtype=X.dtype)
        m = np.empty((n, 1), dtype=X.dtype)
        idx = np.empty((n, 1), dtype=np.uint64)

        def tail(b):
            lo, hi = b
            Z = k.ewBinaryMat(DIV, k.ewBinaryMat(SUB, X[lo:hi], mu), sd)
            r[lo:hi] = k.aggRow(SUM, k.ewBinaryObjSca(POW, Z, 2.0))
            m[lo:hi] = k.aggRow(MAX, Z)
            idx[lo:hi] = k.aggRow(IDXMAX, Z)
            return k.aggAll(SUM, r[lo:hi])

        s = 0.0
        for p in run(tail):
            s = s + float(p)
    return mu, sd, r, s, m, idx


def standardise_tail(X: np.ndarray, mu: np.ndarray, sd: np.ndarray, threads: int = 1, k=None, exact_squares=False):
    """The row part of standardise_aggregate for GIVEN column statistics: (r, row_max, row_idx_max).  With
    exact_squares the squares are z * z (one correctly rounded multiplication) instead of the reference's pow(z, 2),
    which glibc evaluates to within one ulp of it."""
    k = k or backend()[0]
    n = X.shape[0]
    r = np.empty((n, 1), dtype=X.dtype)
    m = np.empty((n, 1), dtype=X.dtype)
    idx = np.empty((n, 1), dtype=np.uint64)

    def tail(b):
        lo, hi = b
        Z = k.ewBinaryMat(DIV, k.ewBinaryMat(SUB, X[lo:hi], mu), sd)
        r[lo:hi] = k.aggRow(SUM, Z * Z if exact_squares else k.ewBinaryObjSca(POW, Z, 2.0))
        m[lo:hi] = k.aggRow(MAX, Z)
        idx[lo:hi] = k.aggRow(IDXMAX, Z)

    with ThreadPoolExecutor(max_workers=max(1, threads)) as ex:
        list(ex.map(tail, _blocks(n, max(1, threads) * 4)))
    return r, m, idx


def normal_equations(X: np.ndarray, y: np.ndarray, lam: float = 0.001, k=None):
    """CPU twin of daphne_b200.pipelines.normal_equations: (A, b, beta)."""
    k = k or backend()[0]
    d = X.shape[1]
    A = k.ewBinaryMat(0, k.syrk(X, True), np.diag(np.full(d, lam)))
    b = k.gemv(X, y)
    return A, b, k.solve(A, b)


def kmeans(X: np.ndarray, C0: np.ndarray, iterations: int = 10, k=None):
    """CPU twin of daphne_b200.pipelines.kmeans: (C, assign)."""
    k = k or backend()[0]
    n, kk = X.shape[0], C0.shape[0]
    xs = k.aggRow(SUM, k.ewBinaryObjSca(POW, X, 2.0))
    rows = np.arange(n, dtype=np.int64)
    C, a = C0, None
    for _ in range(iterations):
        cs = k.transpose(k.aggRow(SUM, k.ewBinaryObjSca(POW, C, 2.0)))
        D = k.ewBinaryMat(0, k.ewBinaryMat(0, k.ewBinaryObjSca(2, k.matMul(X, C, False, True), -2.0), xs), cs)
        a = k.aggRow(4, D).astype(np.int64)
        P = k.ctable(rows, a, 1.0, n, kk)
        C = k.ewBinaryMat(DIV, k.matMul(P, X, True, False), k.transpose(k.aggCol(SUM, P)))
    return C, a


def connected_components(G, maxi: int = 1000, k=None):
    """CPU twin of daphne_b200.pipelines.connected_components on a scipy CSR matrix: (c, iterations)."""
    k = k or backend()[0]
    n = G.shape[0]
    c = k.seq(1.0, float(n), 1.0)
    it, diff = 1, 1.0
    while diff > 0.0 and it <= maxi:
        prod = k.ewMulCsrDense(G, k.transpose(c))
        u = k.ewBinaryMat(14, k.aggRowCsr(MAX, prod), c)
        diff = float(k.aggAll(SUM, k.ewBinaryMat(8, u, c)))
        c = u
        it += 1
    return c, it - 1
