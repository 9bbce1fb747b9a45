"""TEST INFRASTRUCTURE / CPU BASELINE: the reference's own multithreaded vectorized engine (MTWrapper, tasks, workers,
queues; src/runtime/local/vectorized/*) driving the reference's CPU kernels, compiled from a DAPHNE source tree by
oracle/Makefile into oracle/_ref/libdaphne_ref_engine.so (driver: oracle/ref_engine.cpp).  `available()` is False when
that library was not built."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

_PATH = Path(__file__).resolve().parent / "_ref" / "libdaphne_ref_engine.so"
_lib = None

ENGINE = ("VectorizedPipeline<DenseMatrix<double>>::apply -> MTWrapper::executeCpuQueues, STATIC partitioning, "
          "96 KiB batches, one centralized queue; meanCol, varCol, idxmaxRow stand-alone (not vectorizable)")


def available() -> bool:
    global _lib
    if _lib is None and _PATH.exists():
        try:
            _lib = C.CDLL(str(_PATH))
            vp = C.c_void_p
            _lib.ref_engine_standardise.argtypes = [vp, C.c_int64, C.c_int64, C.c_int, C.c_int, vp, vp, vp, vp, vp,
                                                    vp, vp]
            _lib.ref_engine_standardise.restype = C.c_int
        except OSError:
            _lib = False
    return bool(_lib)


def default_threads() -> int:
    """Worker threads the engine starts when none are configured: one per CPU this process may run on."""
    return int(_lib.ref_engine_default_threads())


def standardise_aggregate(X: np.ndarray, threads: int = 0, vectorized: bool = True, results: bool = True):
    """Runs the column standardisation workload once.  Returns (mu, sd, r, s, row_max, row_idx_max, ms) where ms is
    the wall time in milliseconds of (column statistics, pipeline, idxmaxRow, total); with results=False only s and ms
    are filled (nothing is copied out)."""
    X = np.ascontiguousarray(X, dtype=np.float64)
    n, c = X.shape
    ms = (C.c_double * 4)()
    s = C.c_double()
    if results:
        mu, sd = np.empty((1, c)), np.empty((1, c))
        r, m, idx = np.empty((n, 1)), np.empty((n, 1)), np.empty((n, 1), dtype=np.uint64)
        ptrs = [a.ctypes.data for a in (mu, sd, r, m, idx)]
    else:
        mu = sd = r = m = idx = None
        ptrs = [None] * 5
    rc = _lib.ref_engine_standardise(X.ctypes.data, n, c, int(threads), 1 if vectorized else 0, *ptrs,
                                     C.addressof(s), C.addressof(ms))
    if rc != 0:
        raise RuntimeError("the reference engine raised an exception")
    return mu, sd, r, s.value, m, idx, tuple(ms)
