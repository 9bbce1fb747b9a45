"""TEST INFRASTRUCTURE: numpy-facing wrappers over oracle/_ref/libdaphne_ref.so, i.e. the reference's own CPU kernels
compiled from a DAPHNE source tree by oracle/Makefile.  `available()` is False when that library was not built (for
instance on a machine without the source tree); callers then fall back to the restatement in oracle.c."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import pyoracle as _o

_PATH = Path(__file__).resolve().parent / "_ref" / "libdaphne_ref.so"
_lib = None


def available() -> bool:
    global _lib
    if _lib is None and _PATH.exists():
        try:
            _lib = C.CDLL(str(_PATH))
        except OSError:
            _lib = False
    return bool(_lib)


def _f(name, argtypes):
    fn = getattr(_lib, name)
    fn.argtypes = argtypes
    fn.restype = C.c_int
    return fn


i64, vp = C.c_int64, C.c_void_p
_mat, _ld, _p, _SUF, _CT, _chk = _o._mat, _o._ld, _o._p, _o._SUF, _o._CT, _o._chk


def set_blas_threads(n: int) -> None:
    _lib.ref_set_blas_threads(C.c_int(n))


def ewBinaryMat(op, lhs, rhs):
    lhs, rhs = _mat(lhs), _mat(rhs)
    res = np.empty(lhs.shape, dtype=lhs.dtype)
    f = _f(f"ref_ew_binary_{_SUF[lhs.dtype]}", [C.c_int, vp, i64, i64, i64, vp, i64, i64, i64, vp, i64])
    _chk(f(int(op), _p(lhs), lhs.shape[0], lhs.shape[1], _ld(lhs), _p(rhs), rhs.shape[0], rhs.shape[1], _ld(rhs),
           _p(res), max(res.shape[1], 1)))
    return res


def ewBinaryObjSca(op, lhs, scalar):
    lhs = _mat(lhs)
    s = _SUF[lhs.dtype]
    res = np.empty(lhs.shape, dtype=lhs.dtype)
    f = _f(f"ref_ew_binary_sca_{s}", [C.c_int, vp, i64, i64, i64, _CT[s], vp, i64])
    _chk(f(int(op), _p(lhs), lhs.shape[0], lhs.shape[1], _ld(lhs), lhs.dtype.type(scalar).item(), _p(res),
           max(res.shape[1], 1)))
    return res


def ewUnaryMat(op, arg):
    arg = _mat(arg)
    res = np.empty(arg.shape, dtype=arg.dtype)
    f = _f(f"ref_ew_unary_{_SUF[arg.dtype]}", [C.c_int, vp, i64, i64, i64, vp, i64])
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res), max(res.shape[1], 1)))
    return res


def aggRow(op, arg):
    arg = _mat(arg)
    res = np.empty((arg.shape[0], 1), dtype=arg.dtype)
    idx = np.empty((arg.shape[0], 1), dtype=np.uint64)
    f = _f(f"ref_agg_row_{_SUF[arg.dtype]}", [C.c_int, vp, i64, i64, i64, vp, vp, i64])
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res), _p(idx), 1))
    return idx if _o._is_idx(op) else res


def aggCol(op, arg):
    arg = _mat(arg)
    res = np.empty((1, arg.shape[1]), dtype=arg.dtype)
    idx = np.empty((1, arg.shape[1]), dtype=np.uint64)
    f = _f(f"ref_agg_col_{_SUF[arg.dtype]}", [C.c_int, vp, i64, i64, i64, vp, vp])
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res), _p(idx)))
    return idx if _o._is_idx(op) else res


def aggAll(op, arg):
    arg = _mat(arg)
    res = np.zeros(1, dtype=arg.dtype)
    f = _f(f"ref_agg_all_{_SUF[arg.dtype]}", [C.c_int, vp, i64, i64, i64, vp])
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res)))
    return res[0]


def matMul(lhs, rhs, transa=False, transb=False):
    return _o._matmul(_lib, "ref", lhs, rhs, transa, transb)


def syrk(arg, transLeft=True):
    return _o._syrk(_lib, "ref", arg, transLeft)


def gemv(mat, vec):
    mat = _mat(np.asarray(mat, dtype=np.float64))
    vec = np.ascontiguousarray(np.asarray(vec, dtype=np.float64).reshape(-1, 1))
    res = np.empty((mat.shape[1], 1))
    f = _f("ref_gemv_f64", [vp, i64, i64, i64, vp, vp])
    _chk(f(_p(mat), mat.shape[0], mat.shape[1], _ld(mat), _p(vec), _p(res)))
    return res


def solve(a, b):
    return _o._solve(_lib, "ref", a, b)


def transpose(arg):
    arg = _mat(np.asarray(arg, dtype=np.float64))
    res = np.empty((arg.shape[1], arg.shape[0]))
    f = _f("ref_transpose_f64", [vp, i64, i64, i64, vp])
    _chk(f(_p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res)))
    return res


def ctable(lhs, rhs, weight=1.0, resNumRows=-1, resNumCols=-1):
    return _o._ctable(_lib, "ref", lhs, rhs, weight, resNumRows, resNumCols)


def seq(start, end, inc):
    return _o._seq(_lib, "ref", start, end, inc)


def rand(rows, cols, lo, hi, sparsity, seed):
    """The reference's RandMatrix kernel = DaphneDSL rand(rows, cols, lo, hi, sparsity, seed)."""
    res = np.empty((rows, cols))
    f = _f("ref_rand_f64", [i64, i64, C.c_double, C.c_double, C.c_double, i64, vp])
    _chk(f(rows, cols, float(lo), float(hi), float(sparsity), int(seed), _p(res)))
    return res


def ewMulCsrDense(m, rhs):
    return _o._csr_ewmul(_lib, "ref", m, rhs)


def aggRowCsr(op, m):
    vals, cidx, roff, rows, cols = _o._csr_arrays(m)
    res = np.empty((rows, 1))
    f = _f("ref_csr_agg_row_f64", [C.c_int, vp, vp, vp, i64, i64, i64, vp])
    _chk(f(int(op), _p(vals), _p(cidx), _p(roff), rows, cols, vals.size, _p(res)))
    return res


def matMulCsrDense(m, rhs):
    vals, cidx, roff, rows, cols = _o._csr_arrays(m)
    rhs = np.ascontiguousarray(_mat(np.asarray(rhs, dtype=np.float64)))
    res = np.empty((rows, rhs.shape[1]))
    f = _f("ref_csr_gemv_f64", [vp, vp, vp, i64, i64, i64, vp, i64, vp])
    _chk(f(_p(vals), _p(cidx), _p(roff), rows, cols, vals.size, _p(rhs), rhs.shape[1], _p(res)))
    return res


available()  # load the library at import when it exists


_DBDF = {np.dtype(np.float64): "f64", np.dtype(np.float32): "f32", np.dtype(np.int64): "i64"}


def writeDaphne(arr, path) -> None:
    """The reference's own WriteDaphne<DenseMatrix<VT>> (src/runtime/local/io/WriteDaphne.h:62-80)."""
    a = np.ascontiguousarray(arr)
    f = _f(f"ref_write_dbdf_{_DBDF[a.dtype]}", [C.c_char_p, C.c_void_p, C.c_int64, C.c_int64])
    _chk(f(str(path).encode(), C.c_void_p(a.ctypes.data), a.shape[0], a.shape[1]))


def readDaphne(path, dtype=np.float64):
    """The reference's own ReadDaphne<DenseMatrix<VT>> (src/runtime/local/io/ReadDaphne.h:58-100)."""
    import os
    dt = np.dtype(dtype)
    cap = max(1, (os.path.getsize(path) - 45) // dt.itemsize)
    out = np.empty(cap, dtype=dt)
    r, c = C.c_int64(), C.c_int64()
    f = _f(f"ref_read_dbdf_{_DBDF[dt]}", [C.c_char_p, C.c_void_p, C.c_int64, C.POINTER(C.c_int64), C.POINTER(C.c_int64)])
    _chk(f(str(path).encode(), C.c_void_p(out.ctypes.data), cap, C.byref(r), C.byref(c)))
    return out[: r.value * c.value].reshape(r.value, c.value)
