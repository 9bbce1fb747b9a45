"""TEST INFRASTRUCTURE: numpy-facing wrappers over oracle.c (the CPU restatement of the reference's kernels).

The function names mirror daphne_b200.kernels so that a parity test is `oracle.f(x) == product.f(x)`."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

_lib = C.CDLL(str(_build.build()))

_SUF = {np.dtype(np.float64): "f64", np.dtype(np.float32): "f32", np.dtype(np.int64): "i64"}
_CT = {"f64": C.c_double, "f32": C.c_float, "i64": C.c_int64}
i64 = C.c_int64


def _p(a: np.ndarray):
    return C.c_void_p(a.ctypes.data)


def _mat(a) -> np.ndarray:
    a = np.asarray(a)
    if a.ndim == 1:
        a = a.reshape(-1, 1)
    if a.size and (a.strides[1] != a.itemsize or (a.shape[0] > 1 and a.strides[0] % a.itemsize)):
        a = np.ascontiguousarray(a)
    return a


def _ld(a: np.ndarray) -> int:
    if a.shape[0] > 1 and a.size:
        return max(a.strides[0] // a.itemsize, a.shape[1])
    return max(a.shape[1], 1)


class OracleError(RuntimeError):
    def __init__(self, code):
        super().__init__(f"oracle status {code}")
        self.code = code


def _chk(rc):
    if rc != 0:
        raise OracleError(rc)


def ewBinaryMat(op, lhs, rhs) -> np.ndarray:
    lhs, rhs = _mat(lhs), _mat(rhs)
    s = _SUF[lhs.dtype]
    res = np.empty(lhs.shape, dtype=lhs.dtype)
    f = getattr(_lib, f"orc_ew_binary_{s}")
    f.argtypes = [C.c_int, C.c_void_p, i64, i64, i64, C.c_void_p, i64, i64, i64, C.c_void_p, i64]
    _chk(f(int(op), _p(lhs), lhs.shape[0], lhs.shape[1], _ld(lhs), _p(rhs), rhs.shape[0], rhs.shape[1], _ld(rhs),
           _p(res), max(res.shape[1], 1)))
    return res


def ewBinaryObjSca(op, lhs, scalar) -> np.ndarray:
    lhs = _mat(lhs)
    s = _SUF[lhs.dtype]
    res = np.empty(lhs.shape, dtype=lhs.dtype)
    f = getattr(_lib, f"orc_ew_binary_sca_{s}")
    f.argtypes = [C.c_int, C.c_void_p, i64, i64, i64, _CT[s], C.c_void_p, i64]
    _chk(f(int(op), _p(lhs), lhs.shape[0], lhs.shape[1], _ld(lhs), lhs.dtype.type(scalar).item(), _p(res),
           max(res.shape[1], 1)))
    return res


def ewUnaryMat(op, arg) -> np.ndarray:
    arg = _mat(arg)
    s = _SUF[arg.dtype]
    res = np.empty(arg.shape, dtype=arg.dtype)
    f = getattr(_lib, f"orc_ew_unary_{s}")
    f.argtypes = [C.c_int, C.c_void_p, i64, i64, i64, C.c_void_p, i64]
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res), max(res.shape[1], 1)))
    return res


def _is_idx(op) -> bool:
    return int(op) in (4, 5)


def aggRow(op, arg) -> np.ndarray:
    arg = _mat(arg)
    s = _SUF[arg.dtype]
    res = np.empty((arg.shape[0], 1), dtype=arg.dtype)
    idx = np.empty((arg.shape[0], 1), dtype=np.uint64)
    f = getattr(_lib, f"orc_agg_row_{s}")
    f.argtypes = [C.c_int, C.c_void_p, i64, i64, i64, C.c_void_p, C.c_void_p, i64]
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res), _p(idx), 1))
    return idx if _is_idx(op) else res


def aggCol(op, arg) -> np.ndarray:
    arg = _mat(arg)
    s = _SUF[arg.dtype]
    res = np.empty((1, arg.shape[1]), dtype=arg.dtype)
    idx = np.empty((1, arg.shape[1]), dtype=np.uint64)
    f = getattr(_lib, f"orc_agg_col_{s}")
    f.argtypes = [C.c_int, C.c_void_p, i64, i64, i64, C.c_void_p, C.c_void_p]
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res), _p(idx)))
    return idx if _is_idx(op) else res


def aggAll(op, arg):
    arg = _mat(arg)
    s = _SUF[arg.dtype]
    res = np.zeros(1, dtype=arg.dtype)
    f = getattr(_lib, f"orc_agg_all_{s}")
    f.argtypes = [C.c_int, C.c_void_p, i64, i64, i64, C.c_void_p]
    _chk(f(int(op), _p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res)))
    return res[0]
