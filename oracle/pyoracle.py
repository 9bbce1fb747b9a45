"""TEST INFRASTRUCTURE: numpy-facing wrappers over oracle.c (the CPU restatement of the reference's kernels).

The function names mirror daphne_b200.kernels so that a parity test is `oracle.f(x) == product.f(x)`."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import build as _build

_lib = C.CDLL(str(_build.build()))

_SUF = {np.dtype(np.float64): "f64", np.dtype(np.float32): "f32", np.dtype(np.int64): "i64",
        np.dtype(np.uint64): "u64", np.dtype(np.int32): "i32", np.dtype(np.uint32): "u32"}
_CT = {"f64": C.c_double, "f32": C.c_float, "i64": C.c_int64, "u64": C.c_uint64, "i32": C.c_int32,
       "u32": C.c_uint32}
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


def _la_lib(prefix):
    return _lib, prefix


def _matmul(lib, prefix, lhs, rhs, transa=False, transb=False):
    lhs, rhs = _mat(np.asarray(lhs, dtype=np.float64)), _mat(np.asarray(rhs, dtype=np.float64))
    m = lhs.shape[1] if transa else lhs.shape[0]
    n = rhs.shape[0] if transb else rhs.shape[1]
    res = np.empty((m, n))
    f = getattr(lib, f"{prefix}_matmul_f64")
    if prefix == "orc":
        f.argtypes = [C.c_void_p, i64, i64, i64, C.c_void_p, i64, i64, i64, C.c_int, C.c_int, C.c_void_p, i64]
        _chk(f(_p(lhs), lhs.shape[0], lhs.shape[1], _ld(lhs), _p(rhs), rhs.shape[0], rhs.shape[1], _ld(rhs),
               int(transa), int(transb), _p(res), max(n, 1)))
    else:
        f.argtypes = [C.c_void_p, i64, i64, i64, C.c_void_p, i64, i64, i64, C.c_int, C.c_int, C.c_void_p]
        _chk(f(_p(lhs), lhs.shape[0], lhs.shape[1], _ld(lhs), _p(rhs), rhs.shape[0], rhs.shape[1], _ld(rhs),
               int(transa), int(transb), _p(res)))
    return res


def matMul(lhs, rhs, transa=False, transb=False):
    if np.asarray(lhs).dtype in (np.int64, np.int32):
        return _matmul_int(lhs, rhs, transa, transb)
    return _matmul(_lib, "orc", lhs, rhs, transa, transb)


def _matmul_int(lhs, rhs, transa=False, transb=False):
    """The integer forms (int64, int32): wrapping products and sums."""
    dt = np.asarray(lhs).dtype
    lhs, rhs = _mat(np.asarray(lhs, dtype=dt)), _mat(np.asarray(rhs, dtype=dt))
    m = lhs.shape[1] if transa else lhs.shape[0]
    n = rhs.shape[0] if transb else rhs.shape[1]
    res = np.empty((m, n), dtype=dt)
    f = getattr(_lib, "orc_matmul_i64" if dt == np.int64 else "orc_matmul_i32")
    f.argtypes = [C.c_void_p, i64, i64, i64, C.c_void_p, i64, i64, i64, C.c_int, C.c_int, C.c_void_p, i64]
    _chk(f(_p(lhs), lhs.shape[0], lhs.shape[1], _ld(lhs), _p(rhs), rhs.shape[0], rhs.shape[1], _ld(rhs),
           int(transa), int(transb), _p(res), max(n, 1)))
    return res


def _syrk(lib, prefix, arg, transLeft=True):
    arg = _mat(np.asarray(arg, dtype=np.float64))
    n = arg.shape[1] if transLeft else arg.shape[0]
    res = np.empty((n, n))
    f = getattr(lib, f"{prefix}_syrk_f64")
    f.argtypes = [C.c_void_p, i64, i64, i64, C.c_int, C.c_void_p]
    _chk(f(_p(arg), arg.shape[0], arg.shape[1], _ld(arg), int(transLeft), _p(res)))
    return res


def syrk(arg, transLeft=True):
    return _syrk(_lib, "orc", arg, transLeft)


def gemv(mat, vec):
    mat = _mat(np.asarray(mat, dtype=np.float64))
    vec = np.ascontiguousarray(np.asarray(vec, dtype=np.float64).reshape(-1, 1))
    res = np.empty((mat.shape[1], 1))
    f = _lib.orc_gemv_f64
    f.argtypes = [C.c_void_p, i64, i64, i64, C.c_void_p, i64, C.c_void_p]
    _chk(f(_p(mat), mat.shape[0], mat.shape[1], _ld(mat), _p(vec), 1, _p(res)))
    return res


def _solve(lib, prefix, a, b):
    a = np.ascontiguousarray(np.asarray(a, dtype=np.float64))
    b = np.ascontiguousarray(np.asarray(b, dtype=np.float64).reshape(-1, 1))
    x = np.empty((a.shape[0], 1))
    f = getattr(lib, f"{prefix}_solve_f64")
    f.argtypes = [C.c_void_p, i64, C.c_void_p, C.c_void_p]
    _chk(f(_p(a), a.shape[0], _p(b), _p(x)))
    return x


def solve(a, b):
    return _solve(_lib, "orc", a, b)


def transpose(arg):
    arg = _mat(np.asarray(arg, dtype=np.float64))
    res = np.empty((arg.shape[1], arg.shape[0]))
    f = _lib.orc_transpose_f64
    f.argtypes = [C.c_void_p, i64, i64, i64, C.c_void_p]
    _chk(f(_p(arg), arg.shape[0], arg.shape[1], _ld(arg), _p(res)))
    return res


def _ctable(lib, prefix, lhs, rhs, weight=1.0, resNumRows=-1, resNumCols=-1):
    lhs = np.ascontiguousarray(np.asarray(lhs, dtype=np.int64).reshape(-1))
    rhs = np.ascontiguousarray(np.asarray(rhs, dtype=np.int64).reshape(-1))
    f = getattr(lib, f"{prefix}_ctable_f64")
    f.argtypes = [C.c_void_p, C.c_void_p, i64, C.c_double, i64, i64, C.c_void_p, C.c_void_p, C.c_void_p]
    r, c = C.c_int64(), C.c_int64()
    _chk(f(_p(lhs), _p(rhs), lhs.size, float(weight), resNumRows, resNumCols, None, C.byref(r), C.byref(c)))
    res = np.empty((r.value, c.value))
    _chk(f(_p(lhs), _p(rhs), lhs.size, float(weight), resNumRows, resNumCols, _p(res), C.byref(r), C.byref(c)))
    return res


def ctable(lhs, rhs, weight=1.0, resNumRows=-1, resNumCols=-1):
    return _ctable(_lib, "orc", lhs, rhs, weight, resNumRows, resNumCols)


def _seq(lib, prefix, start, end, inc):
    f = getattr(lib, f"{prefix}_seq_f64")
    f.argtypes = [C.c_double, C.c_double, C.c_double, C.c_void_p, i64, C.c_void_p]
    n = C.c_int64()
    _chk(f(float(start), float(end), float(inc), None, 0, C.byref(n)))
    res = np.empty((n.value + 1, 1))
    _chk(f(float(start), float(end), float(inc), _p(res), res.shape[0], C.byref(n)))
    return res[:n.value].copy()


def seq(start, end, inc):
    return _seq(_lib, "orc", start, end, inc)


def outerBinary(op, lhs, rhs) -> np.ndarray:
    """OuterBinary<Dense,Dense,Dense> (src/runtime/local/kernels/OuterBinary.h:52-78): res[r][c] = f(lhs[r], rhs[c])
    with f the scalar function EwBinaryMat uses for the same opcode, so row r is EwBinaryMat of lhs[r] repeated
    against the row vector rhs."""
    lhs, rhs = _mat(lhs), _mat(rhs)
    if lhs.shape[1] != 1:
        raise OracleError("outerBinary: lhs must be a column (mx1) matrix")
    if rhs.shape[0] != 1:
        raise OracleError("outerBinary: rhs must be a row (1xn) matrix")
    return ewBinaryMat(op, np.ascontiguousarray(np.repeat(lhs, rhs.shape[1], axis=1)), rhs)


def cond(cnd, then, els, dtype=np.float64) -> np.ndarray:
    """CondMatMatMat / CondMatMatSca / CondMatScaMat / CondMatScaSca<Dense...> (src/runtime/local/kernels/
    CondMatMatMat.h:50-83 and siblings): res = static_cast<bool>(cond) ? then : else per element; matrix operands
    must have the shape of cond."""
    cnd = _mat(cnd)
    mats = [np.asarray(x) for x in (then, els) if isinstance(x, np.ndarray)]
    dt = mats[0].dtype if mats else np.dtype(dtype)
    for x in mats:
        if _mat(x).shape != cnd.shape:
            raise OracleError("Cond: condition/then/else matrices must have the same shape")
    res = np.empty(cnd.shape, dtype=dt)
    for r in range(cnd.shape[0]):
        for c in range(cnd.shape[1]):
            t = _mat(then)[r, c] if isinstance(then, np.ndarray) else dt.type(then)
            e = _mat(els)[r, c] if isinstance(els, np.ndarray) else dt.type(els)
            res[r, c] = t if bool(cnd[r, c]) else e
    return res


def aggCum(op, arg) -> np.ndarray:
    """AggCum<Dense,Dense> (src/runtime/local/kernels/AggCum.h:48-86): row 0 is copied, row r is f(result row r - 1,
    argument row r) with f the scalar function of the opcode's binary twin (SUM -> ADD, PROD -> MUL, MIN, MAX)."""
    twin = {0: 0, 1: 2, 2: 13, 3: 14}
    if int(op) not in twin:
        raise OracleError("the aggregation function used in aggCum must be a pure binary reduction")
    arg = _mat(arg)
    res = np.empty_like(arg)
    if arg.shape[0] == 0:
        return res
    res[0] = arg[0]
    for r in range(1, arg.shape[0]):
        res[r] = ewBinaryMat(twin[int(op)], np.ascontiguousarray(res[r - 1:r]), np.ascontiguousarray(arg[r:r + 1]))
    return res


def oneHot(arg, info) -> np.ndarray:
    """OneHot<Dense,Dense> (src/runtime/local/kernels/OneHot.h:54-110)."""
    arg, info = _mat(arg), np.asarray(info)
    if info.ndim != 2 or info.shape[0] != 1:
        raise OracleError("OneHot - parameter 'info' must be a row matrix")
    if info.shape[1] != arg.shape[1]:
        raise OracleError("OneHot - parameter 'info' must provide information for each column of parameter arg")
    if (info < -1).any():
        raise OracleError("OneHot: parameter 'info' must be an integer greater or equal than -1")
    width = int(sum(1 if n == -1 else n for n in info[0]))
    if width == 0:
        raise OracleError("OneHot: parameter 'info' must contain at least one non-zero entry")
    res = np.empty((arg.shape[0], width), dtype=arg.dtype)
    for r in range(arg.shape[0]):
        c_res = 0
        for c_arg in range(arg.shape[1]):
            n = int(info[0, c_arg])
            if n == -1:
                res[r, c_res] = arg[r, c_arg]
                c_res += 1
            elif n != 0:
                res[r, c_res:c_res + n] = 0
                v = arg[r, c_arg]
                k = int(v) if v == v and v >= 0 else -1  # static_cast<size_t>: negatives / NaN name no position
                if not 0 <= k < n:
                    raise OracleError("OneHot: arg values that are encoded (info value != -1) must be positive and "
                                      "smaller than the corresponding info value")
                res[r, c_res + k] = 1
                c_res += n
    return res


def colBind(lhs, rhs) -> np.ndarray:
    """ColBind<Dense,Dense,Dense> (src/runtime/local/kernels/ColBind.h:54-88): row r of the result is row r of lhs
    followed by row r of rhs; operands with different row counts are an error."""
    lhs, rhs = _mat(lhs), _mat(rhs)
    if lhs.shape[0] != rhs.shape[0]:
        raise OracleError(f"ColBind - the two operands must have the same number of rows, but lhs has {lhs.shape[0]} "
                          f"and rhs has {rhs.shape[0]} rows")
    res = np.empty((lhs.shape[0], lhs.shape[1] + rhs.shape[1]), dtype=lhs.dtype)
    for r in range(lhs.shape[0]):
        res[r, : lhs.shape[1]] = lhs[r]
        res[r, lhs.shape[1]:] = rhs[r]
    return res


def extractCol(arg, sel) -> np.ndarray:
    """ExtractCol<Dense,Dense,Dense<VTSel>> (src/runtime/local/kernels/ExtractCol.h:64-105): sel is a column matrix of
    column positions; a negative position counts from the end; anything outside [0, cols) is out_of_range."""
    arg, sel = _mat(arg), np.asarray(sel)
    if sel.ndim != 2 or sel.shape[1] != 1:
        raise OracleError("invalid argument passed to ExtractCol: column selection must be given as column matrix but "
                          f"has '{sel.shape[1] if sel.ndim == 2 else '?'}' columns instead of one")
    cols = arg.shape[1]
    res = np.empty((arg.shape[0], sel.shape[0]), dtype=arg.dtype)
    for c in range(sel.shape[0]):
        given = int(sel[c, 0])
        p = given + cols if given < 0 else given
        if p < 0 or p >= cols:
            raise OracleError(f"invalid argument '{given}' passed to ExtractCol: out of bounds for dense matrix with "
                              f"column boundaries '[0, {cols})'")
        res[:, c] = arg[:, p]
    return res


def _slice_bounds(what, lower, upper, extent):
    """The bounds rule shared by SliceRow and SliceCol (src/runtime/local/kernels/SliceRow.h:55-82,
    SliceCol.h:55-84): a negative lower bound counts from the end (and takes an upper bound <= 0 with it), a negative
    upper bound alone counts from the end; then 0 <= lower < extent and lower <= upper <= extent must hold."""
    lo, up = int(lower), int(upper)
    if lo < 0:
        lo += extent
        if up <= 0:
            up += extent
    elif up < 0:
        up += extent
    if lo < 0 or lo >= extent or up < lo or extent < up:
        raise OracleError(f"invalid arguments '{lo}, {up}' passed to {what}")
    return lo, up


def sliceRow(arg, lowerIncl, upperExcl) -> np.ndarray:
    """SliceRow<Dense,Dense,VTSel> (src/runtime/local/kernels/SliceRow.h:71-82): rows [lowerIncl, upperExcl)."""
    arg = _mat(arg)
    lo, up = _slice_bounds("SliceRow", lowerIncl, upperExcl, arg.shape[0])
    return arg[lo:up, :]


def sliceCol(arg, lowerIncl, upperExcl) -> np.ndarray:
    """SliceCol<Dense,Dense,VTSel> (src/runtime/local/kernels/SliceCol.h:73-86): columns [lowerIncl, upperExcl)."""
    arg = _mat(arg)
    lo, up = _slice_bounds("SliceCol", lowerIncl, upperExcl, arg.shape[1])
    return arg[:, lo:up]


def _csr_arrays(m):
    """(values f64, colIdxs u64, rowOffsets u64, rows, cols) from a scipy CSR matrix or an equivalent tuple."""
    if isinstance(m, tuple):
        vals, cols_, offs, rows, cols = m
    else:
        m = m.tocsr()
        m.sort_indices()
        vals, cols_, offs, (rows, cols) = m.data, m.indices, m.indptr, m.shape
    return (np.ascontiguousarray(vals, dtype=np.float64), np.ascontiguousarray(cols_, dtype=np.uint64),
            np.ascontiguousarray(offs, dtype=np.uint64), int(rows), int(cols))


def _csr_ewmul(lib, prefix, m, rhs):
    vals, cidx, roff, rows, cols = _csr_arrays(m)
    rhs = _mat(np.ascontiguousarray(rhs, dtype=np.float64))
    ov, oc, oo = np.empty_like(vals), np.empty_like(cidx), np.empty_like(roff)
    n = C.c_int64()
    f = getattr(lib, f"{prefix}_csr_ewmul_dense_f64")
    if prefix == "orc":
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, i64, i64, C.c_void_p, i64, i64, C.c_void_p, C.c_void_p,
                      C.c_void_p, C.c_void_p]
        _chk(f(_p(vals), _p(cidx), _p(roff), rows, cols, _p(rhs), rhs.shape[0], rhs.shape[1], _p(ov), _p(oc), _p(oo),
               C.byref(n)))
    else:
        f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, i64, i64, i64, C.c_void_p, i64, i64, C.c_void_p, C.c_void_p,
                      C.c_void_p, C.c_void_p]
        _chk(f(_p(vals), _p(cidx), _p(roff), rows, cols, vals.size, _p(rhs), rhs.shape[0], rhs.shape[1], _p(ov),
               _p(oc), _p(oo), C.byref(n)))
    return (ov[:n.value].copy(), oc[:n.value].copy(), oo, rows, cols)


def ewMulCsrDense(m, rhs):
    return _csr_ewmul(_lib, "orc", m, rhs)


def aggRowCsr(op, m):
    vals, cidx, roff, rows, cols = _csr_arrays(m)
    res = np.empty((rows, 1))
    f = _lib.orc_csr_agg_row_f64
    f.argtypes = [C.c_int, C.c_void_p, C.c_void_p, i64, i64, C.c_void_p]
    _chk(f(int(op), _p(vals), _p(roff), rows, cols, _p(res)))
    return res


def matMulCsrDense(m, rhs):
    vals, cidx, roff, rows, cols = _csr_arrays(m)
    rhs = np.ascontiguousarray(_mat(np.asarray(rhs, dtype=np.float64)))
    res = np.empty((rows, rhs.shape[1]))
    f = _lib.orc_csr_gemv_f64
    f.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, i64, C.c_void_p, i64, C.c_void_p]
    _chk(f(_p(vals), _p(cidx), _p(roff), rows, _p(rhs), rhs.shape[1], _p(res)))
    return res
