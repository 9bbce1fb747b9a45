"""Host-side mirror of the reference's kernel interface for the hot path.

Function names, argument order and error behaviour follow the convenience functions of
src/runtime/local/kernels/*.h (ewBinaryMat, ewBinaryObjSca, ewUnaryMat, aggRow, aggCol, aggAll, ...), so the parity
tests read like the reference's own unit tests.  Everything here is a thin ctypes call into the C-ABI runtime
(include/daphne_b200.h); numpy is only used to hand host buffers in and out."""
from __future__ import annotations

import ctypes as C
import enum
from typing import Optional

import numpy as np

from . import lib as _l
from .lib import Db2Error, check, lib

_NP2DT = {np.dtype(np.float64): _l.F64, np.dtype(np.float32): _l.F32, np.dtype(np.int64): _l.I64,
          np.dtype(np.uint64): _l.U64, np.dtype(np.int32): _l.I32, np.dtype(np.uint32): _l.U32,
          np.dtype(np.uint8): _l.U8}
_DT2NP = {v: k for k, v in _NP2DT.items()}


class BinaryOpCode(enum.IntEnum):  # BinaryOpCode.h:29-56
    ADD = 0; SUB = 1; MUL = 2; DIV = 3; POW = 4; MOD = 5; LOG = 6; EQ = 7; NEQ = 8; LT = 9; LE = 10; GT = 11
    GE = 12; MIN = 13; MAX = 14; AND = 15; OR = 16; BITWISE_AND = 17


class UnaryOpCode(enum.IntEnum):  # UnaryOpCode.h:26-56
    MINUS = 0; ABS = 1; SIGN = 2; SQRT = 3; EXP = 4; LN = 5; SIN = 6; COS = 7; TAN = 8; ASIN = 9; ACOS = 10
    ATAN = 11; SINH = 12; COSH = 13; TANH = 14; FLOOR = 15; CEIL = 16; ROUND = 17; ISNAN = 18


class AggOpCode(enum.IntEnum):  # AggOpCode.h:25-35
    SUM = 0; PROD = 1; MIN = 2; MAX = 3; IDXMIN = 4; IDXMAX = 5; MEAN = 6; STDDEV = 7; VAR = 8


class Context:
    """One per device (db2_context): stream, pooled device memory, counters."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        check(lib.db2_context_create(int(device), C.byref(self._h)))
        self.device = int(device)

    @property
    def handle(self):
        return self._h

    @property
    def stream(self) -> int:
        return lib.db2_context_stream(self._h) or 0

    def sync(self) -> None:
        check(lib.db2_context_sync(self._h))

    def side_sync(self) -> None:
        """Waits for the copies queued by DenseMatrix.to_numpy_async (and the collectives of the second stream)."""
        check(lib.db2_context_side_sync(self._h))

    def stats(self) -> dict:
        s = _l.Stats()
        check(lib.db2_context_stats(self._h, C.byref(s)))
        return {f: getattr(s, f) for f, _ in s._fields_}

    def close(self) -> None:
        if self._h:
            lib.db2_context_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class DenseMatrix:
    """Handle to a db2_matrix.  `from_numpy` makes the array the host placement (no copy); the device placement is
    created when a kernel first needs it."""

    def __init__(self, ctx: Context, handle, keep=None):
        self.ctx = ctx
        self._h = handle
        self._keep = keep  # host array backing a borrowed host placement
        dt, r, c = C.c_int(), C.c_int64(), C.c_int64()
        check(lib.db2_matrix_info(self._h, C.byref(dt), C.byref(r), C.byref(c)))
        self.dtype_code, self.rows, self.cols = dt.value, r.value, c.value

    @property
    def handle(self):
        return self._h

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def dtype(self):
        return _DT2NP[self.dtype_code]

    @staticmethod
    def from_numpy(ctx: Context, a: np.ndarray) -> "DenseMatrix":
        if a.ndim == 1:
            a = a.reshape(-1, 1)
        if a.ndim != 2 or a.dtype not in _NP2DT:
            raise Db2Error(1, f"unsupported array: ndim {a.ndim}, dtype {a.dtype}")
        if a.size and (a.strides[1] != a.itemsize or a.strides[0] % a.itemsize):
            a = np.ascontiguousarray(a)
        ld = a.strides[0] // a.itemsize if a.shape[0] > 1 and a.size else a.shape[1]
        ld = max(ld, a.shape[1])
        h = C.c_void_p()
        check(lib.db2_matrix_wrap_host(ctx.handle, _NP2DT[a.dtype], a.shape[0], a.shape[1], ld,
                                       C.c_void_p(a.ctypes.data), C.byref(h)))
        return DenseMatrix(ctx, h, keep=a)

    @staticmethod
    def empty(ctx: Context, rows: int, cols: int, dtype=np.float64, zero: bool = False) -> "DenseMatrix":
        h = C.c_void_p()
        check(lib.db2_matrix_create(ctx.handle, _NP2DT[np.dtype(dtype)], rows, cols, int(zero), C.byref(h)))
        return DenseMatrix(ctx, h)

    @staticmethod
    def wrap_device(ctx: Context, ptr: int, rows: int, cols: int, ld: int, dtype=np.float64, keep=None):
        h = C.c_void_p()
        check(lib.db2_matrix_wrap_device(ctx.handle, _NP2DT[np.dtype(dtype)], rows, cols, ld, C.c_void_p(ptr),
                                         C.byref(h)))
        return DenseMatrix(ctx, h, keep=keep)

    def slice_rows(self, r0: int, r1: int) -> "DenseMatrix":
        h = C.c_void_p()
        check(lib.db2_matrix_slice_rows(self._h, r0, r1, C.byref(h)))
        return DenseMatrix(self.ctx, h, keep=self._keep)

    def device_ptr(self):
        p, ld = C.c_void_p(), C.c_int64()
        check(lib.db2_matrix_device_ptr(self._h, C.byref(p), C.byref(ld)))
        return (p.value or 0), ld.value

    def to_numpy(self) -> np.ndarray:
        out = np.empty((self.rows, self.cols), dtype=self.dtype)
        check(lib.db2_matrix_to_host(self._h, C.c_void_p(out.ctypes.data), max(self.cols, 1)))
        return out

    def to_numpy_async(self, out: np.ndarray) -> np.ndarray:
        """Queues the copy into `out` (C-contiguous, same shape and value type; pinned memory for a true overlap) on the
        context's second stream and returns at once; Context.side_sync() waits for it."""
        if out.shape != (self.rows, self.cols) or out.dtype != self.dtype or not out.flags.c_contiguous:
            raise ValueError("to_numpy_async needs a C-contiguous array of the matrix's shape and value type")
        check(lib.db2_matrix_to_host_async(self._h, C.c_void_p(out.ctypes.data), max(self.cols, 1)))
        return out

    def free(self) -> None:
        if self._h:
            lib.db2_matrix_decref(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _res(ctx: Context, h) -> DenseMatrix:
    return DenseMatrix(ctx, h)


def _scalar(dtype_code: int, value):
    return np.array([value], dtype=_DT2NP[dtype_code])


def ewBinaryMat(op, lhs: DenseMatrix, rhs: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """EwBinaryMat.h:44-47: res = lhs op rhs, rhs may be a row or column vector."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_ewBinaryMat(ctx.handle, int(op), C.byref(h), lhs.handle, rhs.handle))
    return _res(ctx, h)


def ewBinaryObjSca(op, lhs: DenseMatrix, rhs, ctx: Optional[Context] = None) -> DenseMatrix:
    """EwBinaryObjSca.h:47-50: res = lhs op scalar."""
    ctx = ctx or lhs.ctx
    s = _scalar(lhs.dtype_code, rhs)
    h = C.c_void_p()
    check(lib.db2_ewBinaryObjSca(ctx.handle, int(op), C.byref(h), lhs.handle, C.c_void_p(s.ctypes.data)))
    return _res(ctx, h)


def ewUnaryMat(op, arg: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """EwUnaryMat.h:46-48."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_ewUnaryMat(ctx.handle, int(op), C.byref(h), arg.handle))
    return _res(ctx, h)


def aggRow(op, arg: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """AggRow.h:49-51: rows x 1 result; IDXMIN/IDXMAX give uint64 positions."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_aggRow(ctx.handle, int(op), C.byref(h), arg.handle))
    return _res(ctx, h)


def aggCol(op, arg: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """AggCol.h:47-49: 1 x cols result."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_aggCol(ctx.handle, int(op), C.byref(h), arg.handle))
    return _res(ctx, h)


def aggAll(op, arg: DenseMatrix, ctx: Optional[Context] = None):
    """AggAll.h:49-51: scalar result."""
    ctx = ctx or arg.ctx
    out = np.zeros(1, dtype=arg.dtype)
    check(lib.db2_aggAll(ctx.handle, int(op), C.c_void_p(out.ctypes.data), arg.handle))
    return out[0]


def aggAllStart(op, arg: DenseMatrix, slot: int = 0, ctx: Optional[Context] = None) -> None:
    """First half of aggAll (f64): queue the reduction; aggAllWait(slot) delivers the value.  What is queued on the
    context in between runs while the host waits."""
    ctx = ctx or arg.ctx
    check(lib.db2_aggAllStart(ctx.handle, int(op), arg.handle, int(slot)))


def scalarStart(m: DenseMatrix, slot: int = 0, ctx: Optional[Context] = None) -> None:
    """Queue the read of a 1 x 1 f64 matrix; aggAllWait(slot) delivers the value."""
    ctx = ctx or m.ctx
    check(lib.db2_scalarStart(ctx.handle, m.handle, int(slot)))


def aggAllWait(ctx: Context, slot: int = 0) -> float:
    out = C.c_double()
    check(lib.db2_scalarWait(ctx.handle, int(slot), C.byref(out)))
    return out.value


def matMul(lhs: DenseMatrix, rhs: DenseMatrix, transa: bool = False, transb: bool = False,
           ctx: Optional[Context] = None) -> DenseMatrix:
    """MatMul.h:44-47: res = op(lhs) @ op(rhs)."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_matMul(ctx.handle, C.byref(h), lhs.handle, rhs.handle, int(transa), int(transb)))
    return _res(ctx, h)


def syrk(arg: DenseMatrix, transLeft: bool = True, ctx: Optional[Context] = None) -> DenseMatrix:
    """Syrk.h:40-43: t(arg) @ arg if transLeft else arg @ t(arg); full symmetric result."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_syrk(ctx.handle, C.byref(h), arg.handle, int(transLeft)))
    return _res(ctx, h)


def gemv(mat: DenseMatrix, vec: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """Gemv.h:40-43: t(mat) @ vec (cols x 1)."""
    ctx = ctx or mat.ctx
    h = C.c_void_p()
    check(lib.db2_gemv(ctx.handle, C.byref(h), mat.handle, vec.handle))
    return _res(ctx, h)


def solve(lhs: DenseMatrix, rhs: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """Solve.h:40-43: x with lhs @ x = rhs (one right-hand side)."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_solve(ctx.handle, C.byref(h), lhs.handle, rhs.handle))
    return _res(ctx, h)


def transpose(arg: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_transpose(ctx.handle, C.byref(h), arg.handle))
    return _res(ctx, h)


def fill(ctx: Context, value, rows: int, cols: int, dtype=np.float64) -> DenseMatrix:
    v = np.array([value], dtype=dtype)
    h = C.c_void_p()
    check(lib.db2_fill(ctx.handle, C.byref(h), _NP2DT[np.dtype(dtype)], C.c_void_p(v.ctypes.data), rows, cols))
    return _res(ctx, h)


def seq(ctx: Context, start, end, inc, dtype=np.float64) -> DenseMatrix:
    """Seq.h:36-38."""
    a = np.array([start, end, inc], dtype=dtype)
    h = C.c_void_p()
    base = a.ctypes.data
    check(lib.db2_seq(ctx.handle, C.byref(h), _NP2DT[np.dtype(dtype)], C.c_void_p(base), C.c_void_p(base + 8),
                      C.c_void_p(base + 16)))
    return _res(ctx, h)


def diagMatrix(arg: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_diagMatrix(ctx.handle, C.byref(h), arg.handle))
    return _res(ctx, h)


def outerBinary(op, lhs: DenseMatrix, rhs: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """OuterBinary.h:41-44: res[r][c] = lhs[r] (op) rhs[c] for a column vector lhs and a row vector rhs."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_outerBinary(ctx.handle, int(op), C.byref(h), lhs.handle, rhs.handle))
    return _res(ctx, h)


def cond(cnd: DenseMatrix, then, els, dtype=None, ctx: Optional[Context] = None) -> DenseMatrix:
    """CondMatMatMat.h / CondMatMatSca.h / CondMatScaMat.h / CondMatScaSca.h: cnd ? then : els element by element;
    `then` and `els` are matrices of the shape of cnd or scalars (dtype names the value type when both are scalars)."""
    ctx = ctx or cnd.ctx
    mats = [x for x in (then, els) if isinstance(x, DenseMatrix)]
    dt = np.dtype(mats[0].dtype if mats else (dtype or np.float64))
    tm = then.handle if isinstance(then, DenseMatrix) else None
    em = els.handle if isinstance(els, DenseMatrix) else None
    ts = np.array([0 if tm else then], dtype=dt)
    es = np.array([0 if em else els], dtype=dt)
    h = C.c_void_p()
    check(lib.db2_cond(ctx.handle, C.byref(h), _NP2DT[dt], cnd.handle, tm, C.c_void_p(ts.ctypes.data), em,
                       C.c_void_p(es.ctypes.data)))
    return _res(ctx, h)


def aggCum(op, arg: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """AggCum.h:39-42: cumulative SUM / PROD / MIN / MAX down the rows of every column."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_aggCum(ctx.handle, int(op), C.byref(h), arg.handle))
    return _res(ctx, h)


def oneHot(arg: DenseMatrix, info: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """OneHot.h:43-46: info (1 x cols, int64) says per column: -1 keep, 0 drop, k > 0 expand into k indicators."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_oneHot(ctx.handle, C.byref(h), arg.handle, info.handle))
    return _res(ctx, h)


def colBind(lhs: DenseMatrix, rhs: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """ColBind.h:41-44: [lhs | rhs]."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_colBind(ctx.handle, C.byref(h), lhs.handle, rhs.handle))
    return _res(ctx, h)


def extractCol(arg: DenseMatrix, sel: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """ExtractCol.h:45-48: the columns of arg at the positions in the int64 column matrix sel."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_extractCol(ctx.handle, C.byref(h), arg.handle, sel.handle))
    return _res(ctx, h)


def rtc_set_mode(mode: int) -> None:
    """Kernels for elementwise chains without a compiled-in specialisation: 0 = never compile one, 2 = compile on the
    calling thread when the chain is first evaluated (default), 1 = compile on a background thread (call rtc_wait()
    before the process ends)."""
    check(lib.db2_rtc_set_mode(int(mode)))


def rtc_wait() -> None:
    check(lib.db2_rtc_wait())


def rtc_counts() -> dict:
    """Chains with a compiled kernel / being compiled / whose compilation failed."""
    r, p, f = C.c_int(), C.c_int(), C.c_int()
    check(lib.db2_rtc_counts(C.byref(r), C.byref(p), C.byref(f)))
    return {"ready": r.value, "pending": p.value, "failed": f.value}


def readDaphne(ctx: Context, path) -> DenseMatrix:
    """ReadDaphne.h:44-46: a dense matrix from a .dbdf file, streamed straight into its device placement."""
    h = C.c_void_p()
    check(lib.db2_readDaphne(ctx.handle, C.byref(h), str(path).encode()))
    return _res(ctx, h)


def writeDaphne(arg: DenseMatrix, path, ctx: Optional[Context] = None) -> None:
    """WriteDaphne.h:48-50."""
    ctx = ctx or arg.ctx
    check(lib.db2_writeDaphne(ctx.handle, arg.handle, str(path).encode()))


def sliceRow(arg: DenseMatrix, lowerIncl: int, upperExcl: int, ctx: Optional[Context] = None) -> DenseMatrix:
    """SliceRow.h:45-82: rows [lowerIncl, upperExcl) as a zero-copy view; negative bounds count from the end."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_sliceRow(ctx.handle, C.byref(h), arg.handle, int(lowerIncl), int(upperExcl)))
    return DenseMatrix(ctx, h, keep=arg)


def sliceCol(arg: DenseMatrix, lowerIncl: int, upperExcl: int, ctx: Optional[Context] = None) -> DenseMatrix:
    """SliceCol.h:52-86: columns [lowerIncl, upperExcl) as a zero-copy view."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_sliceCol(ctx.handle, C.byref(h), arg.handle, int(lowerIncl), int(upperExcl)))
    return DenseMatrix(ctx, h, keep=arg)


def randMatrix(ctx: Context, rows: int, cols: int, lo, hi, sparsity: float = 1.0, seed: int = -1,
               dtype=np.float64) -> DenseMatrix:
    """RandMatrix.h:82-161 = DaphneDSL rand(rows, cols, lo, hi, sparsity, seed), device-resident."""
    dt = np.dtype(dtype)
    a, b = np.array([lo], dtype=dt), np.array([hi], dtype=dt)
    h = C.c_void_p()
    check(lib.db2_randMatrix(ctx.handle, C.byref(h), _NP2DT[dt], int(rows), int(cols), C.c_void_p(a.ctypes.data),
                             C.c_void_p(b.ctypes.data), float(sparsity), int(seed)))
    return DenseMatrix(ctx, h)


def ctable(lhs: DenseMatrix, rhs: DenseMatrix, weight: float = 1.0, resNumRows: int = -1, resNumCols: int = -1,
           ctx: Optional[Context] = None) -> DenseMatrix:
    """CTable.h:44-48: res[lhs[i], rhs[i]] += weight."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_ctable(ctx.handle, C.byref(h), lhs.handle, rhs.handle, float(weight), resNumRows, resNumCols))
    return _res(ctx, h)


def castObj(arg: DenseMatrix, dtype, ctx: Optional[Context] = None) -> DenseMatrix:
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_castObj(ctx.handle, C.byref(h), arg.handle, _NP2DT[np.dtype(dtype)]))
    return _res(ctx, h)


class CSRMatrix:
    """Handle to a db2_csr.  The host arrays follow the reference's CSRMatrix layout (values, colIdxs and rowOffsets
    with 64-bit indices)."""

    def __init__(self, ctx: Context, handle, keep=None):
        self.ctx, self._h, self._keep = ctx, handle, keep
        r, c = C.c_int64(), C.c_int64()
        check(lib.db2_csr_info(self._h, C.byref(r), C.byref(c), None))
        self.rows, self.cols = r.value, c.value

    @property
    def handle(self):
        return self._h

    @property
    def shape(self):
        return (self.rows, self.cols)

    @staticmethod
    def from_arrays(ctx: Context, rows: int, cols: int, values, col_idx, row_off) -> "CSRMatrix":
        values = np.ascontiguousarray(values, dtype=np.float64)
        col_idx = np.ascontiguousarray(col_idx, dtype=np.uint64)
        row_off = np.ascontiguousarray(row_off, dtype=np.uint64)
        h = C.c_void_p()
        check(lib.db2_csr_wrap_host(ctx.handle, _l.F64, rows, cols, C.c_void_p(values.ctypes.data),
                                    C.c_void_p(col_idx.ctypes.data), C.c_void_p(row_off.ctypes.data), C.byref(h)))
        return CSRMatrix(ctx, h, keep=(values, col_idx, row_off))

    @staticmethod
    def from_scipy(ctx: Context, m) -> "CSRMatrix":
        m = m.tocsr()
        m.sort_indices()
        return CSRMatrix.from_arrays(ctx, m.shape[0], m.shape[1], m.data, m.indices, m.indptr)

    def nnz(self) -> int:
        n = C.c_int64()
        check(lib.db2_csr_info(self._h, None, None, C.byref(n)))
        return n.value

    def slice_rows(self, r0: int, r1: int) -> "CSRMatrix":
        h = C.c_void_p()
        check(lib.db2_csr_slice_rows(self._h, r0, r1, C.byref(h)))
        return CSRMatrix(self.ctx, h, keep=self._keep)

    def to_arrays(self):
        n = self.nnz()
        vals, cols, offs = np.empty(n), np.empty(n, dtype=np.uint64), np.empty(self.rows + 1, dtype=np.uint64)
        check(lib.db2_csr_to_host(self._h, C.c_void_p(vals.ctypes.data), C.c_void_p(cols.ctypes.data),
                                  C.c_void_p(offs.ctypes.data)))
        return vals, cols, offs

    def free(self):
        if self._h:
            lib.db2_csr_decref(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def ewMulCsrDense(lhs: CSRMatrix, rhs: DenseMatrix, ctx: Optional[Context] = None) -> CSRMatrix:
    """EwBinaryMat<CSR,CSR,Dense> with MUL (EwBinaryMat.h:254-317)."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_ewMulCsrDense(ctx.handle, C.byref(h), lhs.handle, rhs.handle))
    return CSRMatrix(ctx, h, keep=(lhs, rhs))


def aggRowCsr(op, arg: CSRMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """AggRow<Dense,CSR> (AggRow.h:178-238)."""
    ctx = ctx or arg.ctx
    h = C.c_void_p()
    check(lib.db2_aggRowCsr(ctx.handle, int(op), C.byref(h), arg.handle))
    return _res(ctx, h)


def matMulCsrDense(lhs: CSRMatrix, rhs: DenseMatrix, ctx: Optional[Context] = None) -> DenseMatrix:
    """Gemv<Dense,CSR,Dense> / MatMul<Dense,CSR,Dense>."""
    ctx = ctx or lhs.ctx
    h = C.c_void_p()
    check(lib.db2_matMulCsrDense(ctx.handle, C.byref(h), lhs.handle, rhs.handle))
    return _res(ctx, h)


PIPELINE_FN = C.CFUNCTYPE(None, C.POINTER(C.POINTER(C.c_void_p)), C.POINTER(C.c_void_p), C.c_void_p)


def vectorizedPipeline(ctx: Context, inputs, splits, combines, body, batch_rows: int = 0):
    """VectorizedPipeline.h:35-69.  `body(ins) -> outs` receives DenseMatrix handles for the (row slices of the)
    inputs and returns one DenseMatrix per output; like the compiled body of the reference it owns its inputs (they
    are released when the handles go out of scope) and hands its results over to the scheduler."""
    n_in, n_out = len(inputs), len(combines)
    keep = []

    def trampoline(outs_pp, ins_p, _ctx):
        ins = [DenseMatrix(ctx, C.c_void_p(ins_p[i])) for i in range(n_in)]
        outs = body(ins)
        assert len(outs) == n_out
        for o, m in enumerate(outs):
            outs_pp[o][0] = m.handle.value
            m._h = C.c_void_p()  # ownership moves to the scheduler
        for m in ins:
            m.free()
        keep.append(outs)

    cb = PIPELINE_FN(trampoline)
    out_h = (C.c_void_p * n_out)()
    in_h = (C.c_void_p * n_in)(*[m.handle.value for m in inputs])
    sp = (C.c_int64 * n_in)(*[int(x) for x in splits])
    cm = (C.c_int64 * n_out)(*[int(x) for x in combines])
    neg = (C.c_int64 * n_out)(*([-1] * n_out))
    scal = (C.c_int * n_in)(*([0] * n_in))
    check(lib.db2_vectorizedPipeline(ctx.handle, out_h, n_out, scal, in_h, n_in, neg, neg, sp, cm,
                                     C.cast(cb, C.c_void_p), int(batch_rows)))
    return [DenseMatrix(ctx, C.c_void_p(out_h[o])) for o in range(n_out)]


class Group:
    """Several GPUs in one process (db2_group): one Context per device.  devices=None takes DAPHNE_B200_DEVICES or all
    visible devices; a device may be listed more than once."""

    def __init__(self, devices=None):
        self._h = C.c_void_p()
        if devices is None:
            check(lib.db2_group_create(None, 0, C.byref(self._h)))
        else:
            arr = (C.c_int * len(devices))(*[int(d) for d in devices])
            check(lib.db2_group_create(arr, len(devices), C.byref(self._h)))
        n = C.c_int()
        check(lib.db2_group_size(self._h, C.byref(n)))
        self.size = n.value
        self.contexts = []
        for i in range(self.size):
            h = C.c_void_p()
            check(lib.db2_group_context(self._h, i, C.byref(h)))
            c = Context.__new__(Context)  # borrowed: the group owns the context
            c._h, c._borrowed = h, True
            dev = C.c_int()
            check(lib.db2_context_device(h, C.byref(dev)))
            c.device = dev.value
            c.close = lambda: None
            self.contexts.append(c)

    @property
    def handle(self):
        return self._h

    @property
    def uses_nccl(self) -> bool:
        y = C.c_int()
        check(lib.db2_group_uses_nccl(self._h, C.byref(y)))
        return bool(y.value)

    def sync(self) -> None:
        check(lib.db2_group_sync(self._h))

    def close(self) -> None:
        if self._h:
            lib.db2_group_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class DistMatrix:
    """Handle to a db2_dist: row blocks (axis 0), column blocks (axis 1) or one copy per device (axis -1)."""

    def __init__(self, group: Group, handle, keep=None):
        self.group, self._h, self._keep = group, handle, keep
        dt, r, c, ax = C.c_int(), C.c_int64(), C.c_int64(), C.c_int()
        check(lib.db2_dist_info(self._h, C.byref(dt), C.byref(r), C.byref(c), C.byref(ax)))
        self.dtype_code, self.rows, self.cols, self.axis = dt.value, r.value, c.value, ax.value

    @property
    def handle(self):
        return self._h

    @property
    def shape(self):
        return (self.rows, self.cols)

    @staticmethod
    def from_numpy(group: Group, a: np.ndarray) -> "DistMatrix":
        """Row blocks of a host array (borrowed): each device fetches its own rows on first use."""
        if a.ndim == 1:
            a = a.reshape(-1, 1)
        if a.ndim != 2 or a.dtype not in _NP2DT:
            raise Db2Error(1, f"unsupported array: ndim {a.ndim}, dtype {a.dtype}")
        if a.size and (a.strides[1] != a.itemsize or a.strides[0] % a.itemsize):
            a = np.ascontiguousarray(a)
        ld = max(a.strides[0] // a.itemsize if a.shape[0] > 1 and a.size else a.shape[1], a.shape[1])
        h = C.c_void_p()
        check(lib.db2_dist_from_host(group.handle, _NP2DT[a.dtype], a.shape[0], a.shape[1], ld,
                                     C.c_void_p(a.ctypes.data), C.byref(h)))
        return DistMatrix(group, h, keep=a)

    @staticmethod
    def from_matrix(group: Group, m: DenseMatrix, replicate: bool = False) -> "DistMatrix":
        h = C.c_void_p()
        check(lib.db2_dist_from_matrix(group.handle, m.handle, int(replicate), C.byref(h)))
        return DistMatrix(group, h, keep=m)

    def shard(self, i: int):
        """(DenseMatrix, first row / column) of device i's block."""
        h, off = C.c_void_p(), C.c_int64()
        check(lib.db2_dist_shard(self._h, i, C.byref(h), C.byref(off)))
        check(lib.db2_matrix_incref(h))
        return DenseMatrix(self.group.contexts[i], h, keep=self), off.value

    def to_numpy(self) -> np.ndarray:
        out = np.empty((self.rows, self.cols), dtype=_DT2NP[self.dtype_code])
        check(lib.db2_dist_to_host(self._h, C.c_void_p(out.ctypes.data), max(self.cols, 1)))
        return out

    def gather(self, index: int = 0) -> DenseMatrix:
        h = C.c_void_p()
        check(lib.db2_dist_gather(self._h, index, C.byref(h)))
        return DenseMatrix(self.group.contexts[index], h)

    def free(self) -> None:
        if self._h:
            lib.db2_dist_decref(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def vectorizedPipelineGroup(group: Group, inputs, splits, combines, body, batch_rows: int = 0):
    """The scheduler over all devices of a group (db2_vectorizedPipelineGroup).  `body(ins, ctx) -> outs` is called
    once per device (and batch), from that device's host thread, with that device's Context."""
    n_in, n_out = len(inputs), len(combines)
    by_ptr = {c.handle.value: c for c in group.contexts}
    keep, errors = [], []

    def trampoline(outs_pp, ins_p, ctx_p):
        try:
            ctx = by_ptr[ctx_p]
            ins = [DenseMatrix(ctx, C.c_void_p(ins_p[i])) for i in range(n_in)]
            outs = body(ins, ctx)
            assert len(outs) == n_out
            for o, m in enumerate(outs):
                outs_pp[o][0] = m.handle.value
                m._h = C.c_void_p()  # ownership moves to the scheduler
            for m in ins:
                m.free()
            keep.append(outs)
        except BaseException as e:  # an exception must not unwind through the C frames of the worker thread
            errors.append(e)

    cb = PIPELINE_FN(trampoline)
    out_h = (C.c_void_p * n_out)()
    in_h = (C.c_void_p * n_in)(*[m.handle.value for m in inputs])
    sp = (C.c_int64 * n_in)(*[int(x) for x in splits])
    cm = (C.c_int64 * n_out)(*[int(x) for x in combines])
    neg = (C.c_int64 * n_out)(*([-1] * n_out))
    scal = (C.c_int * n_in)(*([0] * n_in))
    rc = lib.db2_vectorizedPipelineGroup(group.handle, out_h, n_out, scal, in_h, n_in, neg, neg, sp, cm,
                                         C.cast(cb, C.c_void_p), int(batch_rows))
    if errors:
        raise errors[0]
    check(rc)
    return [DistMatrix(group, C.c_void_p(out_h[o])) for o in range(n_out)]
