"""TEST INFRASTRUCTURE: a numpy/oracle stand-in with the interface of daphne_b200.kernels, used to exercise the
HOST-side sharding and combine logic of daphne_b200.pipelines / daphne_b200.dist on CPU ranks (gloo).  It is never
used by the product."""
import numpy as np

from daphne_b200.kernels import AggOpCode, BinaryOpCode, UnaryOpCode  # noqa: F401  (enums only)
from oracle import pyoracle as o


class DenseMatrix:
    def __init__(self, a):
        self.a = np.ascontiguousarray(a)
        self.rows, self.cols = self.a.shape

    @staticmethod
    def from_numpy(ctx, a):
        a = np.asarray(a)
        return DenseMatrix(a.reshape(-1, 1) if a.ndim == 1 else a)

    def to_numpy(self):
        return self.a

    def slice_rows(self, lo, hi):
        return DenseMatrix(self.a[lo:hi])

    def free(self):
        pass

    def device_ptr(self):
        return 0, self.cols


class CSRMatrix:
    def __init__(self, m):
        self.m = m
        self.rows, self.cols = m.shape


def _w(x):
    return DenseMatrix(x)


def ewBinaryMat(op, a, b): return _w(o.ewBinaryMat(op, a.a, b.a))
def ewBinaryObjSca(op, a, s): return _w(o.ewBinaryObjSca(op, a.a, s))
def ewUnaryMat(op, a): return _w(o.ewUnaryMat(op, a.a))
def aggRow(op, a): return _w(o.aggRow(op, a.a))
def aggCol(op, a): return _w(o.aggCol(op, a.a))
def aggAll(op, a): return o.aggAll(op, a.a)
def matMul(a, b, ta=False, tb=False): return _w(o.matMul(a.a, b.a, ta, tb))
def syrk(a, tl=True): return _w(o.syrk(a.a, tl))
def gemv(a, v): return _w(o.gemv(a.a, v.a))
def solve(a, b): return _w(o.solve(a.a, b.a))
def transpose(a): return _w(o.transpose(a.a))
def fill(ctx, v, r, c, dtype=np.float64): return _w(np.full((r, c), v, dtype=dtype))
def diagMatrix(a): return _w(np.diag(a.a[:, 0]))
def castObj(a, dtype): return _w(a.a.astype(dtype))
def ctable(l, r, w=1.0, rows=-1, cols=-1): return _w(o.ctable(l.a, r.a, w, rows, cols))
def ewMulCsrDense(g, d): return ("prod", g, d)
def aggRowCsr(op, p): return _w(o.aggRowCsr(op, o.ewMulCsrDense(p[1].m, p[2].a)))


def seq(ctx, start, end, inc, dtype=np.float64):
    return _w(o.seq(start, end, inc).astype(dtype))
