"""Known-answer cases of the reference's own unit tests (tests/golden/reference_cases.json, extracted from
test/runtime/local/kernels/*Test.cpp by tests/golden/extract_reference_cases.py), run against the CPU oracle (always)
and against the CUDA library (on a GPU).  Tolerances are the ones the reference's tests use: exact for elementwise
results, matMul, syrk, ctable, seq, diagMatrix and transpose (small integer-valued literals, `*res == *exp`), 1e-5 absolute for
aggregations (checkEqApprox in AggRowTest.cpp:38), 1e-2 for the *Approx unary checks (EwUnaryMatTest.cpp:48), 1e-6
for solve (SolveTest.cpp:39)."""
import json
from pathlib import Path

import numpy as np
import pytest

CASES = json.loads((Path(__file__).parent / "golden" / "reference_cases.json").read_text())["cases"]

BIN = {n: i for i, n in enumerate(["ADD", "SUB", "MUL", "DIV", "POW", "MOD", "LOG", "EQ", "NEQ", "LT", "LE", "GT", "GE",
                                   "MIN", "MAX", "AND", "OR", "BITWISE_AND"])}
UN = {n: i for i, n in enumerate(["MINUS", "ABS", "SIGN", "SQRT", "EXP", "LN", "SIN", "COS", "TAN", "ASIN", "ACOS",
                                  "ATAN", "SINH", "COSH", "TANH", "FLOOR", "CEIL", "ROUND", "ISNAN"])}
AGG = {n: i for i, n in enumerate(["SUM", "PROD", "MIN", "MAX", "IDXMIN", "IDXMAX", "MEAN", "STDDEV", "VAR"])}

DENSE_CHECKS = {"checkAggRow", "checkAggCol", "checkAggAll", "checkEwBinaryMat", "checkEwUnaryMat",
                "checkEwUnaryMatApprox", "checkEwUnaryMatThrow", "checkEwBinaryObjSca", "checkMatMul", "checkSyrk",
                "solveNormalEquations", "ctableSection", "transposeSection", "checkSeq", "checkDiagMatrix", "colBind", "extractCol", "extractColThrow", "outerBinary", "aggCum", "oneHot", "oneHotThrow", "cond", "sliceRow", "sliceRowThrow", "sliceCol", "sliceColThrow"}


def _num(v):
    return {"nan": np.nan, "inf": np.inf, "-inf": -np.inf}.get(v, v) if isinstance(v, str) else v


def _mat(arg):
    vals = np.array([_num(v) for v in arg["values"]], dtype=np.float64)
    rows = arg["rows"]
    return vals.reshape(rows, -1) if rows else vals.reshape(0, 0)


def _dense_cases():
    out = []
    for c in CASES:
        if c["check"] not in DENSE_CHECKS:
            continue
        if c["check"] == "cond":
            out.append(pytest.param(c, id=f"{Path(c['file']).stem}:{c['line']}:{c['op']}"))
            continue
        if c["op"] in ("CONCAT", "UPPER", "LOWER"):
            continue  # string kernels are outside the numeric hot path
        if any("matrix" in a and not a["values"] for a in c["args"]):
            continue
        if c["check"] == "checkEwBinaryObjSca" and (len(c["args"]) != 3 or "scalar" not in c["args"][1]):
            continue  # frame / string variants
        out.append(pytest.param(c, id=f"{Path(c['file']).stem}:{c['line']}:{c['op']}"))
    return out


class _OracleBackend:
    name = "oracle"
    dtypes = (np.float64,)  # the oracle restates the double-precision contractions only

    def __init__(self):
        from oracle import pyoracle as o
        self.o = o
        self.err = o.OracleError

    def binary(self, op, a, b): return self.o.ewBinaryMat(op, a, b)
    def unary(self, op, a): return self.o.ewUnaryMat(op, a)
    def agg_row(self, op, a): return self.o.aggRow(op, a)
    def agg_col(self, op, a): return self.o.aggCol(op, a)
    def agg_all(self, op, a): return self.o.aggAll(op, a)
    def binary_sca(self, op, a, s): return self.o.ewBinaryObjSca(op, a, s)
    def matmul(self, a, b, ta, tb): return self.o.matMul(a, b, ta, tb)
    def syrk(self, a, tl): return self.o.syrk(a, tl)
    def transpose(self, a): return self.o.transpose(a)
    def solve(self, a, b): return self.o.solve(a, b)
    def ctable(self, ys, xs, w, nr, nc): return self.o.ctable(ys, xs, w, nr, nc)
    def seq(self, start, end, inc): return self.o.seq(start, end, inc)
    def col_bind(self, a, b): return self.o.colBind(a, b)
    def outer(self, op, a, b): return self.o.outerBinary(op, a, b)
    def agg_cum(self, op, a): return self.o.aggCum(op, a)
    def one_hot(self, a, info): return self.o.oneHot(a, info)
    def extract_col(self, a, sel): return self.o.extractCol(a, sel)
    def cond(self, c, t, e, dt): return self.o.cond(c, t, e, dtype=dt)
    def slice_row(self, a, lo, up): return self.o.sliceRow(a, lo, up)
    def slice_col(self, a, lo, up): return self.o.sliceCol(a, lo, up)
    diag = None  # DiagMatrix has no restatement in the oracle: a diagonal copy, checked on the device only


class _CudaBackend:
    name = "cuda"
    dtypes = (np.float64, np.float32)  # MatMulTest / SyrkTest are instantiated for float and double

    def __init__(self, ctx):
        import daphne_b200.kernels as k
        self.k, self.ctx, self.err = k, ctx, k.Db2Error

    def _m(self, a): return self.k.DenseMatrix.from_numpy(self.ctx, np.ascontiguousarray(a))
    def binary(self, op, a, b): return self.k.ewBinaryMat(op, self._m(a), self._m(b)).to_numpy()
    def unary(self, op, a): return self.k.ewUnaryMat(op, self._m(a)).to_numpy()
    def agg_row(self, op, a): return self.k.aggRow(op, self._m(a)).to_numpy()
    def agg_col(self, op, a): return self.k.aggCol(op, self._m(a)).to_numpy()
    def agg_all(self, op, a): return self.k.aggAll(op, self._m(a))
    def binary_sca(self, op, a, s): return self.k.ewBinaryObjSca(op, self._m(a), s).to_numpy()
    def matmul(self, a, b, ta, tb): return self.k.matMul(self._m(a), self._m(b), ta, tb).to_numpy()
    def syrk(self, a, tl): return self.k.syrk(self._m(a), tl).to_numpy()
    def transpose(self, a): return self.k.transpose(self._m(a)).to_numpy()
    def solve(self, a, b): return self.k.solve(self._m(a), self._m(b)).to_numpy()

    def ctable(self, ys, xs, w, nr, nc):
        return self.k.ctable(self._m(ys.astype(np.int64)), self._m(xs.astype(np.int64)), w, nr, nc).to_numpy()

    def seq(self, start, end, inc): return self.k.seq(self.ctx, start, end, inc).to_numpy()
    def col_bind(self, a, b): return self.k.colBind(self._m(a), self._m(b)).to_numpy()
    def outer(self, op, a, b): return self.k.outerBinary(op, self._m(a), self._m(b)).to_numpy()
    def agg_cum(self, op, a): return self.k.aggCum(op, self._m(a)).to_numpy()
    def one_hot(self, a, info): return self.k.oneHot(self._m(a), self._m(info)).to_numpy()
    def extract_col(self, a, sel): return self.k.extractCol(self._m(a), self._m(sel)).to_numpy()
    def diag(self, a): return self.k.diagMatrix(self._m(a)).to_numpy()
    def slice_row(self, a, lo, up): return self.k.sliceRow(self._m(a), lo, up).to_numpy()
    def slice_col(self, a, lo, up): return self.k.sliceCol(self._m(a), lo, up).to_numpy()

    def cond(self, c, t, e, dt):
        t, e = (self._m(x) if isinstance(x, np.ndarray) else x for x in (t, e))
        return self.k.cond(self._m(c), t, e, dtype=dt).to_numpy()


def _run_case(be, c):
    chk, op, args = c["check"], c["op"], c["args"]
    if chk == "checkEwBinaryMat":
        lhs, rhs, exp = (_mat(a) for a in args)
        got = be.binary(BIN[op], lhs, rhs)
        assert np.array_equal(got, exp, equal_nan=True), f"{c['file']}:{c['line']}"
    elif chk == "checkEwUnaryMat":
        arg, exp = (_mat(a) for a in args)
        assert np.array_equal(be.unary(UN[op], arg), exp, equal_nan=True), f"{c['file']}:{c['line']}"
    elif chk == "checkEwUnaryMatApprox":
        arg, exp = (_mat(a) for a in args)
        np.testing.assert_allclose(be.unary(UN[op], arg), exp, atol=1e-2, rtol=0, equal_nan=True)
    elif chk == "checkEwUnaryMatThrow":
        with pytest.raises(be.err):
            be.unary(UN[op], _mat(args[0]))
    elif chk in ("checkAggRow", "checkAggCol"):
        arg, exp = (_mat(a) for a in args)
        f = be.agg_row if chk == "checkAggRow" else be.agg_col
        got = f(AGG[op], arg).astype(np.float64)
        np.testing.assert_allclose(got.reshape(-1), exp.reshape(-1), atol=1e-5, rtol=0)
    elif chk == "checkAggAll":
        arg, exp = _mat(args[0]), _num(args[1]["scalar"])
        got = float(be.agg_all(AGG[op], arg))
        assert abs(got - exp) <= 1e-5 * max(1.0, abs(exp)), f"{c['file']}:{c['line']}: {got} vs {exp}"
    elif chk == "checkEwBinaryObjSca":
        arg, sca, exp = _mat(args[0]), float(_num(args[1]["scalar"])), _mat(args[2])
        assert np.array_equal(be.binary_sca(BIN[op], arg, sca), exp, equal_nan=True), f"{c['file']}:{c['line']}"
    elif chk == "checkMatMul":
        lhs, rhs, exp = (_mat(a) for a in args[:3])
        flags = [bool(_num(a["scalar"])) for a in args[3:]] + [False, False]
        for dt in be.dtypes:
            got = be.matmul(lhs.astype(dt), rhs.astype(dt), flags[0], flags[1])
            assert got.dtype == dt and np.array_equal(got, exp.astype(dt)), f"{c['file']}:{c['line']} {dt.__name__}"
    elif chk == "checkSyrk":  # syrk against transpose followed by matMul, both orientations (SyrkTest.cpp:32-58)
        arg = _mat(args[0])
        for dt in be.dtypes:
            a = arg.astype(dt)
            assert np.array_equal(be.syrk(a, True), be.matmul(be.transpose(a), a, False, False))
            assert np.array_equal(be.syrk(a, False), be.matmul(a, be.transpose(a), False, False))
            assert np.array_equal(be.syrk(a, True), (arg.T @ arg).astype(dt))
    elif chk == "solveNormalEquations":  # SolveTest.cpp:43-60
        X, w = _mat(args[0]), _mat(args[1])
        y = be.matmul(X, w, False, False)
        tX = be.transpose(X)
        A, b = be.matmul(tX, X, False, False), be.matmul(tX, y, False, False)
        got = be.solve(A, b)
        assert got.shape == w.shape
        np.testing.assert_allclose(got, w, atol=1e-6, rtol=0)
    elif chk == "ctableSection":
        ys, xs, exp = _mat(args[0]), _mat(args[1]), _mat(args[5])
        w, nr, nc = (_num(a["scalar"]) for a in args[2:5])
        got = be.ctable(ys.reshape(-1, 1), xs.reshape(-1, 1), float(w), int(nr), int(nc))
        assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk == "checkSeq":  # SeqTest.cpp:26-29: a column vector start, start + inc, ..., end
        start, end, inc = (float(_num(a["scalar"])) for a in args[:3])
        exp = _mat(args[3])
        got = np.asarray(be.seq(start, end, inc), dtype=np.float64)
        assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk == "checkDiagMatrix":  # DiagMatrixTest.cpp:30-35
        if be.diag is not None:
            arg, exp = _mat(args[0]), _mat(args[1])
            got = be.diag(arg)
            assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk in ("oneHot", "oneHotThrow"):  # OneHotTest.cpp:29-89, the double instantiation
        arg = _mat(args[0])
        info = np.array([_num(v) for v in args[1]["values"]], dtype=np.int64).reshape(args[1]["rows"], -1)
        if chk == "oneHotThrow":
            with pytest.raises(be.err):
                be.one_hot(arg, info)
        else:
            exp = _mat(args[2])
            got = be.one_hot(arg, info)
            assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk == "aggCum":  # AggCumTest.cpp:33-37 (small integer-valued literals: exact)
        arg, exp = (_mat(a) for a in args)
        got = be.agg_cum(AGG[op], arg)
        assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk == "outerBinary":  # OuterBinaryTest.cpp:39-60
        lhs, rhs, exp = (_mat(a) for a in args)
        got = be.outer(BIN[op], lhs, rhs)
        assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk == "colBind":  # ColBindTest.cpp:62-64
        lhs, rhs, exp = (_mat(a) for a in args)
        got = be.col_bind(lhs, rhs)
        assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk in ("extractCol", "extractColThrow"):  # ExtractColTest.cpp:36-44
        arg = _mat(args[0])
        sel = np.array([_num(v) for v in args[1]["values"]], dtype=np.int64).reshape(-1, 1)
        if chk == "extractColThrow":
            with pytest.raises(be.err):
                be.extract_col(arg, sel)
        else:
            exp = np.array([_num(v) for v in args[2]["values"]], dtype=np.float64).reshape(args[2]["rows"], -1)
            got = be.extract_col(arg, sel)
            assert got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk == "cond":  # CondMatMatMatTest.cpp:35-52 and its three siblings; op names the value type
        dt = np.float64 if op == "double" else np.int64
        cnd = _mat(args[0]).astype(dt)
        then, els = (dt(_num(a["scalar"])) if "scalar" in a else _mat(a).astype(dt) for a in args[1:3])
        exp = _mat(args[3]).astype(dt)
        got = be.cond(cnd, then, els, dt)
        assert got.dtype == dt and got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk in ("sliceRow", "sliceCol", "sliceRowThrow", "sliceColThrow"):  # SliceRowTest.cpp:31-82, SliceColTest.cpp
        arg = _mat(args[0])
        lo, up = (int(_num(a["scalar"])) for a in args[1:3])
        f = be.slice_row if chk.startswith("sliceRow") else be.slice_col
        for dt in (np.float64, np.int64, np.uint32):
            if chk.endswith("Throw"):
                with pytest.raises(be.err):
                    f(arg.astype(dt), lo, up)
            else:
                exp = _mat(args[3]).astype(dt)
                got = f(arg.astype(dt), lo, up)
                assert got.dtype == dt and got.shape == exp.shape and np.array_equal(got, exp), f"{c['file']}:{c['line']}"
    elif chk == "transposeSection":
        m, mt = _mat(args[0]), _mat(args[1])
        assert np.array_equal(be.transpose(m), mt), f"{c['file']}:{c['line']}"
    else:
        raise AssertionError(chk)


def test_fixture_is_not_trivial():
    assert len(_dense_cases()) >= 146


@pytest.mark.parametrize("case", _dense_cases())
def test_oracle_reproduces_reference_known_answers(case):
    _run_case(_OracleBackend(), case)


@pytest.mark.gpu
@pytest.mark.parametrize("case", _dense_cases())
def test_cuda_reproduces_reference_known_answers(ctx, case):
    _run_case(_CudaBackend(ctx), case)
