"""Known-answer cases of the reference's own unit tests (tests/golden/reference_cases.json, extracted from
test/runtime/local/kernels/*Test.cpp by tests/golden/extract_reference_cases.py), run against the CPU oracle (always)
and against the CUDA library (on a GPU).  Tolerances are the ones the reference's tests use: exact for elementwise
results, 1e-5 absolute for aggregations (checkEqApprox in AggRowTest.cpp:38), 1e-2 for the *Approx unary checks
(EwUnaryMatTest.cpp:48)."""
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
                "checkEwUnaryMatApprox", "checkEwUnaryMatThrow"}


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
        if c["op"] in ("CONCAT", "UPPER", "LOWER"):
            continue  # string kernels are outside the numeric hot path
        if any("matrix" in a and not a["values"] for a in c["args"]):
            continue
        out.append(pytest.param(c, id=f"{Path(c['file']).stem}:{c['line']}:{c['op']}"))
    return out


class _OracleBackend:
    name = "oracle"

    def __init__(self):
        from oracle import pyoracle as o
        self.o = o
        self.err = o.OracleError

    def binary(self, op, a, b): return self.o.ewBinaryMat(op, a, b)
    def unary(self, op, a): return self.o.ewUnaryMat(op, a)
    def agg_row(self, op, a): return self.o.aggRow(op, a)
    def agg_col(self, op, a): return self.o.aggCol(op, a)
    def agg_all(self, op, a): return self.o.aggAll(op, a)


class _CudaBackend:
    name = "cuda"

    def __init__(self, ctx):
        import daphne_b200.kernels as k
        self.k, self.ctx, self.err = k, ctx, k.Db2Error

    def _m(self, a): return self.k.DenseMatrix.from_numpy(self.ctx, np.ascontiguousarray(a))
    def binary(self, op, a, b): return self.k.ewBinaryMat(op, self._m(a), self._m(b)).to_numpy()
    def unary(self, op, a): return self.k.ewUnaryMat(op, self._m(a)).to_numpy()
    def agg_row(self, op, a): return self.k.aggRow(op, self._m(a)).to_numpy()
    def agg_col(self, op, a): return self.k.aggCol(op, self._m(a)).to_numpy()
    def agg_all(self, op, a): return self.k.aggAll(op, self._m(a))


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
    else:
        raise AssertionError(chk)


def test_fixture_is_not_trivial():
    assert len(_dense_cases()) >= 80


@pytest.mark.parametrize("case", _dense_cases())
def test_oracle_reproduces_reference_known_answers(case):
    _run_case(_OracleBackend(), case)


@pytest.mark.gpu
@pytest.mark.parametrize("case", _dense_cases())
def test_cuda_reproduces_reference_known_answers(ctx, case):
    _run_case(_CudaBackend(ctx), case)
