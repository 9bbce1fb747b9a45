"""The reference's vectorized-engine script tests (test/api/cli/vectorized/run*.daphne, expected outputs run*.txt;
compared by VectorizedPipelineTest.cpp), restated as kernel-call sequences.

Each script draws rand(rows, cols, lo, hi, sparsity, seed) matrices -- the reference's std::mt19937 stream -- and prints
a few aggregates; DaphneDSL prints a double the way `std::cout` does, i.e. "%g".  The expected strings are the
reference's own (tests/golden/script_outputs.json, extracted as text).  CPU: the reference's RandMatrix compiled from its
sources feeds the oracle's kernels, which pins the oracle at script level.  GPU: db2_randMatrix feeds the device
kernels.  Six significant digits of sums over 10^7 values do not depend on the order of summation."""
import json
from pathlib import Path

import numpy as np
import pytest

GOLD = json.loads((Path(__file__).parent / "golden" / "script_outputs.json").read_text())["scripts"]

BIN = {n: i for i, n in enumerate(["ADD", "SUB", "MUL", "DIV", "POW", "MOD", "LOG", "EQ", "NEQ", "LT", "LE", "GT", "GE",
                                   "MIN", "MAX", "AND", "OR", "BITWISE_AND"])}
SUM, MIN, MAX = 0, 2, 3   # AggOpCode
SQRT = 3                  # UnaryOpCode


class _Cpu:
    """rand by the reference's own kernel, everything else by the oracle"""
    def __init__(self):
        from oracle import pyoracle as o
        from oracle import refkernels as ref
        self.o, self.ref = o, ref
    def rand(self, r, c, lo, hi, sp, seed): return self.ref.rand(r, c, lo, hi, sp, seed)
    def total(self, op, m): return float(self.o.aggAll(op, m))
    def agg_row(self, op, m): return self.o.aggRow(op, m)
    def agg_col(self, op, m): return self.o.aggCol(op, m)
    def binary(self, op, a, b): return self.o.ewBinaryMat(op, a, b)
    def binary_sca(self, op, a, s): return self.o.ewBinaryObjSca(op, a, s)
    def unary(self, op, a): return self.o.ewUnaryMat(op, a)
    def matmul(self, a, b): return self.o.matMul(a, b)
    def syrk(self, a): return self.o.syrk(a, True)
    def outer(self, op, a, b): return self.o.outerBinary(op, a, b)
    def transpose(self, a): return self.o.transpose(a)
    def cbind(self, a, b): return self.o.colBind(a, b)
    def columns(self, a, first, last): return self.o.extractCol(a, np.arange(first, last + 1, dtype=np.int64).reshape(-1, 1))


class _Gpu:
    def __init__(self, ctx):
        import daphne_b200.kernels as k
        self.k, self.ctx = k, ctx
    def rand(self, r, c, lo, hi, sp, seed): return self.k.randMatrix(self.ctx, r, c, lo, hi, sp, seed)
    def total(self, op, m): return float(self.k.aggAll(op, m))
    def agg_row(self, op, m): return self.k.aggRow(op, m)
    def agg_col(self, op, m): return self.k.aggCol(op, m)
    def binary(self, op, a, b): return self.k.ewBinaryMat(op, a, b)
    def binary_sca(self, op, a, s): return self.k.ewBinaryObjSca(op, a, s)
    def unary(self, op, a): return self.k.ewUnaryMat(op, a)
    def matmul(self, a, b): return self.k.matMul(a, b)
    def syrk(self, a): return self.k.syrk(a, True)
    def outer(self, op, a, b): return self.k.outerBinary(op, a, b)
    def transpose(self, a): return self.k.transpose(a)
    def cbind(self, a, b): return self.k.colBind(a, b)
    def columns(self, a, first, last):
        sel = self.k.DenseMatrix.from_numpy(self.ctx, np.arange(first, last + 1, dtype=np.int64).reshape(-1, 1))
        return self.k.extractCol(a, sel)


def _prints(be, name):
    """what the script prints, as numbers, in order"""
    X = be.rand(10000, 1 if name == "runOuterBinary" else 1000, 0.0, 1.0, 1.0, 7)
    if name == "runRowAgg":      # sum(X, 0) and aggMin(X, 0): one value per row
        return [be.total(SUM, be.agg_row(SUM, X)), be.total(SUM, be.agg_row(MIN, X))]
    if name == "runColAgg":      # sum(X, 1): one value per column
        return [be.total(SUM, be.agg_col(SUM, X))]
    if name == "runFullAgg":
        return [be.total(SUM, X), be.total(MIN, X), be.total(MAX, X)]
    if name == "runEwBinary":
        Y = be.rand(10000, 1000, 0.0, 1.0, 1.0, 3)
        out = [be.total(SUM, be.binary(BIN["ADD"], X, Y)), be.total(SUM, be.binary_sca(BIN["ADD"], X, 1.1))]
        out += [be.total(SUM, be.binary(BIN[op], X, Y)) for op in ("SUB", "MUL", "DIV", "POW", "MIN", "MAX")]
        Z = be.rand(1, 1000, -1.0, 1.0, 0.5, 11)  # a row vector, broadcast over the rows of X
        out += [be.total(SUM, be.binary(BIN[op], X, Z)) for op in ("EQ", "NEQ", "LT", "LE", "GT", "GE")]
        return out
    if name == "runEwUnary":
        return [be.total(SUM, be.unary(SQRT, X))]
    if name == "runMatMult":
        return [be.total(SUM, be.matmul(X, be.rand(1000, 10, 1.0, 1.0, 1.0, 3)))]
    if name == "runOther":
        return [be.total(SUM, be.syrk(X))]
    if name == "runOuterBinary":
        return [be.total(SUM, be.outer(BIN["ADD"], X, be.rand(1, 1000, 0.0, 1.0, 1.0, 3)))]
    if name == "runReorganization":
        Y = be.rand(10000, 10, 1.0, 1.0, 1.0, 3)
        return [be.total(SUM, be.transpose(X)), be.total(SUM, be.cbind(X, Y))]
    if name == "runIndexing":    # X[, seq(0, ncol(X) / 2, 1)]: columns 0 .. 500
        return [be.total(SUM, be.columns(X, 0, 500))]
    raise AssertionError(name)


def _check(be, name):
    got = ["%g" % v for v in _prints(be, name)]
    assert got == GOLD[name]["expected"], f"{GOLD[name]['file']}: printed {got}"


def test_fixture_holds_the_ten_scripts():
    assert len(GOLD) == 10 and sum(len(v["expected"]) for v in GOLD.values()) == 27
    assert GOLD["runRowAgg"]["rand"]["X"] == ["10000", "1000", "0.0", "1.0", "1.0", "7"]


@pytest.mark.parametrize("name", sorted(GOLD))
def test_oracle_prints_what_the_reference_script_prints(name):
    try:
        be = _Cpu()
    except (OSError, ImportError) as e:
        pytest.skip(f"the reference's kernels are not built (oracle/_ref): {e}")
    _check(be, name)


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLD))
def test_device_prints_what_the_reference_script_prints(ctx, name):
    _check(_Gpu(ctx), name)
