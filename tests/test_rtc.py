"""Chains without a compiled-in specialisation: the kernel template is instantiated by the run-time compiler.

CPU part: every combination the deferred evaluation can record must compile for sm_100a (the compiler needs no device).
GPU part: the compiled kernel must give the bits of the kernel that reads the chain at run time, and of the oracle."""
import ctypes as C

import numpy as np
import pytest

from daphne_b200.lib import lib, check, Db2Error

OPS = ["ADD", "SUB", "MUL", "DIV", "SQUARE", "EQ", "NEQ", "LT", "LE", "GT", "GE", "MIN", "MAX", "AND", "OR", "NEG", "ABS",
       "SIGN", "FLOOR", "CEIL", "ROUND", "ISNAN"]
KINDS = {"M": 0, "R": 1, "C": 2, "S": 3, "U": 4}
TAPS = {"SUM": 0, "PROD": 1, "MIN": 2, "MAX": 3, "MEAN": 4}


def _compile(steps, taps, ew, column_pass=False):
    """steps: [("SUB", "R", False), ...]; taps: [("SUM", after), ...]; column_pass: the column sums of the chain"""
    arr = lambda xs: (C.c_int * max(len(xs), 1))(*xs)
    ops, kinds, rev = arr([OPS.index(s[0]) for s in steps]), arr([KINDS[s[1]] for s in steps]), arr([int(s[2]) for s in steps])
    after, tk = arr([t[1] for t in taps]), arr([TAPS[t[0]] for t in taps])
    n = C.c_size_t(0)
    check(lib.db2_rtc_compile(ops, kinds, rev, len(steps), after, tk, -1 if column_pass else len(taps), int(ew),
                              C.byref(n)))
    return n.value


def _have_nvrtc():
    try:
        _compile([], [("SUM", 0)], False)
        return True
    except Db2Error as e:
        if "libnvrtc not found" in str(e):
            return False
        raise


needs_nvrtc = pytest.mark.skipif(not _have_nvrtc(), reason="libnvrtc is not installed")


@needs_nvrtc
@pytest.mark.parametrize("steps,taps,ew", [
    ([("SUB", "R", False), ("MUL", "R", False), ("ADD", "S", False)], [("SUM", 3)], False),
    ([("SUB", "R", False), ("MUL", "R", False), ("ADD", "S", False)], [], True),
    ([("DIV", "C", False), ("DIV", "S", True), ("ABS", "U", False)], [("MIN", 1), ("MAX", 3), ("MEAN", 3)], True),
    ([("MUL", "M", False), ("GT", "S", False), ("AND", "M", True), ("FLOOR", "U", False), ("ISNAN", "U", False)],
     [("PROD", 0), ("SUM", 5)], False),
    ([(op, "R", False) for op in OPS[:10]], [("SUM", 10), ("MIN", 4), ("MAX", 7), ("MEAN", 0)], True),
])
def test_chains_compile_for_sm_100a(steps, taps, ew):
    assert _compile(steps, taps, ew) > 10_000  # a device binary, not an empty one


@needs_nvrtc
def test_every_operation_and_operand_kind_compiles():
    for op in OPS:
        unary = op in ("SQUARE", "NEG", "ABS", "SIGN", "FLOOR", "CEIL", "ROUND", "ISNAN")
        for kind in (["U", "S"] if unary else ["M", "R", "C", "S"]):
            for rev in ([False] if unary else [False, True]):
                assert _compile([(op, kind, rev)], [("SUM", 1)], False) > 10_000, (op, kind, rev)


@needs_nvrtc
def test_the_form_for_rows_off_16_byte_boundaries_compiles():
    steps = [("SUB", "R", False), ("DIV", "R", False), ("MUL", "C", False), ("MAX", "M", True), ("ABS", "U", False)]
    taps = [("SUM", 5), ("MIN", 2), ("MAX", 0)]
    assert _compile(steps, taps, 2) > 10_000       # row aggregations only
    assert _compile(steps, taps, 3) > 10_000       # and the values stored
    assert _compile([], [("MEAN", 0)], 2) > 10_000


@needs_nvrtc
def test_column_sums_of_a_chain_compile():
    assert _compile([("SUB", "R", False), ("MUL", "C", False), ("DIV", "M", False), ("ABS", "U", False)], [], False,
                    column_pass=True) > 5_000
    assert _compile([("DIV", "R", False), ("DIV", "S", True)], [], False, column_pass=True) > 5_000


@needs_nvrtc
def test_binaries_are_kept_on_disk_between_processes(tmp_path, monkeypatch):
    """The device binary of a chain is written to DB2_RTC_CACHE and read back from there instead of compiling again; a
    damaged file is thrown away and replaced; DB2_RTC_CACHE=0 writes nothing."""
    import time
    monkeypatch.setenv("DB2_RTC_CACHE", str(tmp_path))
    chain = ([("MUL", "R", False), ("SUB", "S", True), ("CEIL", "U", False)], [("MAX", 3)], False)
    t0 = time.perf_counter()
    n1 = _compile(*chain)
    t_compile = time.perf_counter() - t0
    files = list(tmp_path.glob("*.cubin"))
    assert len(files) == 1 and files[0].stat().st_size > n1 and not list(tmp_path.glob("*.tmp*"))
    t0 = time.perf_counter()
    n2 = _compile(*chain)
    t_cached = time.perf_counter() - t0
    assert n2 == n1 and t_cached < t_compile / 5, (t_compile, t_cached)
    # another chain, another file; the same chain for the other layout, a third one
    _compile(chain[0], [("MIN", 3)], False)
    _compile(chain[0], chain[1], 2)
    assert len(list(tmp_path.glob("*.cubin"))) == 3
    # a file that was cut short is not used: compiled again and written again
    def whole(path):  # a complete file again (the compiler's output is not the same bytes every time)
        b = path.read_bytes()
        size, name = int.from_bytes(b[8:16], "little"), int.from_bytes(b[24:32], "little")
        return b[:8] == b"DB2RTC1\0" and len(b) == 32 + name + size
    data = files[0].read_bytes()
    assert whole(files[0])
    files[0].write_bytes(data[: len(data) // 2])
    assert not whole(files[0])
    assert _compile(*chain) > 10_000 and whole(files[0])
    # a file whose contents were altered fails the checksum
    files[0].write_bytes(data[:-8] + bytes(8))
    t0 = time.perf_counter()
    assert _compile(*chain) > 10_000
    assert time.perf_counter() - t0 > 5 * t_cached       # it was compiled, not read
    assert files[0].read_bytes()[-8:] != bytes(8) and whole(files[0])
    # switched off: nothing is written
    off = tmp_path / "off"
    off.mkdir()
    monkeypatch.setenv("DB2_RTC_CACHE", "0")
    _compile([("ADD", "S", False)], [("SUM", 1)], False)
    monkeypatch.setenv("DB2_RTC_CACHE", str(off))
    assert not list(off.iterdir())


def test_bad_arguments_are_refused():
    with pytest.raises(Db2Error):
        _compile([("ADD", "R", False)] * 11, [], True)       # more steps than a program holds
    with pytest.raises(Db2Error):
        _compile([("ADD", "R", False)], [("SUM", 2)], False)  # an aggregation after a step that does not exist
    with pytest.raises(Db2Error):
        check(lib.db2_rtc_set_mode(7))


@pytest.mark.gpu
@needs_nvrtc
@pytest.mark.parametrize("shape", [(70000, 48), (4099, 50), (2049, 128), (300, 400)])
def test_compiled_chain_gives_the_bits_of_the_run_time_kernel_and_of_the_oracle(ctx, shape):
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    from tests.util import RTOL_REDUCE_F64, assert_bits_equal, assert_close_rel, rng_matrix
    B, U, A = k.BinaryOpCode, k.UnaryOpCode, k.AggOpCode
    r, c = shape
    x, y = rng_matrix(3, r, c) - 5.0, rng_matrix(4, r, c) - 5.0
    rv, cv = rng_matrix(5, 1, c) - 4.0, rng_matrix(6, r, 1) - 4.0
    y[::7] = x[::7]
    x[3, :4] = [0.0, -0.0, np.inf, np.nan]   # zeros, infinities and NaNs through every division
    x[5, 0], cv[9, 0], rv[0, 2] = -0.0, 0.0, 1e-310

    def run(kk, mk):
        X, Y, RV, CV = mk(x), mk(y), mk(rv), mk(cv)
        t = kk.ewBinaryMat(B.SUB, X, RV)            # row vector
        t = kk.ewBinaryMat(B.DIV, t, CV)            # division by a column vector (no staged reciprocal)
        t = kk.ewBinaryMat(B.DIV, t, RV)            # division by a row vector (staged reciprocal)
        t = kk.ewBinaryObjSca(B.DIV, t, 3.7)        # by a scalar
        t = kk.ewBinaryMat(B.DIV, t, Y)             # by a matrix
        u = kk.ewUnaryMat(U.ABS, kk.ewBinaryMat(B.MAX, t, Y))
        w = kk.ewBinaryMat(B.DIV, X, kk.ewBinaryMat(B.SUB, Y, u))  # reversed steps
        z = kk.ewBinaryObjSca(B.ADD, kk.ewBinaryMat(B.MUL, kk.ewBinaryMat(B.SUB, X, RV), RV), 0.5)
        return t, u, w, z

    cpu = run(type("O", (), {"ewBinaryMat": staticmethod(o.ewBinaryMat), "ewBinaryObjSca": staticmethod(o.ewBinaryObjSca),
                             "ewUnaryMat": staticmethod(o.ewUnaryMat)}), lambda a: a)
    ready0 = C.c_int()
    check(lib.db2_rtc_counts(C.byref(ready0), None, None))
    try:
        for mode, name in ((0, "run-time chain"), (2, "compiled chain")):
            check(lib.db2_rtc_set_mode(mode))
            dev = run(k, lambda a: k.DenseMatrix.from_numpy(ctx, a))
            for i, (g, e) in enumerate(zip(dev, cpu)):
                with np.errstate(all="ignore"):
                    assert_bits_equal(k.aggRow(A.MIN, g).to_numpy(), o.aggRow(A.MIN, e), f"{name}: rowMin {i}")
                    assert_bits_equal(k.aggRow(A.IDXMAX, g).to_numpy(), o.aggRow(A.IDXMAX, e), f"{name}: idxMax {i}")
                    assert_bits_equal(g.to_numpy(), e, f"{name}: values {i}")
            ok = ~np.isnan(cpu[3]).any(1) & ~np.isinf(cpu[3]).any(1)
            got = k.aggRow(A.SUM, dev[3]).to_numpy()[ok]
            assert_close_rel(got, o.aggRow(A.SUM, cpu[3])[ok], RTOL_REDUCE_F64, f"{name}: rowSum", scale=1e-9)
        ready, pending, failed = C.c_int(), C.c_int(), C.c_int()
        check(lib.db2_rtc_counts(C.byref(ready), C.byref(pending), C.byref(failed)))
        assert failed.value == 0 and pending.value == 0
        if c % 2 == 0:  # odd widths go through the general interpreter and are never compiled
            assert ready.value > ready0.value or ready0.value > 0
    finally:
        check(lib.db2_rtc_set_mode(2))


@pytest.mark.gpu
@needs_nvrtc
def test_background_compilation_takes_over_after_it_finishes(ctx):
    """Background mode: the first call is served by the run-time kernel while the compiler works; after db2_rtc_wait the
    same chain runs compiled.  Both must give the same bits."""
    import daphne_b200.kernels as k
    from tests.util import assert_bits_equal
    B, A = k.BinaryOpCode, k.AggOpCode
    rng = np.random.default_rng(77)
    x, rv = rng.standard_normal((50000, 32)), rng.standard_normal((1, 32)) + 3.0
    X, RV = k.DenseMatrix.from_numpy(ctx, x), k.DenseMatrix.from_numpy(ctx, rv)

    def run():
        z = k.ewBinaryObjSca(B.SUB, k.ewBinaryMat(B.DIV, k.ewBinaryMat(B.ADD, X, RV), RV), 0.125)
        return k.aggRow(A.MAX, z).to_numpy(), k.aggRow(A.SUM, z).to_numpy()
    check(lib.db2_rtc_set_mode(1))
    try:
        first = run()
        check(lib.db2_rtc_wait())
        pending = C.c_int()
        check(lib.db2_rtc_counts(None, C.byref(pending), None))
        assert pending.value == 0
        second = run()
    finally:
        check(lib.db2_rtc_set_mode(2))
    for a, b in zip(first, second):
        assert_bits_equal(b, a, "compiled against run-time chain")
    ref = (x + rv) / rv - 0.125
    assert_bits_equal(second[0], ref.max(1, keepdims=True), "row maximum")


@pytest.mark.gpu
@needs_nvrtc
@pytest.mark.parametrize("shape", [(70000, 48), (4099, 50), (100001, 6)])
def test_column_sums_of_a_chain_without_compiled_in_kernel(ctx, shape):
    """colSums / colMeans of ((X - mu) / cv) * Y: general column pass, then the kernel compiled for the chain; the two
    sum in different orders, so they agree with the oracle within the reduction tolerance, not bit for bit."""
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    from tests.util import RTOL_REDUCE_F64, assert_close_rel, rng_matrix
    B, A = k.BinaryOpCode, k.AggOpCode
    r, c = shape
    x, y = rng_matrix(13, r, c) - 5.0, rng_matrix(14, r, c) + 1.0
    mu, cv = rng_matrix(15, 1, c), rng_matrix(16, r, 1) + 2.0
    ref = o.ewBinaryMat(B.MUL, o.ewBinaryMat(B.DIV, o.ewBinaryMat(B.SUB, x, mu), cv), y)
    ready, failed = C.c_int(), C.c_int()
    try:
        for mode in (0, 2):
            check(lib.db2_rtc_set_mode(mode))
            X, Y, MU, CV = (k.DenseMatrix.from_numpy(ctx, a) for a in (x, y, mu, cv))
            z = k.ewBinaryMat(B.MUL, k.ewBinaryMat(B.DIV, k.ewBinaryMat(B.SUB, X, MU), CV), Y)
            assert_close_rel(k.aggCol(A.SUM, z).to_numpy(), o.aggCol(A.SUM, ref), RTOL_REDUCE_F64, f"colSums mode {mode}",
                             scale=float(np.abs(ref).sum(0).max()))
            z = k.ewBinaryMat(B.MUL, k.ewBinaryMat(B.DIV, k.ewBinaryMat(B.SUB, X, MU), CV), Y)
            assert_close_rel(k.aggCol(A.MEAN, z).to_numpy(), o.aggCol(A.MEAN, ref), RTOL_REDUCE_F64,
                             f"colMeans mode {mode}", scale=float(np.abs(ref).mean(0).max()))
        check(lib.db2_rtc_counts(C.byref(ready), None, C.byref(failed)))
        assert failed.value == 0 and ready.value > 0
    finally:
        check(lib.db2_rtc_set_mode(2))


@pytest.mark.gpu
@needs_nvrtc
@pytest.mark.parametrize("shape,view", [((70001, 33), None), ((4099, 7), None), ((3001, 129), None), ((2049, 1), None),
                                        ((50000, 64), (3, 40)), ((50000, 65), (1, 65)), ((300, 401), (200, 333))])
def test_rows_off_16_byte_boundaries_take_the_compiled_kernel_too(ctx, shape, view):
    """Odd numbers of columns, odd leading dimensions and column views that start at an odd column: the kernel copies
    its chunks element by element.  Values, row extrema with positions and row sums against the oracle, for the
    kernel compiled at run time and for the general interpreter that serves such layouts without it."""
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    from tests.util import RTOL_REDUCE_F64, assert_bits_equal, assert_close_rel, rng_matrix
    B, U, A = k.BinaryOpCode, k.UnaryOpCode, k.AggOpCode
    r, c = shape
    full = rng_matrix(23, r, c) - 5.0
    lo, hi = view if view else (0, c)
    full[min(3, r - 1), lo] = 0.0
    x = np.ascontiguousarray(full[:, lo:hi])
    w = hi - lo
    rv, cv, y = rng_matrix(24, 1, w) - 4.0, rng_matrix(25, r, 1) + 2.0, rng_matrix(26, r, w)

    def run(kk, X, RV, CV, Y):
        t = kk.ewBinaryMat(B.DIV, kk.ewBinaryMat(B.SUB, X, RV), RV)   # staged operand and its reciprocals
        t = kk.ewBinaryMat(B.MUL, t, CV)
        u = kk.ewUnaryMat(U.ABS, kk.ewBinaryMat(B.MIN, t, Y))
        return t, u

    cpu = run(type("O", (), {"ewBinaryMat": staticmethod(o.ewBinaryMat), "ewUnaryMat": staticmethod(o.ewUnaryMat)}),
              x, rv, cv, y)
    try:
        for mode, name in ((0, "interpreter"), (2, "compiled")):
            check(lib.db2_rtc_set_mode(mode))
            F = k.DenseMatrix.from_numpy(ctx, full)
            X = k.sliceCol(F, lo, hi) if view else F
            dev = run(k, X, *(k.DenseMatrix.from_numpy(ctx, a) for a in (rv, cv, y)))
            for i, (g, e) in enumerate(zip(dev, cpu)):
                assert_bits_equal(k.aggRow(A.MAX, g).to_numpy(), o.aggRow(A.MAX, e), f"{name}: rowMax {i}")
                assert_bits_equal(k.aggRow(A.IDXMIN, g).to_numpy(), o.aggRow(A.IDXMIN, e), f"{name}: idxMin {i}")
                assert_close_rel(k.aggRow(A.SUM, g).to_numpy(), o.aggRow(A.SUM, e), RTOL_REDUCE_F64, f"{name}: rowSum {i}",
                                 scale=float(np.abs(e).sum(1).max()))
                assert_bits_equal(g.to_numpy(), e, f"{name}: values {i}")
        failed = C.c_int()
        check(lib.db2_rtc_counts(None, None, C.byref(failed)))
        assert failed.value == 0
    finally:
        check(lib.db2_rtc_set_mode(2))


@pytest.mark.gpu
@needs_nvrtc
def test_a_second_process_loads_the_kernel_from_disk(tmp_path):
    """Process A compiles a chain's kernel and leaves it in DB2_RTC_CACHE; process B, which has no compiler at all
    (DB2_RTC_NO_COMPILER), runs the same chain with that kernel and gets the same bits; process C, without compiler and
    with an empty directory, falls back to the kernel that reads the chain at run time."""
    import os
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    code = "\n".join([
        "import sys, ctypes as C, numpy as np",
        f"sys.path.insert(0, {str(root)!r})",
        "import daphne_b200.kernels as k",
        "from daphne_b200.lib import lib, check",
        "B, A = k.BinaryOpCode, k.AggOpCode",
        "ctx = k.Context(0)",
        "rng = np.random.default_rng(5)",
        "X = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((50000, 32)))",
        "RV = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((1, 32)) + 3.0)",
        "z = k.ewBinaryObjSca(B.ADD, k.ewBinaryMat(B.MUL, k.ewBinaryMat(B.SUB, X, RV), RV), 0.25)",
        "m = k.aggRow(A.MAX, z).to_numpy()",
        "ready, failed = C.c_int(), C.c_int()",
        "check(lib.db2_rtc_counts(C.byref(ready), None, C.byref(failed)))",
        "print(ready.value, failed.value, float(m.sum()).hex(), float(m[777, 0]).hex())",
        "ctx.close()"])

    def run(cache, no_compiler):
        env = dict(os.environ, DB2_RTC_CACHE=str(cache))
        env.pop("DB2_RTC", None)
        if no_compiler:
            env["DB2_RTC_NO_COMPILER"] = "1"
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        ready, failed, total, one = r.stdout.strip().split()[-4:]
        return int(ready), int(failed), total, one

    shared, empty = tmp_path / "shared", tmp_path / "empty"
    shared.mkdir()
    empty.mkdir()
    a = run(shared, False)
    assert a[0] >= 1 and a[1] == 0 and len(list(shared.glob("*.cubin"))) >= 1
    b = run(shared, True)
    assert b[0] >= 1 and b[1] == 0 and b[2:] == a[2:]
    c = run(empty, True)
    assert c[0] == 0 and c[1] >= 1 and c[2:] == a[2:] and not list(empty.glob("*.cubin"))
