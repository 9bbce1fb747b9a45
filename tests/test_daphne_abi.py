"""The DAPHNE-facing adapter (daphne_b200/_abi_build/libCUDAKernels.so): the library DAPHNE's kernel catalog would
load in place of its own libCUDAKernels.so.  Built by daphne_b200/csrc/daphne_abi/build_adapter.py from a DAPHNE
source tree; skipped where it was not built.

CPU: every function of the generated catalog is an exported symbol, and the names are the reference's.
GPU: a driver that plays the JIT (owns real DenseMatrix objects, resolves kernels by symbol name, reads results back
through DenseMatrix::getValues()) against the CPU oracle."""
import ctypes as C
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
ABI = ROOT / "daphne_b200" / "_abi_build"
pytestmark = pytest.mark.skipif(not (ABI / "libCUDAKernels.so").exists(), reason="adapter library not built")


def test_catalog_symbols_are_exported_with_the_reference_names():
    cat = json.loads((ABI / "CUDAcatalog.json").read_text())
    out = subprocess.run(["nm", "-D", "--defined-only", str(ABI / "libCUDAKernels.so")], capture_output=True,
                         text=True, check=True).stdout
    syms = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    names = {e["kernelFuncName"] for e in cat}
    assert len(names) >= 250
    assert not (names - syms)
    for must in ("CUDA_sumRow__DenseMatrix_double__DenseMatrix_double", "CUDA_sumAll__double__DenseMatrix_double",
                 "CUDA_ewAdd__DenseMatrix_double__DenseMatrix_double__double",
                 "CUDA_matMul__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double__bool__bool",
                 "CUDA_syrk__DenseMatrix_double__DenseMatrix_double__bool", "CUDA_createCUDAContext",
                 "CUDA_gemv__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double",
                 "CUDA_solve__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double",
                 "CUDA_transpose__DenseMatrix_double__DenseMatrix_double",
                 "CUDA_fill__DenseMatrix_double__double__size_t__size_t",
                 "CUDA_colBind__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double",
                 "CUDA_extractCol__DenseMatrix_double__DenseMatrix_double__DenseMatrix_int64_t"):
        assert must in syms, must
    assert all(e["backend"] == "CUDA" and e["libPath"] == "libCUDAKernels.so" for e in cat)


def test_extension_catalog_registers_cpu_names_for_ops_without_cuda_support():
    """Operators the reference's compiler never tags for CUDA (no CUDASupport trait) are served through an extension
    catalog under backend "CPP" (daphne --kernel-ext B200ExtCatalog.json:1)."""
    cat = json.loads((ABI / "B200ExtCatalog.json").read_text())
    out = subprocess.run(["nm", "-D", "--defined-only", str(ABI / "libB200ExtKernels.so")], capture_output=True,
                         text=True, check=True).stdout
    syms = {ln.split()[-1] for ln in out.splitlines() if " T " in ln}
    names = {e["kernelFuncName"] for e in cat}
    assert len(names) >= 100 and not (names - syms)
    assert all(e["backend"] == "CPP" and e["libPath"] == "libB200ExtKernels.so" for e in cat)
    assert ("_vectorizedPipeline__DenseMatrix_double_variadic__size_t__bool__Structure_variadic__size_t__int64_t__"
            "int64_t__int64_t__int64_t__size_t__void_variadic") in syms  # the scheduler under DAPHNE's own name
    for must in ("_ewSqrt__DenseMatrix_double__DenseMatrix_double", "_idxminRow__DenseMatrix_size_t__DenseMatrix_double",
                 "_idxmaxRow__DenseMatrix_size_t__DenseMatrix_double", "_meanCol__DenseMatrix_double__DenseMatrix_double",
                 "_varCol__DenseMatrix_double__DenseMatrix_double", "_stddevCol__DenseMatrix_double__DenseMatrix_double",
                 "_ctable__DenseMatrix_double__DenseMatrix_int64_t__DenseMatrix_int64_t__double__int64_t__int64_t"):
        assert must in names, must
    # nothing that the CUDA catalog already serves is shadowed
    assert not any(e["opMnemonic"] in ("sumRow", "minRow", "maxRow", "sumCol", "sumAll") and
                   not any("CSRMatrix" in t for t in e["argTypes"]) for e in cat)
    # the sparse operators of connected components: no CUDA instantiation exists in the reference
    for must in ("_ewMul__CSRMatrix_double__CSRMatrix_double__DenseMatrix_double",
                 "_maxRow__DenseMatrix_double__CSRMatrix_double",
                 "_matMul__DenseMatrix_double__CSRMatrix_double__DenseMatrix_double__bool__bool"):
        assert must in names, must


def _load_driver():
    C.CDLL(str(ROOT / "daphne_b200" / "libdaphne_b200.so"), mode=C.RTLD_GLOBAL)
    C.CDLL(str(ABI / "libCUDAKernels.so"), mode=C.RTLD_GLOBAL)
    C.CDLL(str(ABI / "libB200ExtKernels.so"), mode=C.RTLD_GLOBAL)
    d = C.CDLL(str(ABI / "libabi_driver.so"), mode=C.RTLD_GLOBAL)
    d.drv_last_error.restype = C.c_char_p
    assert d.drv_init() == 0, d.drv_last_error()
    return d


@pytest.fixture(scope="module")
def drv():
    return _load_driver()


def _p(a):
    return C.c_void_p(a.ctypes.data)


def _call(d, fn, *args, cap=1 << 22):
    out = np.empty(cap)
    r, c = C.c_int64(), C.c_int64()
    rc = fn(*args, _p(out), C.c_int64(cap), C.byref(r), C.byref(c))
    if rc != 0:
        raise RuntimeError(d.drv_last_error().decode())
    return out[: r.value * c.value].reshape(r.value, c.value).copy()


i64 = C.c_int64


@pytest.mark.gpu
def test_kernels_called_by_symbol_through_daphne_objects(drv):
    from oracle import pyoracle as o
    rng = np.random.default_rng(0)
    a = np.ascontiguousarray(rng.standard_normal((3000, 40)))
    b = np.ascontiguousarray(rng.standard_normal((3000, 40)))
    for name, f, op in (("sumRow", o.aggRow, 0), ("minRow", o.aggRow, 2), ("maxRow", o.aggRow, 3),
                        ("sumCol", o.aggCol, 0), ("minCol", o.aggCol, 2), ("maxCol", o.aggCol, 3)):
        got = _call(drv, drv.drv_unary, f"CUDA_{name}__DenseMatrix_double__DenseMatrix_double".encode(), _p(a),
                    i64(3000), i64(40))
        np.testing.assert_allclose(got, f(op, a), rtol=1e-12)
    for name, op in (("sumAll", 0), ("minAll", 2), ("maxAll", 3)):
        v = C.c_double()
        assert drv.drv_scalar(f"CUDA_{name}__double__DenseMatrix_double".encode(), _p(a), i64(3000), i64(40),
                              C.byref(v)) == 0, drv.drv_last_error()
        assert abs(v.value - o.aggAll(op, a)) <= 1e-12 * abs(o.aggAll(op, a))
    for name, op in (("ewAdd", 0), ("ewSub", 1), ("ewMul", 2), ("ewDiv", 3), ("ewMax", 14), ("ewNeq", 8)):
        sym = f"CUDA_{name}__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double".encode()
        got = _call(drv, drv.drv_binary, sym, _p(a), i64(3000), i64(40), _p(b), i64(3000), i64(40))
        assert np.array_equal(got, o.ewBinaryMat(op, a, b)), name
        rv = np.ascontiguousarray(b[:1])
        got = _call(drv, drv.drv_binary, sym, _p(a), i64(3000), i64(40), _p(rv), i64(1), i64(40))
        assert np.array_equal(got, o.ewBinaryMat(op, a, rv)), name + " row vector"
        sym = f"CUDA_{name}__DenseMatrix_double__DenseMatrix_double__double".encode()
        got = _call(drv, drv.drv_binary_sca, sym, _p(a), i64(3000), i64(40), C.c_double(1.5))
        assert np.array_equal(got, o.ewBinaryObjSca(op, a, 1.5)), name + " scalar"
    got = _call(drv, drv.drv_unary, b"CUDA_transpose__DenseMatrix_double__DenseMatrix_double", _p(a), i64(3000),
                i64(40))
    assert np.array_equal(got, a.T)
    for ta, tb, x, y in ((0, 0, a, np.ascontiguousarray(b[:40, :17])), (1, 0, a, b), (0, 1, a, b[:50].copy())):
        got = _call(drv, drv.drv_matmul, _p(x), i64(x.shape[0]), i64(x.shape[1]), _p(y), i64(y.shape[0]),
                    i64(y.shape[1]), C.c_int(ta), C.c_int(tb))
        exp = o.matMul(x, y, ta, tb)
        assert np.abs(got - exp).max() <= 1e-12 * np.abs(exp).max()
    got = _call(drv, drv.drv_syrk, _p(a), i64(3000), i64(40), C.c_int(1))
    assert np.abs(got - o.syrk(a)).max() <= 1e-12 * np.abs(o.syrk(a)).max()
    y = np.ascontiguousarray(rng.standard_normal((3000, 1)))
    got = _call(drv, drv.drv_binary, b"CUDA_gemv__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double", _p(a),
                i64(3000), i64(40), _p(y), i64(3000), i64(1))
    assert np.abs(got - o.gemv(a, y)).max() <= 1e-12 * np.abs(o.gemv(a, y)).max()
    s = o.syrk(a) + 0.001 * np.eye(40)
    rhs = o.gemv(a, y)
    got = _call(drv, drv.drv_binary, b"CUDA_solve__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double", _p(s),
                i64(40), i64(40), _p(rhs), i64(40), i64(1))
    assert np.abs(got - o.solve(s, rhs)).max() <= 1e-9 * np.abs(o.solve(s, rhs)).max()
    got = _call(drv, drv.drv_binary, b"CUDA_colBind__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double", _p(a),
                i64(3000), i64(40), _p(y), i64(3000), i64(1))
    assert np.array_equal(got, np.hstack([a, y]))


@pytest.mark.gpu
def test_chained_calls_keep_intermediates_on_the_device_and_views_keep_their_offset(drv):
    rng = np.random.default_rng(1)
    x = np.ascontiguousarray(rng.standard_normal((80000, 16)))
    mu = np.ascontiguousarray(x.mean(axis=0, keepdims=True))
    got = _call(drv, drv.drv_chain, _p(x), i64(80000), i64(16), _p(mu), C.c_double(3.0), i64(1000), i64(71000))
    exp = (((x + 0.0)[1000:71000] - mu) * 3.0)
    seq = np.zeros((70000, 1))
    for c in range(16):  # the fused row pass adds left to right like the reference
        seq[:, 0] += exp[:, c]
    assert np.array_equal(got, seq)


@pytest.mark.gpu
def test_errors_surface_as_exceptions_with_the_reference_message(drv):
    a, b = np.ones((4, 5)), np.ones((3, 2))
    out = np.empty(100)
    r, c = C.c_int64(), C.c_int64()
    rc = drv.drv_binary(b"CUDA_ewAdd__DenseMatrix_double__DenseMatrix_double__DenseMatrix_double", _p(a), i64(4),
                        i64(5), _p(b), i64(3), i64(2), _p(out), i64(100), C.byref(r), C.byref(c))
    assert rc == 1
    assert b"lhs and rhs must either have the same dimensions" in drv.drv_last_error()


@pytest.mark.gpu
def test_extension_kernels_by_symbol_name(drv):
    from oracle import pyoracle as o
    rng = np.random.default_rng(9)
    n, d = 3000, 17
    x = rng.random((n, d)) * 4.0
    x[5, 3] = x[5, 9] = 0.0  # a tie: the lowest index wins
    ys = rng.integers(0, 6, size=500).astype(np.int64)
    xs = rng.integers(0, 4, size=500).astype(np.int64)
    out = np.empty(n + 2 * d + 24)
    rc = drv.drv_ext(_p(x), C.c_int64(n), C.c_int64(d), _p(ys), _p(xs), C.c_int64(500), C.c_double(2.0),
                     C.c_int64(6), C.c_int64(4), _p(out))
    assert rc == 0, drv.drv_last_error()
    s = np.sqrt(x)
    assert np.array_equal(out[:n], o.aggRow(4, s).ravel())          # IDXMIN
    np.testing.assert_allclose(out[n:n + d], o.aggCol(6, s).ravel(), rtol=1e-12)           # MEAN
    np.testing.assert_allclose(out[n + d:n + 2 * d], o.aggCol(8, s).ravel(), rtol=1e-11)   # VAR
    assert np.array_equal(out[n + 2 * d:].reshape(6, 4), o.ctable(ys, xs, 2.0, 6, 4))


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [None, 1000, 7777])
def test_scheduler_under_daphnes_symbol_name(drv, batch, monkeypatch):
    """_vectorizedPipeline__DenseMatrix_double_variadic__... with a body that calls CUDA_* kernels by name: one batch
    (results are the body's objects) and several batches (ROWS results copied into place, ADD results folded)."""
    import os
    if batch is None:
        os.environ.pop("DAPHNE_B200_BATCH_ROWS", None)
    else:
        os.environ["DAPHNE_B200_BATCH_ROWS"] = str(batch)
    try:
        rng = np.random.default_rng(10)
        n, d = 20000, 24
        x, mu, s = rng.standard_normal((n, d)), rng.standard_normal((1, d)), 1.75
        out = np.empty(n + d)
        rc = drv.drv_pipeline(_p(x), C.c_int64(n), C.c_int64(d), _p(mu), C.c_double(s), _p(out))
        assert rc == 0, drv.drv_last_error()
        np.testing.assert_allclose(out[:n], ((x - mu) * s).sum(1), rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(out[n:], (x - mu).sum(0), rtol=1e-10, atol=1e-9)
    finally:
        os.environ.pop("DAPHNE_B200_BATCH_ROWS", None)


def _check_pipeline_all(d, n=20001, cols=12, deferred=0):
    rng = np.random.default_rng(11)
    x, s = rng.standard_normal((n, cols)), 0.625
    out = np.empty(2 * n + 3 * cols)
    rc = d.drv_pipeline_all(_p(x), C.c_int64(n), C.c_int64(cols), C.c_double(s), C.c_int(deferred), _p(out))
    assert rc == 0, d.drv_last_error()
    np.testing.assert_allclose(out[:n], (x * s).sum(1), rtol=1e-12, atol=1e-12)                      # ROWS
    np.testing.assert_allclose(out[n:n + cols], x.sum(0), rtol=1e-10, atol=1e-9)                     # ADD
    assert np.array_equal(out[n + cols:n + 2 * cols], x.max(0))                                      # MAX
    assert np.array_equal(out[n + 2 * cols:n + 3 * cols], x.min(0))                                  # MIN
    assert np.array_equal(out[n + 3 * cols:], x.max(1))                                              # COLS


@pytest.mark.gpu
@pytest.mark.parametrize("batch", [None, 3000])
def test_scheduler_all_combines_under_daphnes_symbol_name(drv, batch):
    import os
    if batch is not None:
        os.environ["DAPHNE_B200_BATCH_ROWS"] = str(batch)
    try:
        _check_pipeline_all(drv)
        _check_pipeline_all(drv, deferred=1)
    finally:
        os.environ.pop("DAPHNE_B200_BATCH_ROWS", None)


@pytest.mark.gpu
def test_all_five_scheduler_entry_points_are_exported():
    out = subprocess.run(["nm", "-D", "--defined-only", str(ABI / "libB200ExtKernels.so")], capture_output=True,
                         text=True, check=True).stdout
    for dt in ("DenseMatrix_double", "DenseMatrix_float", "DenseMatrix_int64_t", "CSRMatrix_double", "CSRMatrix_float"):
        assert (f"_vectorizedPipeline__{dt}_variadic__size_t__bool__Structure_variadic__size_t__int64_t__int64_t__"
                "int64_t__int64_t__size_t__void_variadic") in out, dt


@pytest.mark.gpu
def test_connected_components_by_symbol_name_on_a_real_csr_matrix(drv):
    """The cfg4 loop through DAPHNE's names (_ewMul__CSRMatrix..., _maxRow__DenseMatrix_double__CSRMatrix_double, CUDA_ewMax,
    CUDA_ewNeq, CUDA_sumAll) on CSRMatrix objects: labels bit-equal to the reference's CPU kernels."""
    from oracle import cpu_pipelines as cpu
    from tests.test_pipelines_gpu import _graph
    for n, deg, seed in [(3000, 2, 1), (100000, 8, 4)]:
        g = _graph(n, deg, seed)
        vals = np.ascontiguousarray(g.data, dtype=np.float64)
        cols = np.ascontiguousarray(g.indices, dtype=np.uint64)
        offs = np.ascontiguousarray(g.indptr, dtype=np.uint64)
        labels, iters = np.empty(n), C.c_int64()
        rc = drv.drv_components(_p(vals), _p(cols), _p(offs), C.c_int64(n), C.c_int64(1000), _p(labels),
                                C.byref(iters))
        assert rc == 0, drv.drv_last_error()
        c, it = cpu.connected_components(g)
        assert iters.value == it
        assert np.array_equal(labels.view(np.uint64), c[:, 0].view(np.uint64))


@pytest.mark.gpu
@pytest.mark.parametrize("devices", ["0,0", "0,0,0", "all"])
def test_scheduler_over_several_devices_in_one_process(devices):
    """The scheduler under DAPHNE's name with a device group of more than one context (DAPHNE_B200_DEVICES): two or
    three contexts that share device 0, and every visible device.  A fresh process, because the group is made once."""
    import os
    import sys
    code = "\n".join([
        "import sys",
        f"sys.path.insert(0, {str(ROOT)!r})",
        "from tests import test_daphne_abi as t",
        "d = t._load_driver()",
        "n = d.drv_devices()",
        "t._check_pipeline_all(d)",
        "t._check_pipeline_all(d, n=4099, deferred=1)",
        "t._check_pipeline_all(d, n=2, cols=3)",
        "print('devices', n)"])
    env = dict(os.environ, DAPHNE_B200_DEVICES=devices)
    r = subprocess.run([sys.executable, "-c", code.replace("\n", "\n")], capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    n = int(r.stdout.strip().split()[-1])
    assert n == (devices.count(",") + 1 if devices != "all" else n) and n >= 1


def _same(op, dtype, out, exp):
    if np.dtype(dtype).kind == "f":
        return np.allclose(out, exp, rtol=1e-5) if op in (4, 6) else np.array_equal(out, exp)
    if op == 6:  # truncated log quotients may flip by one next to an integer; log(a) / log(1) has no defined result
        fin = exp.astype(np.float64) < 1e9
        return np.abs(out.astype(np.int64) - exp.astype(np.int64))[fin].max(initial=0) <= 1
    return np.array_equal(out, exp)


@pytest.mark.gpu
def test_every_value_type_of_the_elementwise_catalog_entries_computes(drv):
    """The CUDA catalog names the elementwise binary kernels for six value types (double, float, int64_t, uint64_t,
    int32_t, uint32_t) and fill also for bool and uint8_t: every one of them is served by a device kernel, called here
    by its catalog name on DenseMatrix objects of that type."""
    from oracle import pyoracle as o
    from tests.test_oracle_vs_ref import _int_operands
    cat = json.loads((ABI / "CUDAcatalog.json").read_text())
    names = {e["kernelFuncName"] for e in cat}
    types = {"float": (np.float32, 1), "int64_t": (np.int64, 2), "uint64_t": (np.uint64, 3), "int32_t": (np.int32, 4),
             "uint32_t": (np.uint32, 5)}
    ops = {"ewAdd": 0, "ewSub": 1, "ewMul": 2, "ewDiv": 3, "ewPow": 4, "ewMod": 5, "ewLog": 6, "ewEq": 7, "ewNeq": 8,
           "ewLt": 9, "ewLe": 10, "ewGt": 11, "ewGe": 12, "ewMin": 13, "ewMax": 14, "ewAnd": 15, "ewOr": 16,
           "ewBitwise_and": 17}
    called = 0
    for vt, (dtype, code) in types.items():
        if np.dtype(dtype).kind == "f":
            rng = np.random.default_rng(3)
            a = (rng.random((300, 17)) * 5 + 1).astype(dtype)
            b = (rng.random((300, 17)) * 3 + 1).astype(dtype)
            rv = b[:1].copy()
        else:
            a, b, rv, _ = _int_operands(dtype, 3, 300, 17)
            a = (np.abs(a.astype(np.int64)) % 5 + 9).astype(dtype)
        for mn, op in ops.items():
            if op == 17 and np.dtype(dtype).kind == "f":
                continue  # no reference semantics: BITWISE_AND is declared for integer value types only
            x = (a % 5 + 1).astype(dtype) if op == 4 and np.dtype(dtype).kind != "f" else a
            mat = f"CUDA_{mn}__DenseMatrix_{vt}__DenseMatrix_{vt}__DenseMatrix_{vt}"
            sca = f"CUDA_{mn}__DenseMatrix_{vt}__DenseMatrix_{vt}__{vt}"
            out = np.empty_like(x)
            if mat in names:
                for rhs in (b, rv):
                    rc = drv.drv_binary_typed(mat.encode(), code, _p(x), i64(300), i64(17), _p(rhs),
                                              i64(rhs.shape[0]), i64(17), None, _p(out))
                    assert rc == 0, (mat, drv.drv_last_error())
                    exp = o.ewBinaryMat(op, x, rhs)
                    assert _same(op, dtype, out, exp), mat
                    called += 1
            if sca in names:
                s = np.array([3], dtype=dtype)
                rc = drv.drv_binary_typed(sca.encode(), code, _p(x), i64(300), i64(17), None, i64(0), i64(0), _p(s),
                                          _p(out))
                assert rc == 0, (sca, drv.drv_last_error())
                exp = o.ewBinaryObjSca(op, x, s[0])
                assert _same(op, dtype, out, exp), sca
                called += 1
    assert called >= 5 * 35 + 5 * 17 - 2  # every ew* entry of the five non-double types, matrix entries twice
    buf = np.empty(35, dtype=np.uint8)
    for as_bool, v in ((1, 1), (0, 203)):
        assert drv.drv_fill_u8(as_bool, v, i64(7), i64(5), _p(buf)) == 0, drv.drv_last_error()
        assert np.all(buf == v)


@pytest.mark.gpu
def test_float_entries_of_the_contraction_kernels_compute(drv):
    """CUDA_solve / CUDA_gemv / CUDA_matMul / CUDA_syrk are registered for float as well as double: the float names
    compute too (solve in double with one final rounding, the products on the tf32 tensor-core path)."""
    cat = json.loads((ABI / "CUDAcatalog.json").read_text())
    names = {e["kernelFuncName"] for e in cat}
    rng = np.random.default_rng(12)
    n = 96
    a = (rng.standard_normal((n, n)) + n * np.eye(n)).astype(np.float32)
    a[[0, n - 1]] = a[[n - 1, 0]]
    b = rng.standard_normal((n, 1)).astype(np.float32)
    solve = "CUDA_solve__DenseMatrix_float__DenseMatrix_float__DenseMatrix_float"
    gemv = "CUDA_gemv__DenseMatrix_float__DenseMatrix_float__DenseMatrix_float"
    assert solve in names and gemv in names
    out = np.empty((n, 1), dtype=np.float32)
    rc = drv.drv_binary_typed(solve.encode(), 1, _p(a), i64(n), i64(n), _p(b), i64(n), i64(1), None, _p(out))
    assert rc == 0, drv.drv_last_error()
    exact = np.linalg.solve(a.astype(np.float64), b.astype(np.float64))
    assert np.abs(out - exact).max() <= 2.0 ** -22 * np.abs(exact).max()      # one float rounding of the exact solution
    m = rng.standard_normal((500, 40)).astype(np.float32)
    v = rng.standard_normal((500, 1)).astype(np.float32)
    out = np.empty((40, 1), dtype=np.float32)
    rc = drv.drv_binary_typed(gemv.encode(), 1, _p(m), i64(500), i64(40), _p(v), i64(500), i64(1), None, _p(out))
    assert rc == 0, drv.drv_last_error()
    exact = m.astype(np.float64).T @ v.astype(np.float64)
    bound = (500 * 2.0 ** -24 + 2.0 ** -19) * (np.abs(m).astype(np.float64).T @ np.abs(v).astype(np.float64))
    assert np.all(np.abs(out - exact) <= bound)


@pytest.mark.gpu
def test_integer_matmul_by_its_catalog_name(drv):
    """_matMul__DenseMatrix_int64_t__... / _int32_t__... (the reference's Eigen path) are served by the extension
    catalog: bit-exact against the wrapping triple loop, all transpose combinations."""
    from oracle import pyoracle as o
    ext = json.loads((ABI / "B200ExtCatalog.json").read_text())
    names = {e["kernelFuncName"] for e in ext}
    rng = np.random.default_rng(5)
    for vt, dtype, code in (("int64_t", np.int64, 2), ("int32_t", np.int32, 4)):
        name = f"_matMul__DenseMatrix_{vt}__DenseMatrix_{vt}__DenseMatrix_{vt}__bool__bool"
        assert name in names
        for ta in (0, 1):
            for tb in (0, 1):
                a = rng.integers(-2000, 2000, size=(33, 70) if ta else (70, 33)).astype(dtype)
                b = rng.integers(-2000, 2000, size=(45, 33) if tb else (33, 45)).astype(dtype)
                out = np.empty((70, 45), dtype=dtype)
                rc = drv.drv_matmul_int(name.encode(), code, _p(a), i64(a.shape[0]), i64(a.shape[1]), _p(b),
                                        i64(b.shape[0]), i64(b.shape[1]), ta, tb, _p(out))
                assert rc == 0, drv.drv_last_error()
                assert np.array_equal(out, o.matMul(a, b, bool(ta), bool(tb))), (vt, ta, tb)
