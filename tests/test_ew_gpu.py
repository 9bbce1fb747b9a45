"""Parity of the elementwise CUDA kernels with the CPU oracle (EwBinaryMat / EwBinaryObjSca / EwUnaryMat)."""
import numpy as np
import pytest

from tests.util import (RTOL_TRANSCENDENTAL_F32, RTOL_TRANSCENDENTAL_F64, assert_bits_equal, assert_close_rel,
                        rng_matrix)

pytestmark = pytest.mark.gpu

EXACT_BIN = ["ADD", "SUB", "MUL", "DIV", "EQ", "NEQ", "LT", "LE", "GT", "GE", "MIN", "MAX", "AND", "OR"]
SHAPES = [(1, 1), (3, 5), (7, 32), (257, 33), (1000, 64), (4099, 50), (1, 100003), (100003, 1), (513, 1024)]


def _k():
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    return k, o


@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.int64])
@pytest.mark.parametrize("opname", EXACT_BIN)
def test_binary_same_shape_bit_exact(ctx, dtype, opname):
    k, o = _k()
    op = k.BinaryOpCode[opname]
    for i, (r, c) in enumerate(SHAPES):
        a = rng_matrix(10 + i, r, c, dtype)
        b = rng_matrix(20 + i, r, c, dtype)
        if np.dtype(dtype) == np.int64 and opname == "DIV":
            b[b == 0] = 7
        if opname in ("EQ", "NEQ", "LE", "GE", "AND", "OR"):
            b[::2] = a[::2]  # make ties / equalities happen
            a[1::3] = 0
        got = k.ewBinaryMat(op, k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
        assert_bits_equal(got, o.ewBinaryMat(op, a, b), f"{opname} {dtype.__name__} {r}x{c}")


@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.int64])
@pytest.mark.parametrize("opname", ["ADD", "SUB", "MUL", "DIV", "MAX", "MIN", "NEQ", "LE"])
def test_binary_broadcast_bit_exact(ctx, dtype, opname):
    k, o = _k()
    op = k.BinaryOpCode[opname]
    for i, (r, c) in enumerate(SHAPES):
        a = rng_matrix(30 + i, r, c, dtype)
        rv = rng_matrix(40 + i, 1, c, dtype)
        cv = rng_matrix(50 + i, r, 1, dtype)
        if np.dtype(dtype) == np.int64:
            rv[rv == 0] = 3
            cv[cv == 0] = 3
        A = k.DenseMatrix.from_numpy(ctx, a)
        got_r = k.ewBinaryMat(op, A, k.DenseMatrix.from_numpy(ctx, rv)).to_numpy()
        assert_bits_equal(got_r, o.ewBinaryMat(op, a, rv), f"{opname} rowvec {r}x{c}")
        got_c = k.ewBinaryMat(op, A, k.DenseMatrix.from_numpy(ctx, cv)).to_numpy()
        assert_bits_equal(got_c, o.ewBinaryMat(op, a, cv), f"{opname} colvec {r}x{c}")


def test_binary_special_values_bit_exact(ctx):
    k, o = _k()
    sp = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 5e-324, 1.7976931348623157e308, 1e-310, 3.0, 0.1])
    a = np.repeat(sp, len(sp)).reshape(len(sp), len(sp)).copy()
    b = np.tile(sp, len(sp)).reshape(len(sp), len(sp)).copy()
    for opname in ["ADD", "SUB", "MUL", "DIV", "MIN", "MAX", "EQ", "NEQ", "LT", "GE", "AND", "OR"]:
        op = k.BinaryOpCode[opname]
        got = k.ewBinaryMat(op, k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
        exp = o.ewBinaryMat(op, a, b)
        # NaN payload/sign of a produced NaN is not defined by IEEE; compare NaN-ness there and bits elsewhere
        nan = np.isnan(exp)
        assert np.array_equal(np.isnan(got), nan), opname
        assert_bits_equal(np.where(nan, 0.0, got), np.where(nan, 0.0, exp), f"special {opname}")


def test_binary_shape_mismatch_raises(ctx):
    k, o = _k()
    a = k.DenseMatrix.from_numpy(ctx, np.ones((4, 5)))
    b = k.DenseMatrix.from_numpy(ctx, np.ones((3, 2)))
    with pytest.raises(k.Db2Error, match="lhs and rhs must either have the same dimensions"):
        k.ewBinaryMat(k.BinaryOpCode.ADD, a, b)
    with pytest.raises(o.OracleError):
        o.ewBinaryMat(0, np.ones((4, 5)), np.ones((3, 2)))


def test_binary_row_views_keep_their_offset(ctx):
    """A row view of a device-resident matrix must address its own rows (the reference's view returns the parent's
    base pointer, src/runtime/local/datastructures/DenseMatrix.cpp:98-115,235-236)."""
    k, o = _k()
    a = rng_matrix(1, 1000, 32)
    b = rng_matrix(2, 1000, 32)
    A, B = k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)
    A.device_ptr()
    got = k.ewBinaryMat(k.BinaryOpCode.SUB, A.slice_rows(100, 613), B.slice_rows(300, 813)).to_numpy()
    assert_bits_equal(got, a[100:613] - b[300:813], "views")


def test_binary_strided_and_unaligned_host_layouts(ctx):
    k, o = _k()
    big = rng_matrix(3, 300, 40)
    a = big[:, 3:36]  # ld 40, cols 33, first element not 16-byte aligned
    b = rng_matrix(4, 300, 33)
    got = k.ewBinaryMat(k.BinaryOpCode.MUL, k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b))
    assert_bits_equal(got.to_numpy(), a * b, "strided")


@pytest.mark.parametrize("dtype", [np.float64, np.float32, np.int64])
@pytest.mark.parametrize("opname", ["ADD", "SUB", "MUL", "DIV", "MAX", "MIN", "NEQ", "GT", "EQ"])
def test_binary_scalar_bit_exact(ctx, dtype, opname):
    k, o = _k()
    op = k.BinaryOpCode[opname]
    for i, (r, c) in enumerate(SHAPES):
        a = rng_matrix(60 + i, r, c, dtype)
        s = 3 if np.dtype(dtype) == np.int64 else 2.5
        got = k.ewBinaryObjSca(op, k.DenseMatrix.from_numpy(ctx, a), s).to_numpy()
        assert_bits_equal(got, o.ewBinaryObjSca(op, a, s), f"{opname} scalar {r}x{c}")


def test_pow_log_mod_within_ulps(ctx):
    k, o = _k()
    a = np.abs(rng_matrix(70, 513, 37)) + 0.1
    b = rng_matrix(71, 513, 37, kind="uniform") * 3 + 0.5
    A, B = k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)
    for opname in ["POW", "LOG"]:
        op = k.BinaryOpCode[opname]
        assert_close_rel(k.ewBinaryMat(op, A, B).to_numpy(), o.ewBinaryMat(op, a, b), RTOL_TRANSCENDENTAL_F64, opname)
    assert_bits_equal(k.ewBinaryMat(k.BinaryOpCode.MOD, A, B).to_numpy(), o.ewBinaryMat(k.BinaryOpCode.MOD, a, b),
                      "MOD")
    # x^2 (the form the standardisation and k-means scripts use): the device computes the correctly rounded x*x;
    # glibc's pow(x, 2.0) is within 1 ulp of that but not always equal to it, so the bound is 1 ulp (2^-52 relative)
    z = rng_matrix(72, 1000, 32)
    got = k.ewBinaryObjSca(k.BinaryOpCode.POW, k.DenseMatrix.from_numpy(ctx, z), 2.0).to_numpy()
    assert_bits_equal(got, z * z, "POW 2 is the correctly rounded square")
    assert_close_rel(got, o.ewBinaryObjSca(k.BinaryOpCode.POW, z, 2.0), 2.0 ** -52, "POW 2 vs libm")
    got = k.ewBinaryObjSca(k.BinaryOpCode.POW, k.DenseMatrix.from_numpy(ctx, np.abs(z)), 1.7).to_numpy()
    assert_close_rel(got, o.ewBinaryObjSca(k.BinaryOpCode.POW, np.abs(z), 1.7), RTOL_TRANSCENDENTAL_F64, "POW 1.7")


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_unary(ctx, dtype):
    k, o = _k()
    exact = ["MINUS", "ABS", "SIGN", "SQRT", "FLOOR", "CEIL", "ROUND", "ISNAN"]
    approx = ["EXP", "LN", "SIN", "COS", "TAN", "ATAN", "SINH", "COSH", "TANH"]
    rt = RTOL_TRANSCENDENTAL_F64 if dtype == np.float64 else RTOL_TRANSCENDENTAL_F32
    for i, (r, c) in enumerate(SHAPES[:6]):
        a = np.abs(rng_matrix(80 + i, r, c, dtype, kind="uniform")) * 4 + 0.01
        a.reshape(-1)[::7] = 0.0
        a.reshape(-1)[3::11] += 0.5
        A = k.DenseMatrix.from_numpy(ctx, a)
        for name in exact:
            op = k.UnaryOpCode[name]
            src = a if name in ("SQRT",) else (a - 2.0).astype(dtype)
            S = A if name in ("SQRT",) else k.DenseMatrix.from_numpy(ctx, src)
            assert_bits_equal(k.ewUnaryMat(op, S).to_numpy(), o.ewUnaryMat(op, src), f"{name} {r}x{c}")
        for name in approx:
            op = k.UnaryOpCode[name]
            src = (a + 0.5).astype(dtype) if name == "LN" else (a - 2.0).astype(dtype)
            got = k.ewUnaryMat(op, k.DenseMatrix.from_numpy(ctx, src)).to_numpy()
            assert_close_rel(got, o.ewUnaryMat(op, src), rt, f"{name} {r}x{c}", scale=1e-3)
        u = (rng_matrix(90 + i, r, c, dtype, kind="uniform") * 2 - 1).astype(dtype)
        for name in ["ASIN", "ACOS"]:
            op = k.UnaryOpCode[name]
            got = k.ewUnaryMat(op, k.DenseMatrix.from_numpy(ctx, u)).to_numpy()
            assert_close_rel(got, o.ewUnaryMat(op, u), rt, name, scale=1e-3)


def test_unary_domain_error(ctx):
    """sqrt/ln of a negative value and asin/acos outside [-1,1] throw std::domain_error in the reference
    (EwUnarySca.h:134-156,186-195)."""
    k, o = _k()
    a = np.ones((50, 7))
    a[33, 4] = -1e-3
    for name in ["SQRT", "LN"]:
        with pytest.raises(k.Db2Error, match="invalid argument"):
            k.ewUnaryMat(k.UnaryOpCode[name], k.DenseMatrix.from_numpy(ctx, a))
        with pytest.raises(o.OracleError):
            o.ewUnaryMat(k.UnaryOpCode[name], a)
    b = np.zeros((5, 5))
    b[2, 2] = 1.5
    with pytest.raises(k.Db2Error):
        k.ewUnaryMat(k.UnaryOpCode.ASIN, k.DenseMatrix.from_numpy(ctx, b))
    # the context stays usable, -0.0 is inside the domain
    z = np.array([[-0.0, 0.0, 4.0]])
    assert_bits_equal(k.ewUnaryMat(k.UnaryOpCode.SQRT, k.DenseMatrix.from_numpy(ctx, z)).to_numpy(),
                      o.ewUnaryMat(k.UnaryOpCode.SQRT, z), "sqrt after error")


def test_empty_matrices(ctx):
    k, o = _k()
    e = k.DenseMatrix.from_numpy(ctx, np.zeros((0, 5)))
    assert k.ewBinaryMat(k.BinaryOpCode.ADD, e, e).to_numpy().shape == (0, 5)
    assert k.ewBinaryObjSca(k.BinaryOpCode.MUL, e, 2.0).to_numpy().shape == (0, 5)
    assert k.ewUnaryMat(k.UnaryOpCode.ABS, e).to_numpy().shape == (0, 5)


def test_outer_binary_all_opcodes_and_shapes(ctx):
    """OuterBinary.h:52-78 against its restatement: every opcode EwBinaryMat implements, f64 / f32 / i64, empty and
    ragged shapes, a row view as lhs, and the reference's shape errors."""
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    rng = np.random.default_rng(41)
    B = k.BinaryOpCode
    ops = [B.ADD, B.SUB, B.MUL, B.DIV, B.MIN, B.MAX, B.EQ, B.NEQ, B.LT, B.LE, B.GT, B.GE, B.AND, B.OR]
    for dtype in (np.float64, np.float32, np.int64):
        for m, n in [(1, 1), (5, 3), (1000, 33), (70001, 7), (3, 5000), (0, 4), (4, 0)]:
            lhs = (rng.integers(-5, 6, size=(m, 1)) if dtype == np.int64 else rng.standard_normal((m, 1))).astype(dtype)
            rhs = (rng.integers(1, 6, size=(1, n)) if dtype == np.int64 else rng.standard_normal((1, n))).astype(dtype)
            L, R = k.DenseMatrix.from_numpy(ctx, lhs), k.DenseMatrix.from_numpy(ctx, rhs)
            for op in ops:
                got = k.outerBinary(op, L, R).to_numpy()
                if m == 0 or n == 0:
                    assert got.shape == (m, n)
                    continue
                exp = o.outerBinary(int(op), lhs, rhs)
                assert got.shape == exp.shape and got.dtype == exp.dtype
                assert np.array_equal(got, exp, equal_nan=True), (dtype, m, n, op)
    big = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((3000, 1)))
    v = big.slice_rows(100, 2100)
    r = rng.standard_normal((1, 17))
    got = k.outerBinary(B.SUB, v, k.DenseMatrix.from_numpy(ctx, r)).to_numpy()
    assert np.array_equal(got, o.outerBinary(int(B.SUB), big.to_numpy()[100:2100], r))
    M = k.DenseMatrix.from_numpy(ctx, rng.standard_normal((4, 4)))
    with pytest.raises(k.Db2Error, match="lhs must be a column"):
        k.outerBinary(B.ADD, M, k.DenseMatrix.from_numpy(ctx, r))
    with pytest.raises(k.Db2Error, match="rhs must be a row"):
        k.outerBinary(B.ADD, big, M)


def test_cond_four_operand_forms(ctx):
    """CondMatMatMat / CondMatMatSca / CondMatScaMat / CondMatScaSca against their restatement: value types f64, f32,
    i64; conditions f64 (incl. NaN = true, -0.0 = false) and i64; views; the reference's shape errors."""
    import daphne_b200.kernels as k
    from oracle import pyoracle as o
    rng = np.random.default_rng(43)
    for vt in (np.float64, np.float32, np.int64):
        for ct in (np.float64, np.int64):
            for rows, cols in [(1, 1), (7, 5), (1000, 33), (40001, 6), (0, 3)]:
                cnd = rng.integers(-1, 2, size=(rows, cols)).astype(ct)
                if ct == np.float64 and cnd.size:
                    cnd.flat[0] = np.nan
                    cnd.flat[-1] = -0.0
                t = (rng.standard_normal((rows, cols)) * 10).astype(vt)
                e = (rng.standard_normal((rows, cols)) * 10).astype(vt)
                Cn, T, E = (k.DenseMatrix.from_numpy(ctx, a) for a in (cnd, t, e))
                for then, els, dthen, dels in ((T, E, t, e), (T, 2, t, 2), (3, E, 3, e), (3, 2, 3, 2)):
                    got = k.cond(Cn, then, els, dtype=vt).to_numpy()
                    assert got.dtype == np.dtype(vt) and got.shape == (rows, cols)
                    if rows * cols and rows * cols <= 40000:
                        assert np.array_equal(got, o.cond(cnd, dthen, dels, dtype=vt)), (vt, ct, rows, cols)
                    elif rows * cols:
                        tt = dthen if isinstance(dthen, np.ndarray) else np.full((rows, cols), dthen, dtype=vt)
                        ee = dels if isinstance(dels, np.ndarray) else np.full((rows, cols), dels, dtype=vt)
                        assert np.array_equal(got, np.where(cnd != 0, tt, ee))
    big = rng.standard_normal((5000, 8))
    B_ = k.DenseMatrix.from_numpy(ctx, big)
    v = B_.slice_rows(1000, 3000)
    cnd = (rng.random((2000, 8)) < 0.5).astype(np.float64)
    got = k.cond(k.DenseMatrix.from_numpy(ctx, cnd), v, -1.0).to_numpy()
    assert np.array_equal(got, np.where(cnd != 0, big[1000:3000], -1.0))
    with pytest.raises(k.Db2Error, match="CondMatMatMat: condition/then/else matrices must have the same shape"):
        k.cond(k.DenseMatrix.from_numpy(ctx, cnd), B_, B_)
    with pytest.raises(k.Db2Error, match="CondMatMatSca: condition/then matrices must have the same shape"):
        k.cond(k.DenseMatrix.from_numpy(ctx, cnd), B_, 1.0)


def _int_result_equal(op, got, exp, what):
    """Bit-exact, except LOG on integers: the truncated quotient log(a) / log(b) flips by one where it is within an
    ulp of an integer (log_3 9), and the device's log is not the host's to the last bit; there a difference of one
    is accepted (and only there: every other value must be equal)."""
    if op != 6:
        assert_bits_equal(got, exp, what)
        return
    fin = exp.astype(np.float64) < 1e9  # log(a) / log(1) is infinite: its conversion to an integer is undefined
    diff = np.abs(got.astype(np.int64) - exp.astype(np.int64))[fin]
    assert diff.max(initial=0) <= 1 and (diff != 0).mean() < 0.05, what


@pytest.mark.parametrize("dtype", [np.uint64, np.int32, np.uint32])
def test_binary_other_integer_types_bit_exact(ctx, dtype):
    """uint64_t, int32_t and uint32_t: the value types the reference's CUDA library instantiates besides double, float
    and int64_t (kernels/CUDA/EwBinaryMat.cu:265-270, EwBinaryObjSca.cu:89-94); all 17 matrix opcodes and the 18
    scalar opcodes, same shape / row vector / column vector / scalar."""
    from tests.test_oracle_vs_ref import _int_operands
    k, o = _k()
    for i, (r, c) in enumerate([(1, 1), (7, 32), (257, 33), (4099, 50), (1, 100003), (100003, 1)]):
        a, b, rv, cv = _int_operands(dtype, i, r, c)
        for op in range(18):
            x = a
            if op in (4, 5, 6) or (op == 1 and np.dtype(dtype).kind == "u"):
                x = (np.abs(a.astype(np.int64)) % 7 + 9).astype(dtype)
            if op == 4:
                x = (x % 5 + 1).astype(dtype)
            X = k.DenseMatrix.from_numpy(ctx, x)
            if op < 17:
                for rhs in (b, rv, cv):
                    got = k.ewBinaryMat(op, X, k.DenseMatrix.from_numpy(ctx, rhs)).to_numpy()
                    assert got.dtype == np.dtype(dtype)
                    _int_result_equal(op, got, o.ewBinaryMat(op, x, rhs), f"op {op} {np.dtype(dtype).name} {rhs.shape}")
            _int_result_equal(op, k.ewBinaryObjSca(op, X, 3).to_numpy(), o.ewBinaryObjSca(op, x, 3), f"scalar op {op}")
    # wrap-around of unsigned and 32-bit arithmetic
    big = np.array([[np.iinfo(dtype).max, 5, 0, 1]], dtype=dtype)
    one = np.array([[1, 7, 1, 1]], dtype=dtype)
    for op in (0, 2) + ((1,) if np.dtype(dtype).kind == "u" else ()):
        with np.errstate(over="ignore"):
            exp = {0: big + one, 1: big - one * 9, 2: big * (one + 1)}[op]
        rhs = {0: one, 1: (one * 9).astype(dtype), 2: (one + 1).astype(dtype)}[op]
        got = k.ewBinaryMat(op, k.DenseMatrix.from_numpy(ctx, big), k.DenseMatrix.from_numpy(ctx, rhs)).to_numpy()
        assert_bits_equal(got, exp.astype(dtype), f"wrap-around op {op}")
    # unsigned division has no overflow case: (2^63) / (2^64 - 1) is 0
    if dtype == np.uint64:
        a = np.array([[2 ** 63, 2 ** 64 - 1]], dtype=np.uint64)
        b = np.array([[2 ** 64 - 1, 2 ** 63]], dtype=np.uint64)
        got = k.ewBinaryMat(3, k.DenseMatrix.from_numpy(ctx, a), k.DenseMatrix.from_numpy(ctx, b)).to_numpy()
        assert_bits_equal(got, np.array([[0, 1]], dtype=np.uint64), "unsigned division")


def test_fill_and_transpose_of_the_other_value_types(ctx):
    k, _ = _k()
    for dtype, v in ((np.uint64, 2 ** 64 - 3), (np.int32, -7), (np.uint32, 4000000000), (np.uint8, 200)):
        got = k.fill(ctx, v, 37, 5, dtype=dtype).to_numpy()
        assert got.dtype == np.dtype(dtype) and np.all(got == np.array(v, dtype=dtype))
    for dtype in (np.uint64, np.int32, np.uint32):
        a = np.random.default_rng(1).integers(0, 1000, size=(70, 33)).astype(dtype)
        assert_bits_equal(k.transpose(k.DenseMatrix.from_numpy(ctx, a)).to_numpy(), np.ascontiguousarray(a.T),
                          f"transpose {np.dtype(dtype).name}")
