"""The allocation-free column aggregation (db2k_agg_col_static) against the ordinary entry point (db2k_agg_col).

Some callers cannot allocate device memory at the point of the call (host callbacks, code that must not touch the
allocator inside a latency-critical loop, embedders with a fixed memory budget).  For them the library keeps the
scratch of the column aggregation in a fixed 4 MiB device array; this test drives that entry point through the C-ABI
on device buffers the TEST allocates, twice in a row on different inputs (the array is shared between calls and keeps
old contents), and requires the results of the ordinary entry point: bit-identical for MIN/MAX/IDXMIN/IDXMAX, within
the 1e-12 relative tolerance of the f64 reductions otherwise.  Collected last on purpose (file name)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(lib, check, a):
    p = C.c_void_p()
    check(lib.db2_malloc(C.byref(p), max(a.nbytes, 16)))
    check(lib.db2_memcpy_h2d(p, C.c_void_p(a.ctypes.data), a.nbytes, None))
    return p


def test_static_scratch_column_aggregation_matches_the_allocating_entry_point_twice_in_a_row():
    from daphne_b200.lib import Db2Error, check, lib
    assert lib.db2k_agg_col_static_max_bytes() == 4 << 20
    rng = np.random.default_rng(11)
    inputs = [5.0 + 2.0 * rng.standard_normal((50021, 32)), rng.standard_normal((777, 200)) * 1e3]
    held = []
    for call, a in enumerate(inputs):
        rows, cols = a.shape
        d_in = _dev(lib, check, a)
        held.append(d_in)
        sb = lib.db2k_agg_col_scratch_bytes(0, 0, rows, cols)
        assert sb <= lib.db2k_agg_col_static_max_bytes()
        scratch, r0, r1 = C.c_void_p(), C.c_void_p(), C.c_void_p()
        for p, n in ((scratch, sb), (r0, cols * 8), (r1, cols * 8)):
            check(lib.db2_malloc(C.byref(p), n))
            held.append(p)
        for op in (0, 2, 3, 4, 5, 6, 7, 8):  # SUM MIN MAX IDXMIN IDXMAX MEAN STDDEV VAR
            check(lib.db2k_agg_col(0, op, d_in, rows, cols, cols, r0, scratch, sb, None))
            check(lib.db2k_agg_col_static(0, op, d_in, rows, cols, cols, r1, None))
            check(lib.db2_device_sync())
            dt = np.uint64 if op in (4, 5) else np.float64
            x, y = np.empty(cols, dtype=dt), np.empty(cols, dtype=dt)
            check(lib.db2_memcpy_d2h(C.c_void_p(x.ctypes.data), r0, cols * 8, None))
            check(lib.db2_memcpy_d2h(C.c_void_p(y.ctypes.data), r1, cols * 8, None))
            check(lib.db2_device_sync())
            if op in (2, 3, 4, 5):
                assert np.array_equal(x, y), f"call {call} op {op}"
            else:
                np.testing.assert_allclose(y, x, rtol=1e-12, atol=0, err_msg=f"call {call} op {op}")
        # and against numpy, so that both being wrong the same way cannot pass
        check(lib.db2k_agg_col_static(0, 0, d_in, rows, cols, cols, r1, None))
        check(lib.db2_device_sync())
        y = np.empty(cols)
        check(lib.db2_memcpy_d2h(C.c_void_p(y.ctypes.data), r1, cols * 8, None))
        check(lib.db2_device_sync())
        np.testing.assert_allclose(y, a.sum(axis=0), rtol=1e-12, atol=1e-9)
    # beyond the fixed array: rejected with a clear message, nothing launched
    wide = C.c_void_p()
    check(lib.db2_malloc(C.byref(wide), 8 * 4 * 4096))
    held.append(wide)
    with pytest.raises(Db2Error, match="built-in array holds"):
        check(lib.db2k_agg_col_static(0, 0, wide, 4, 4096, 4096, wide, None))
    for p in held:
        lib.db2_free(p)
