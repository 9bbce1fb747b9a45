"""Error paths that a healthy run never takes, provoked on the HOST: a collective library whose calls fail, an
allocator that runs out of budget, a shard of the wrong height.  Nothing here faults, traps or hangs a GPU."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NCCL_SYSTEM_ERROR = 2


def _fake_table(fail: bool):
    """Stand-ins with NCCL's signatures; they copy nothing and return success or ncclSystemError."""
    rc = NCCL_SYSTEM_ERROR if fail else 0
    sz, vp, i = C.c_size_t, C.c_void_p, C.c_int
    allreduce = C.CFUNCTYPE(i, vp, vp, sz, i, i, vp, vp)(lambda *a: rc)
    allgather = C.CFUNCTYPE(i, vp, vp, sz, i, vp, vp)(lambda *a: rc)
    broadcast = C.CFUNCTYPE(i, vp, vp, sz, i, i, vp, vp)(lambda *a: rc)
    gstart = C.CFUNCTYPE(i)(lambda: 0)
    gend = C.CFUNCTYPE(i)(lambda: 0)
    fns = (allreduce, allgather, broadcast, gstart, gend)
    table = (C.c_void_p * 5)(*[C.cast(f, C.c_void_p) for f in fns])
    return table, fns


def test_a_failing_collective_is_reported_as_enccl():
    import daphne_b200.kernels as k
    from daphne_b200.lib import lib
    lib.db2_comm_test_override.argtypes = [C.c_void_p]
    lib.db2_comm_test_attach.argtypes = [C.c_void_p, C.c_int, C.c_int]
    c = k.Context(0)
    try:
        table, keep = _fake_table(fail=True)
        assert lib.db2_comm_test_override(table) == 0
        assert lib.db2_comm_test_attach(c.handle, 1, 3) == 0
        m = k.DenseMatrix.from_numpy(c, np.ones((1, 8)))
        with pytest.raises(k.Db2Error) as e:
            k.check(lib.db2_allreduce(c.handle, m.handle, 3))
        assert e.value.code == 6 and "AllReduce" in str(e.value)
        # rank 1 of 3 over 10 rows holds 3 rows: a 4-row shard is refused before the collective
        bad = k.DenseMatrix.from_numpy(c, np.ones((4, 1)))
        h = C.c_void_p()
        with pytest.raises(k.Db2Error) as e:
            k.check(lib.db2_allgatherv_rows(c.handle, bad.handle, 10, C.byref(h)))
        assert e.value.code == 1 and "holds 4 rows" in str(e.value)
        ok = k.DenseMatrix.from_numpy(c, np.ones((3, 1)))
        with pytest.raises(k.Db2Error) as e:  # ragged blocks: grouped broadcasts, which fail here
            k.check(lib.db2_allgatherv_rows(c.handle, ok.handle, 10, C.byref(h)))
        assert e.value.code == 6
        # the same calls succeed with a library that works, and the context stays usable
        table2, keep2 = _fake_table(fail=False)
        assert lib.db2_comm_test_override(table2) == 0
        k.check(lib.db2_allreduce(c.handle, m.handle, 3))
        assert np.array_equal(m.to_numpy(), np.ones((1, 8)))
    finally:
        lib.db2_comm_test_attach(c.handle, 0, 1)
        lib.db2_comm_test_override(None)
        c.close()


def test_an_exhausted_memory_budget_is_reported_as_enomem():
    import daphne_b200.kernels as k
    from daphne_b200.lib import lib
    c = k.Context(0)
    try:
        k.check(lib.db2_context_set_mem_budget(c.handle, 8 << 20))
        small = k.DenseMatrix.empty(c, 1000, 100)          # 0.8 MB fits
        with pytest.raises(k.Db2Error) as e:
            k.DenseMatrix.empty(c, 4000, 1000)             # 32 MB does not
        assert e.value.code == 3 and "budget" in str(e.value)
        x = np.ones((3000, 1000))
        with pytest.raises(k.Db2Error) as e:               # neither does the device placement of a host matrix
            k.aggCol(k.AggOpCode.SUM, k.DenseMatrix.from_numpy(c, x))
        assert e.value.code == 3
        k.check(lib.db2_context_set_mem_budget(c.handle, 0))
        got = k.aggCol(k.AggOpCode.SUM, k.DenseMatrix.from_numpy(c, x)).to_numpy()
        assert np.array_equal(got, np.full((1, 1000), 3000.0))
        small.free()
    finally:
        c.close()


def test_a_bounded_wait_that_runs_out_is_reported_as_etimeout():
    """The tcgen05 kernel of the f32 matMul bounds every mbarrier wait.  With the MMA issuer switched off (a barrier
    that nothing completes) and the limit shortened to about a millisecond, the waits of the other roles run out: the
    kernel must leave through its common exit, release its tensor memory and raise the status bit, the call must
    return DB2_ETIMEOUT, and the next product on the same context must be correct."""
    import daphne_b200.kernels as k
    from daphne_b200.lib import lib
    lib.db2k_test_tf32_starve.argtypes = [C.c_longlong, C.c_int]
    c = k.Context(0)
    try:
        rng = np.random.default_rng(0)
        a = rng.standard_normal((512, 640)).astype(np.float32)
        b = rng.standard_normal((640, 384)).astype(np.float32)
        A, B = k.DenseMatrix.from_numpy(c, a), k.DenseMatrix.from_numpy(c, b)
        ok = k.matMul(A, B).to_numpy()
        assert lib.db2k_test_tf32_starve(2_000_000, 1) == 0
        try:
            with pytest.raises(k.Db2Error) as e:
                k.matMul(A, B)
            assert e.value.code == 7 and "gave up waiting" in str(e.value)
        finally:
            assert lib.db2k_test_tf32_starve(0, 0) == 0
        again = k.matMul(A, B).to_numpy()
        assert np.array_equal(again, ok), "the context is usable and tensor memory was released"
        np.testing.assert_allclose(again, a.astype(np.float64) @ b.astype(np.float64), rtol=2e-4, atol=2e-3)
    finally:
        c.close()
