"""ctypes binding of libdaphne_b200.so (the C-ABI declared in include/daphne_b200.h).

There is no CPU fallback: if the shared library is missing the import fails with a message that says how to build it,
and every compute call needs a CUDA device."""
from __future__ import annotations

import atexit
import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libdaphne_b200.so"

# value type codes (include/daphne_b200.h)
F64, F32, I64, U64, I32, U32, U8 = 0, 1, 2, 3, 4, 5, 6


class Db2Error(RuntimeError):
    """A non-zero status from the C-ABI; mirrors the std::runtime_error the reference's kernels throw."""

    def __init__(self, code: int, msg: str):
        super().__init__(msg)
        self.code = code


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m daphne_b200.build` "
            "(needs nvcc; daphne_b200 has no CPU fallback)")
    return C.CDLL(str(LIB_PATH), mode=C.RTLD_GLOBAL)


lib = _load()

i32, i64, u64, sz, vp = C.c_int, C.c_int64, C.c_uint64, C.c_size_t, C.c_void_p
_P = C.POINTER

_SIGS = {
    # name: (restype, argtypes)
    "db2_last_error": (C.c_char_p, []),
    "db2_version": (C.c_char_p, []),
    "db2_device_count": (i32, [_P(i32)]),
    "db2_set_device": (i32, [i32]),
    "db2_sm_count": (i32, [_P(i32)]),
    "db2_malloc": (i32, [_P(vp), sz]),
    "db2_free": (i32, [vp]),
    "db2_malloc_host": (i32, [_P(vp), sz]),
    "db2_free_host": (i32, [vp]),
    "db2_memcpy_h2d": (i32, [vp, vp, sz, vp]),
    "db2_memcpy_d2h": (i32, [vp, vp, sz, vp]),
    "db2_memcpy_d2d": (i32, [vp, vp, sz, vp]),
    "db2_memset": (i32, [vp, i32, sz, vp]),
    "db2_stream_create": (i32, [_P(vp)]),
    "db2_stream_destroy": (i32, [vp]),
    "db2_stream_sync": (i32, [vp]),
    "db2_device_sync": (i32, []),
    "db2_event_create": (i32, [_P(vp)]),
    "db2_event_destroy": (i32, [vp]),
    "db2_event_record": (i32, [vp, vp]),
    "db2_event_elapsed_ms": (i32, [vp, vp, _P(C.c_float)]),
    "db2_launch_count": (u64, []),
    "db2k_ew_binary": (i32, [i32, i32, vp, i64, i64, i64, vp, i64, i64, i64, vp, i64, vp]),
    "db2k_ew_binary_sca": (i32, [i32, i32, vp, i64, i64, i64, vp, vp, i64, vp]),
    "db2k_ew_unary": (i32, [i32, i32, vp, i64, i64, i64, vp, i64, vp, vp]),
    "db2k_agg_row": (i32, [i32, i32, vp, i64, i64, i64, vp, i64, vp]),
    "db2k_agg_col_scratch_bytes": (sz, [i32, i32, i64, i64]),
    "db2k_agg_col": (i32, [i32, i32, vp, i64, i64, i64, vp, vp, sz, vp]),
    "db2k_agg_col_static_max_bytes": (sz, []),
    "db2k_agg_col_static": (i32, [i32, i32, vp, i64, i64, i64, vp, vp]),
    "db2k_agg_all_scratch_bytes": (sz, [i32, i32, i64, i64]),
    "db2k_agg_all": (i32, [i32, i32, vp, i64, i64, i64, vp, vp, sz, vp]),
    "db2k_matmul_scratch_bytes": (sz, [i32, i64, i64, i64]),
    "db2k_matmul": (i32, [i32, vp, i64, i64, i64, vp, i64, i64, i64, i32, i32, vp, i64, vp, sz, vp]),
    "db2k_syrk_scratch_bytes": (sz, [i32, i64, i64, i32]),
    "db2k_syrk": (i32, [i32, vp, i64, i64, i64, i32, vp, i64, vp, sz, vp]),
    "db2k_syrk_gemv_scratch_bytes": (sz, [i64, i64]),
    "db2k_syrk_gemv_supported": (i32, [i64, i64]),
    "db2k_syrk_gemv": (i32, [vp, i64, i64, i64, vp, vp, i64, vp, vp, sz, vp]),
    "db2k_transpose": (i32, [i32, vp, i64, i64, i64, vp, i64, vp]),
    "db2k_fill": (i32, [i32, vp, i64, i64, i64, vp, vp]),
    "db2k_seq": (i32, [i32, vp, i64, vp, vp, vp]),
    "db2k_diag_matrix": (i32, [i32, vp, i64, i64, vp, i64, vp]),
    "db2k_outer_binary": (i32, [i32, i32, vp, i64, i64, vp, i64, vp, i64, vp]),
    "db2k_cond": (i32, [i32, i32, vp, i64, vp, i64, vp, vp, i64, vp, i64, i64, vp, i64, vp]),
    "db2k_agg_cum_scratch_bytes": (sz, [i64, i64]),
    "db2k_agg_cum": (i32, [i32, i32, vp, i64, i64, i64, vp, i64, vp, sz, vp]),
    "db2k_one_hot": (i32, [i32, vp, i64, i64, vp, vp, vp, i64, vp, i64, vp, vp]),
    "db2k_col_bind": (i32, [i32, vp, i64, i64, vp, i64, i64, i64, vp, i64, vp]),
    "db2k_extract_col": (i32, [i32, vp, i64, i64, vp, i64, vp, i64, vp]),
    "db2k_max_i64": (i32, [vp, i64, i64, vp, vp]),
    "db2k_ctable": (i32, [vp, i64, vp, i64, i64, C.c_double, vp, i64, i64, i64, i32, vp]),
    "db2k_solve_scratch_bytes": (sz, [i64]),
    "db2k_solve": (i32, [i32, vp, i64, vp, vp, vp, sz, vp]),
    # runtime
    "db2_context_create": (i32, [i32, _P(vp)]),
    "db2_context_destroy": (i32, [vp]),
    "db2_context_device": (i32, [vp, _P(i32)]),
    "db2_context_ordinal": (i32, [vp, _P(i32)]),
    "db2_context_stream": (vp, [vp]),
    "db2_context_sync": (i32, [vp]),
    "db2_context_stats": (i32, [vp, vp]),
    "db2_context_set_mem_budget": (i32, [vp, sz]),
    "db2_comm_unique_id": (i32, [vp]),
    "db2_comm_init": (i32, [vp, i32, i32, vp]),
    "db2_comm_destroy": (i32, [vp]),
    "db2_comm_info": (i32, [vp, _P(i32), _P(i32)]),
    "db2_allreduce": (i32, [vp, vp, i32]),
    "db2_allreduce_async": (i32, [vp, vp, i32]),
    "db2_comm_group_begin": (i32, [vp]),
    "db2_comm_group_end": (i32, [vp]),
    "db2_allgather_rows": (i32, [vp, vp, _P(vp)]),
    "db2_allgatherv_rows": (i32, [vp, vp, i64, _P(vp)]),
    "db2_group_create": (i32, [_P(i32), i32, _P(vp)]),
    "db2_group_destroy": (i32, [vp]),
    "db2_group_size": (i32, [vp, _P(i32)]),
    "db2_group_context": (i32, [vp, i32, _P(vp)]),
    "db2_group_uses_nccl": (i32, [vp, _P(i32)]),
    "db2_group_sync": (i32, [vp]),
    "db2_dist_from_host": (i32, [vp, i32, i64, i64, i64, vp, _P(vp)]),
    "db2_dist_from_matrix": (i32, [vp, vp, i32, _P(vp)]),
    "db2_dist_from_shards": (i32, [vp, _P(vp), i32, _P(vp)]),
    "db2w_standardise": (i32, [vp, vp, i64, vp, vp, vp, vp, vp, vp, vp, vp]),
    "db2w_standardise_group": (i32, [vp, vp, _P(vp), _P(vp), _P(vp), _P(vp), _P(vp), _P(vp)]),
    "db2_dist_info": (i32, [vp, _P(i32), _P(i64), _P(i64), _P(i32)]),
    "db2_dist_shard": (i32, [vp, i32, _P(vp), _P(i64)]),
    "db2_dist_incref": (i32, [vp]),
    "db2_dist_decref": (i32, [vp]),
    "db2_dist_to_host": (i32, [vp, vp, i64]),
    "db2_dist_gather": (i32, [vp, i32, _P(vp)]),
    "db2_group_run": (i32, [vp, vp, vp]),
    "db2_matrix_to_host_async": (i32, [vp, vp, i64]),
    "db2_context_side_sync": (i32, [vp]),
    "db2_rtc_set_mode": (i32, [i32]),
    "db2_rtc_wait": (i32, []),
    "db2_rtc_counts": (i32, [_P(i32), _P(i32), _P(i32)]),
    "db2_rtc_compile": (i32, [_P(i32), _P(i32), _P(i32), i32, _P(i32), _P(i32), i32, i32, _P(sz)]),
    "db2_group_allreduce": (i32, [vp, _P(vp), i32]),
    "db2_matrix_to_context": (i32, [vp, vp, _P(vp)]),
    "db2_matrix_copy_block": (i32, [vp, i64, i64, vp]),
    "db2_vectorizedPipelineGroup": (i32, [vp, _P(vp), sz, _P(i32), _P(vp), sz, _P(i64), _P(i64), _P(i64), _P(i64), vp,
                                         i64]),
    "db2_matrix_create": (i32, [vp, i32, i64, i64, i32, _P(vp)]),
    "db2_matrix_wrap_host": (i32, [vp, i32, i64, i64, i64, vp, _P(vp)]),
    "db2_matrix_wrap_device": (i32, [vp, i32, i64, i64, i64, vp, _P(vp)]),
    "db2_matrix_slice_rows": (i32, [vp, i64, i64, _P(vp)]),
    "db2_matrix_slice_cols": (i32, [vp, i64, i64, _P(vp)]),
    "db2_sliceRow": (i32, [vp, _P(vp), vp, i64, i64]),
    "db2_sliceCol": (i32, [vp, _P(vp), vp, i64, i64]),
    "db2_randMatrix": (i32, [vp, _P(vp), i32, i64, i64, vp, vp, C.c_double, i64]),
    "db2_matrix_incref": (i32, [vp]),
    "db2_matrix_decref": (i32, [vp]),
    "db2_matrix_info": (i32, [vp, _P(i32), _P(i64), _P(i64)]),
    "db2_matrix_device_ptr": (i32, [vp, _P(vp), _P(i64)]),
    "db2_matrix_to_host": (i32, [vp, vp, i64]),
    "db2_ewBinaryMat": (i32, [vp, i32, _P(vp), vp, vp]),
    "db2_ewBinaryObjSca": (i32, [vp, i32, _P(vp), vp, vp]),
    "db2_ewUnaryMat": (i32, [vp, i32, _P(vp), vp]),
    "db2_aggRow": (i32, [vp, i32, _P(vp), vp]),
    "db2_aggCol": (i32, [vp, i32, _P(vp), vp]),
    "db2_aggAll": (i32, [vp, i32, vp, vp]),
    "db2_aggAllStart": (i32, [vp, i32, vp, i32]),
    "db2_scalarStart": (i32, [vp, vp, i32]),
    "db2_scalarWait": (i32, [vp, i32, vp]),
    "db2_matMul": (i32, [vp, _P(vp), vp, vp, i32, i32]),
    "db2_syrk": (i32, [vp, _P(vp), vp, i32]),
    "db2_gemv": (i32, [vp, _P(vp), vp, vp]),
    "db2_solve": (i32, [vp, _P(vp), vp, vp]),
    "db2_transpose": (i32, [vp, _P(vp), vp]),
    "db2_fill": (i32, [vp, _P(vp), i32, vp, i64, i64]),
    "db2_seq": (i32, [vp, _P(vp), i32, vp, vp, vp]),
    "db2_diagMatrix": (i32, [vp, _P(vp), vp]),
    "db2_colBind": (i32, [vp, _P(vp), vp, vp]),
    "db2_oneHot": (i32, [vp, _P(vp), vp, vp]),
    "db2_aggCum": (i32, [vp, i32, _P(vp), vp]),
    "db2_cond": (i32, [vp, _P(vp), i32, vp, vp, vp, vp, vp]),
    "db2_outerBinary": (i32, [vp, i32, _P(vp), vp, vp]),
    "db2_extractCol": (i32, [vp, _P(vp), vp, vp]),
    "db2_ctable": (i32, [vp, _P(vp), vp, vp, C.c_double, i64, i64]),
    "db2_castObj": (i32, [vp, _P(vp), vp, i32]),
    "db2_readDaphne": (i32, [vp, _P(vp), C.c_char_p]),
    "db2_writeDaphne": (i32, [vp, vp, C.c_char_p]),
    "db2_vectorizedPipeline": (i32, [vp, _P(vp), sz, _P(i32), _P(vp), sz, _P(i64), _P(i64), _P(i64), _P(i64), vp, i64]),
    "db2w_connected_components": (i32, [vp, vp, i64, i64, _P(vp), _P(i64)]),
    "db2w_kmeans": (i32, [vp, vp, vp, i32, _P(vp), _P(vp)]),
    "db2w_normal_equations": (i32, [vp, vp, vp, C.c_double, _P(vp), _P(vp), _P(vp)]),
    "db2_csr_wrap_host": (i32, [vp, i32, i64, i64, vp, vp, vp, _P(vp)]),
    "db2_csr_slice_rows": (i32, [vp, i64, i64, _P(vp)]),
    "db2_csr_incref": (i32, [vp]),
    "db2_csr_decref": (i32, [vp]),
    "db2_csr_info": (i32, [vp, _P(i64), _P(i64), _P(i64)]),
    "db2_csr_to_host": (i32, [vp, vp, vp, vp]),
    "db2_ewMulCsrDense": (i32, [vp, _P(vp), vp, vp]),
    "db2_aggRowCsr": (i32, [vp, i32, _P(vp), vp]),
    "db2_matMulCsrDense": (i32, [vp, _P(vp), vp, vp]),
}


class Stats(C.Structure):
    """db2_stats (include/daphne_b200.h)."""
    _fields_ = [(n, C.c_uint64) for n in ("h2d_bytes", "d2h_bytes", "d2d_bytes", "allocs", "alloc_bytes", "frees",
                                          "launches", "live_bytes", "peak_bytes", "collectives",
                                          "collective_bytes")]


def declare(sigs: dict) -> None:
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)  # AttributeError here = the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args


declare(_SIGS)

# a background compilation of a chain's kernel (db2_rtc_set_mode(1)) must have finished before the process ends
atexit.register(lib.db2_rtc_wait)


def exported_symbols() -> list[str]:
    return sorted(_SIGS)


def last_error() -> str:
    return (lib.db2_last_error() or b"").decode("utf-8", "replace")


def check(rc: int) -> None:
    if rc != 0:
        raise Db2Error(rc, last_error())


def device_count() -> int:
    n = i32(0)
    rc = lib.db2_device_count(C.byref(n))
    return n.value if rc == 0 else 0


def require_device() -> None:
    if device_count() < 1:
        raise Db2Error(2, "daphne_b200 needs a CUDA device (there is no CPU fallback)")
