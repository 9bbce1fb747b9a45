/*
 * daphne_b200 -- B200-native (sm_100a) runtime kernel library for the kernels
 * that DAPHNE's vectorized pipelines execute.
 *
 * This header is the C-ABI boundary: plain pointers and sizes, no C++ or torch
 * types.  It has three layers:
 *
 *   db2k_*  kernel launchers on DEVICE pointers (one per reference kernel
 *           template registered in src/runtime/local/kernels/kernels.json),
 *   db2_*   the runtime: context (device, stream, pooled device memory),
 *           matrix handles with host/device residency, operator calls on
 *           handles, and the row-partition pipeline scheduler,
 *   db2h_*  host-buffer conveniences (copy in, run, copy out) used by the
 *           end-to-end measurement.
 *
 * The DAPHNE-named entry points (CUDA_sumRow__DenseMatrix_double__... etc.),
 * which take DAPHNE's C++ data objects, live in the adapter library built from
 * daphne_b200/csrc/daphne_abi/ against a DAPHNE source tree; they forward to
 * the functions declared here.
 *
 * Conventions
 *   - every function returns 0 on success, a DB2_E* code otherwise;
 *     db2_last_error() returns the message of the calling thread's last error
 *     (the reference reports errors as C++ exceptions: the adapter rethrows the
 *     message as std::runtime_error, like
 *     src/runtime/local/kernels/CUDA/HostUtils.h:37-80 does for CUDA errors);
 *   - matrices are row-major with a leading dimension `ld` in ELEMENTS
 *     (DenseMatrix::getRowSkip(), src/runtime/local/datastructures/DenseMatrix.h:42-62);
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream);
 *   - op codes are the reference's enum values
 *     (BinaryOpCode.h:29-56, UnaryOpCode.h:26-56, AggOpCode.h:25-35).
 */
#ifndef DAPHNE_B200_H
#define DAPHNE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------- */
/* enums                                                                      */
/* ------------------------------------------------------------------------- */

enum { DB2_OK = 0, DB2_EINVAL = 1, DB2_ECUDA = 2, DB2_ENOMEM = 3, DB2_EUNSUPPORTED = 4, DB2_EDOMAIN = 5,
       DB2_ENCCL = 6, DB2_ETIMEOUT = 7 };

/* value types (kernels.json instantiates the hot kernels for double, float, int64_t; size_t is the value type of
 * idxMin/idxMax results, AggRow.h:71-96).  The elementwise binary kernels (matrix and scalar rhs), fill and transpose
 * also take uint64_t, int32_t and uint32_t like the reference's CUDA instantiations (kernels/CUDA/EwBinaryMat.cu:265-270,
 * EwBinaryObjSca.cu:89-94); DB2_U8 (uint8_t and bool) exists for fill only (CUDA/Fill.cu:44-49). */
enum { DB2_F64 = 0, DB2_F32 = 1, DB2_I64 = 2, DB2_U64 = 3, DB2_I32 = 4, DB2_U32 = 5, DB2_U8 = 6 };

/* BinaryOpCode (src/runtime/local/kernels/BinaryOpCode.h:29-56) */
enum { DB2_ADD = 0, DB2_SUB, DB2_MUL, DB2_DIV, DB2_POW, DB2_MOD, DB2_LOG, DB2_EQ, DB2_NEQ, DB2_LT, DB2_LE, DB2_GT,
       DB2_GE, DB2_MIN, DB2_MAX, DB2_AND, DB2_OR, DB2_BITWISE_AND };

/* UnaryOpCode (src/runtime/local/kernels/UnaryOpCode.h:26-56) */
enum { DB2_U_MINUS = 0, DB2_U_ABS, DB2_U_SIGN, DB2_U_SQRT, DB2_U_EXP, DB2_U_LN, DB2_U_SIN, DB2_U_COS, DB2_U_TAN,
       DB2_U_ASIN, DB2_U_ACOS, DB2_U_ATAN, DB2_U_SINH, DB2_U_COSH, DB2_U_TANH, DB2_U_FLOOR, DB2_U_CEIL,
       DB2_U_ROUND, DB2_U_ISNAN };

/* AggOpCode (src/runtime/local/kernels/AggOpCode.h:25-35) */
enum { DB2_AGG_SUM = 0, DB2_AGG_PROD, DB2_AGG_MIN, DB2_AGG_MAX, DB2_AGG_IDXMIN, DB2_AGG_IDXMAX, DB2_AGG_MEAN,
       DB2_AGG_STDDEV, DB2_AGG_VAR };

/* VectorSplit / VectorCombine (src/ir/daphneir/DaphneVectorizableOpInterface.td:23-36) */
enum { DB2_SPLIT_NONE = 0, DB2_SPLIT_ROWS = 1 };
enum { DB2_COMBINE_ROWS = 1, DB2_COMBINE_COLS = 2, DB2_COMBINE_ADD = 3, DB2_COMBINE_MIN = 4, DB2_COMBINE_MAX = 5 };

/* ------------------------------------------------------------------------- */
/* errors, device memory helpers                                              */
/* ------------------------------------------------------------------------- */

const char *db2_last_error(void);
const char *db2_version(void);
int db2_device_count(int *count);
int db2_set_device(int device);
int db2_sm_count(int *count);

int db2_malloc(void **dptr, size_t bytes);                /* cudaMalloc                    */
int db2_free(void *dptr);                                 /* cudaFree                      */
int db2_malloc_host(void **hptr, size_t bytes);           /* pinned host memory            */
int db2_free_host(void *hptr);
int db2_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream);
int db2_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream);
int db2_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream);
int db2_memset(void *dst, int byte, size_t bytes, void *stream);
int db2_stream_create(void **stream);
int db2_stream_destroy(void *stream);
int db2_stream_sync(void *stream);
int db2_device_sync(void);
/* CUDA-event timing on a stream (used by the measurement harness). */
int db2_event_create(void **event);
int db2_event_destroy(void *event);
int db2_event_record(void *event, void *stream);
int db2_event_elapsed_ms(void *start, void *stop, float *ms); /* synchronises on `stop` */
/* number of kernels this library launched since load (all threads) */
uint64_t db2_launch_count(void);

/* ------------------------------------------------------------------------- */
/* db2k_*: kernel launchers on device pointers                                */
/* ------------------------------------------------------------------------- */

/* res = lhs op rhs.  rhs has the shape of lhs, or is a 1 x cols row vector, or a rows x 1 column vector;
 * the result has the shape of lhs.  Replaces EwBinaryMat<Dense,Dense,Dense>
 * (src/runtime/local/kernels/EwBinaryMat.h:54-108; CUDA twin kernels/CUDA/EwBinaryMat.cu:97-263).
 * Comparison results are 0/1 in the value type. */
int db2k_ew_binary(int dtype, int op, const void *lhs, int64_t lhs_rows, int64_t lhs_cols, int64_t lhs_ld,
                   const void *rhs, int64_t rhs_rows, int64_t rhs_cols, int64_t rhs_ld, void *res, int64_t res_ld,
                   void *stream);

/* res[r][c] = lhs[r] (op) rhs[c] for a column vector lhs (rows elements, stride lhs_ld) and a row vector rhs (cols
 * elements).  Replaces OuterBinary<Dense,Dense,Dense> (src/runtime/local/kernels/OuterBinary.h:52-78; no CUDA twin). */
int db2k_outer_binary(int dtype, int op, const void *lhs, int64_t lhs_ld, int64_t rows, const void *rhs, int64_t cols,
                      void *res, int64_t res_ld, void *stream);
/* res = lhs op scalar; `scalar` is a HOST pointer to one value of `dtype`.  Replaces EwBinaryObjSca<Dense,Dense,VT>
 * (src/runtime/local/kernels/EwBinaryObjSca.h:58-79; CUDA twin kernels/CUDA/EwBinaryObjSca.cu:31-88). */
int db2k_ew_binary_sca(int dtype, int op, const void *lhs, int64_t rows, int64_t cols, int64_t ld,
                       const void *scalar, void *res, int64_t res_ld, void *stream);

/* res = f(arg).  Replaces EwUnaryMat<Dense,Dense> (src/runtime/local/kernels/EwUnaryMat.h:57-77; scalar functions
 * EwUnarySca.h:182-206).  SQRT/LN of a negative value and ASIN/ACOS outside [-1,1] are domain errors in the
 * reference (EwUnarySca.h:134-156): the kernel then sets *dev_status (a device int32, may be NULL) to 1 and the
 * caller reports DB2_EDOMAIN after synchronising. */
int db2k_ew_unary(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                  int64_t res_ld, int32_t *dev_status, void *stream);

/* Row aggregation -> rows x 1 (ld = res_ld).  SUM/PROD/MIN/MAX/MEAN/STDDEV/VAR results have value type `dtype`;
 * IDXMIN/IDXMAX results are uint64 and ties go to the lowest index.  Replaces AggRow<Dense,Dense>
 * (src/runtime/local/kernels/AggRow.h:60-161; CUDA twin kernels/CUDA/AggRow.cu:108-143). */
int db2k_agg_row(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                 int64_t res_ld, void *stream);

/* Column aggregation -> 1 x cols.  Same result types as db2k_agg_row.  VAR/STDDEV are the population two-pass
 * form of the reference.  `scratch` is device memory of at least db2k_agg_col_scratch_bytes() bytes.
 * Replaces AggCol<Dense,Dense> (src/runtime/local/kernels/AggCol.h:58-178; CUDA twin kernels/CUDA/AggCol.cu:45-86). */
size_t db2k_agg_col_scratch_bytes(int dtype, int op, int64_t rows, int64_t cols);
int db2k_agg_col(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                 void *scratch, size_t scratch_bytes, void *stream);

/* Column aggregation that allocates nothing (no counterpart in the reference).
 *
 * For callers that are not allowed to allocate device memory at the point of the call: code running inside a
 * host callback or another context where cudaMalloc is forbidden or would synchronise the device, latency-critical
 * loops that must not touch the allocator, and embedders that hand this library a fixed memory budget up front.
 * The scratch that db2k_agg_col takes from the caller lives here in one fixed array of
 * db2k_agg_col_static_max_bytes() (4 MiB) in device memory, which every GPU that loads the library holds until the
 * process exits.  Inputs and outputs are still the caller's.
 *   - Limit: db2k_agg_col_scratch_bytes(dtype, op, rows, cols) must fit the array (about 220 f64 columns on a
 *     148-SM device); wider matrices are rejected with DB2_EINVAL and a message, nothing is launched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents (every partial is rewritten before
 *     it is read, so nothing needs clearing); two calls that may overlap on the GPU (different streams without
 *     ordering) race on it -- serialise them.
 *   - Calls no cudaMalloc/cudaFree and no allocating library routine.  Same kernels and results as db2k_agg_col. */
size_t db2k_agg_col_static_max_bytes(void);
int db2k_agg_col_static(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                        void *stream);

/* Full aggregation -> one DEVICE scalar of `dtype`.  Replaces AggAll<VT,Dense>
 * (src/runtime/local/kernels/AggAll.h:124-193; CUDA twin kernels/CUDA/AggAll.cu:109-151). */
size_t db2k_agg_all_scratch_bytes(int dtype, int op, int64_t rows, int64_t cols);
int db2k_agg_all(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                 void *scratch, size_t scratch_bytes, void *stream);

/* res (m x n) = op(lhs) op(rhs), op = transpose iff the flag is set; double or float.  DB2_F64: FP64 tensor-core
 * (DMMA) kernel.  DB2_F32: tcgen05 kind::tf32 kernel with split operands (three MMAs per product, single-precision
 * accuracy); `scratch` is then always required, and its first 4 bytes receive a status word when the launch has
 * finished: bit 0 = a bounded wait inside the kernel expired (the result is not valid), bit 1 = a result was
 * inf / NaN and the product was recomputed by a plain FMA kernel (not an error).
 * Contractions over a long row range (t(A) B with tall operands) are split over the grid and reduced in a fixed
 * order through `scratch` (db2k_matmul_scratch_bytes(dtype, m, n, k) bytes, m/n/k = the product's dimensions).
 * Replaces MatMul<Dense,Dense,Dense> (src/runtime/local/kernels/MatMul.cpp:248-290: cblas_ddot / dgemv / dgemm;
 * CUDA twin kernels/CUDA/MatMul.cpp:45-91: cuBLAS gemm). */
size_t db2k_matmul_scratch_bytes(int dtype, int64_t m, int64_t n, int64_t k);
int db2k_matmul(int dtype, const void *lhs, int64_t lhs_rows, int64_t lhs_cols, int64_t lhs_ld, const void *rhs,
                int64_t rhs_rows, int64_t rhs_cols, int64_t rhs_ld, int transa, int transb, void *res,
                int64_t res_ld, void *scratch, size_t scratch_bytes, void *stream);

/* res (n x n, full symmetric) = t(arg) arg if trans_left else arg t(arg); double or float (float: the tcgen05
 * kernel of db2k_matmul on the full square, scratch and status word as there; the lower triangle is the mirror of the
 * upper one).  For double only the tiles on and above the diagonal are computed, the rest is mirrored.  Replaces Syrk<Dense,Dense> (src/runtime/local/kernels/Syrk.h:51-71:
 * cblas_dsyrk + mirror loop; CUDA twin kernels/CUDA/Syrk.cu:54-87). */
size_t db2k_syrk_scratch_bytes(int dtype, int64_t rows, int64_t cols, int trans_left);
int db2k_syrk(int dtype, const void *arg, int64_t rows, int64_t cols, int64_t ld, int trans_left, void *res,
              int64_t res_ld, void *scratch, size_t scratch_bytes, void *stream);
/* t(X) X and t(X) y in ONE pass over X (f64, more than 64 columns; the reference calls syrk and gemv, Syrk.h:40-43 and
 * Gemv.h:51-63, and reads X for each): the warps of the diagonal tiles that have no sub-tile to compute form the products
 * with y from the operand stages that pass through shared memory anyway.  res: cols x cols; yvec: rows contiguous
 * doubles (16-byte aligned); yres: cols contiguous doubles. */
size_t db2k_syrk_gemv_scratch_bytes(int64_t rows, int64_t cols);
int db2k_syrk_gemv_supported(int64_t rows, int64_t cols);
int db2k_syrk_gemv(const void *arg, int64_t rows, int64_t cols, int64_t ld, const void *yvec, void *res, int64_t res_ld,
                   void *yres, void *scratch, size_t scratch_bytes, void *stream);

/* Out-of-place transpose (any 4- or 8-byte value type).  Replaces Transpose<Dense,Dense>
 * (src/runtime/local/kernels/Transpose.h:51-76; CUDA twin kernels/CUDA/Transpose.cpp:70-90: cuBLAS geam). */
int db2k_transpose(int dtype, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res, int64_t res_ld,
                   void *stream);
/* Constant fill; `value` is a host pointer to one element.  Replaces Fill (kernels/Fill.h; CUDA/Fill.cu:29-42). */
int db2k_fill(int dtype, void *res, int64_t rows, int64_t cols, int64_t ld, const void *value, void *stream);
/* res[i] = start + i * inc for i < n (Seq, src/runtime/local/kernels/Seq.h:49-99; n is computed by the caller). */
int db2k_seq(int dtype, void *res, int64_t n, const void *start, const void *inc, void *stream);
/* n x n matrix with vec on its diagonal (DiagMatrix<Dense,Dense>, src/runtime/local/kernels/DiagMatrix.h:55-78). */
int db2k_diag_matrix(int dtype, const void *vec, int64_t vec_ld, int64_t n, void *res, int64_t res_ld, void *stream);
/* res (rows x (lhs_cols + rhs_cols)) = [lhs | rhs].  Replaces ColBind<Dense,Dense,Dense>
 * (src/runtime/local/kernels/ColBind.h:54-88; CUDA twin kernels/CUDA/ColBind.cu:24-75). */
int db2k_col_bind(int dtype, const void *lhs, int64_t lhs_ld, int64_t lhs_cols, const void *rhs, int64_t rhs_ld,
                  int64_t rhs_cols, int64_t rows, void *res, int64_t res_ld, void *stream);
/* res[:, c] = arg[:, positions[c]] for c < nsel; `dev_positions` are nsel int64 column positions on the device,
 * already resolved and inside [0, cols) (the caller validates them, see db2_extractCol).  Replaces
 * ExtractCol<Dense,Dense,Dense<int64>> (src/runtime/local/kernels/ExtractCol.h:64-105; CUDA twin
 * kernels/CUDA/ExtractCol.cu:22-66). */
int db2k_extract_col(int dtype, const void *arg, int64_t ld, int64_t rows, const void *dev_positions, int64_t nsel,
                     void *res, int64_t res_ld, void *stream);
/* res = cond ? then : else, element by element.  then_m / else_m are matrices of the shape of cond (value type
 * `dtype`) or NULL, in which case the host scalar then_s / else_s (one element of `dtype`) is used; cond has value
 * type cond_dtype and picks with static_cast<bool>.  Replaces CondMatMatMat / CondMatMatSca / CondMatScaMat /
 * CondMatScaSca<Dense...> (src/runtime/local/kernels/CondMatMatMat.h:50-83 and the three siblings; no CUDA twin). */
int db2k_cond(int dtype, int cond_dtype, const void *cond, int64_t cond_ld, const void *then_m, int64_t then_ld,
              const void *then_s, const void *else_m, int64_t else_ld, const void *else_s, int64_t rows, int64_t cols,
              void *res, int64_t res_ld, void *stream);
/* Cumulative aggregation down the rows: res[0] = arg[0], res[r] = f(res[r-1], arg[r]) per column; op is the
 * AggOpCode SUM (0), PROD (1), MIN (2) or MAX (3).  Blocked scan: floating-point sums / products are rounded in a
 * different order than the sequential loop, MIN / MAX and integer types are exact.  `scratch`: device memory of
 * db2k_agg_cum_scratch_bytes(rows, cols).  Replaces AggCum<Dense,Dense> (src/runtime/local/kernels/AggCum.h:48-86;
 * no CUDA twin). */
size_t db2k_agg_cum_scratch_bytes(int64_t rows, int64_t cols);
int db2k_agg_cum(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res, int64_t res_ld,
                 void *scratch, size_t scratch_bytes, void *stream);
/* One-hot encoding with a prepared column table on the device: result column j copies argument column src[j] when
 * hot[j] < 0, else it is (integer part of arg[:, src[j]] == hot[j]); width[j] = size of j's block; *dev_status is set
 * to 1 when a value lies outside its block.  f64 and int64.  Replaces OneHot<Dense,Dense>
 * (src/runtime/local/kernels/OneHot.h:54-110; no CUDA twin). */
int db2k_one_hot(int dtype, const void *arg, int64_t ld, int64_t rows, const void *dev_src, const void *dev_hot,
                 const void *dev_width, int64_t cols_res, void *res, int64_t res_ld, void *dev_status, void *stream);
/* maximum of an int64 vector into a device int64 (used to size ctable results like CTable.h:79-84 does) */
int db2k_max_i64(const void *vec, int64_t ld, int64_t n, void *dev_out, void *stream);
/* Contingency table res[lhs[i], rhs[i]] += weight over int64 coordinate vectors (f64 result, overwritten).
 * Coordinates outside res are ignored.  lhs_is_row_index != 0 promises lhs = 0,1,..,n-1 (the one-hot use).
 * Replaces CTable<Dense<double>,Dense<int64>,Dense<int64>,double> (src/runtime/local/kernels/CTable.h:55-106). */
int db2k_ctable(const void *lhs, int64_t lhs_ld, const void *rhs, int64_t rhs_ld, int64_t n, double weight, void *res,
                int64_t res_rows, int64_t res_cols, int64_t res_ld, int lhs_is_row_index, void *stream);
/* Solves A x = b by blocked LU with partial pivoting.  a_work: n x n row-major COPY of A (destroyed); x_inout: b on
 * entry, x on exit; *dev_status (device int32) = 0, or k+1 if U(k,k) is exactly zero; scratch: device memory of
 * db2k_solve_scratch_bytes(n) bytes (pivot indices).  Replaces Solve<Dense,Dense,Dense>
 * (src/runtime/local/kernels/Solve.h:86-116: LAPACKE_dgesv; CUDA twin kernels/CUDA/Solve.cpp:75-151). */
size_t db2k_solve_scratch_bytes(int64_t n);
int db2k_solve(int dtype, void *a_work, int64_t n, void *x_inout, int32_t *dev_status, void *scratch,
               size_t scratch_bytes, void *stream);

/* ------------------------------------------------------------------------- */
/* db2_*: runtime -- context, matrix handles with residency, operator calls   */
/* ------------------------------------------------------------------------- */

/* One context per device: a compute stream, stream-ordered pooled device memory, reusable scratch, transfer and
 * launch counters.  Replaces CUDAContext (src/runtime/local/context/CUDAContext.h:29-114, .cpp:41-137), which is
 * created by CUDA::createCUDAContext (src/runtime/local/kernels/CUDA/CreateCUDAContext.cpp:4-9) for device 0 only,
 * allocates with one cudaMalloc per object and runs everything on the default stream. */
typedef struct db2_context db2_context;

/* A dense row-major matrix with up to two placements (host, device) and "latest" tracking, plus zero-copy row
 * views that keep their row offset on the device.  Replaces the residency part of DenseMatrix
 * (src/runtime/local/datastructures/DenseMatrix.cpp:126-237), MetaDataObject/DataPlacement
 * (MetaDataObject.h:39-57, DataPlacement.h:29-42) and AllocationDescriptorCUDA (AllocationDescriptorCUDA.h:24-75). */
typedef struct db2_matrix db2_matrix;

typedef struct db2_stats {
    uint64_t h2d_bytes, d2h_bytes, d2d_bytes; /* transfers issued by the residency layer            */
    uint64_t allocs, alloc_bytes, frees;      /* pooled device allocations                          */
    uint64_t launches;                        /* kernels launched through this context              */
    uint64_t live_bytes, peak_bytes;          /* device bytes held by matrices / scratch            */
    uint64_t collectives, collective_bytes;   /* cross-GPU combines issued through this context     */
} db2_stats;

int db2_context_create(int device, db2_context **ctx);
int db2_context_destroy(db2_context *ctx);
int db2_context_device(const db2_context *ctx, int *device);
/* 0 for the first context of a device group on its device, k for the k-th further context that shares the device */
int db2_context_ordinal(const db2_context *ctx, int *dup);
void *db2_context_stream(db2_context *ctx);
int db2_context_sync(db2_context *ctx);
int db2_context_stats(db2_context *ctx, db2_stats *out);
/* Upper bound on the bytes the context's matrices and scratch may hold (0 = the device's capacity); an allocation
 * that would exceed it fails with DB2_ENOMEM.  The reference's context has such a budget too (0.9 x device memory,
 * src/runtime/local/context/CUDAContext.cpp:41-75) but only consults it when deciding what to place on the GPU. */
int db2_context_set_mem_budget(db2_context *ctx, size_t bytes);

/* Row-sharded multi-GPU execution: one process (and context) per GPU.  rank 0 creates an id with
 * db2_comm_unique_id, every rank passes the same 128 bytes to db2_comm_init (exchange them with any host-side
 * mechanism).  The reference has no multi-GPU path (device 0 is hard-coded, e.g. kernels/CUDA/AggRow.cu:113) and
 * combines ADD/MIN/MAX partials on the host under a mutex (src/runtime/local/vectorized/Tasks.cpp:51-82); here they
 * are combined on the device with one NCCL all-reduce on the context's stream. */
int db2_comm_unique_id(void *id128);
int db2_comm_init(db2_context *ctx, int rank, int world, const void *id128);
int db2_comm_destroy(db2_context *ctx);
int db2_comm_info(const db2_context *ctx, int *rank, int *world);
/* in-place combine of a small contiguous partial over all ranks; combine = DB2_COMBINE_ADD / MIN / MAX */
int db2_allreduce(db2_context *ctx, db2_matrix *m, int combine);
/* the same, on a stream of its own behind what the context's stream has queued so far; the context's stream goes on
 * at once and the next use of m (or its release) waits for the combine */
int db2_allreduce_async(db2_context *ctx, db2_matrix *m, int combine);
/* collectives issued between the two calls are launched together (one NCCL group) */
int db2_comm_group_begin(db2_context *ctx);
int db2_comm_group_end(db2_context *ctx);
/* concatenation of equally tall row shards in rank order */
int db2_allgather_rows(db2_context *ctx, db2_matrix *local, db2_matrix **full);
/* concatenation of the row shards of the scheduler's partition: total_rows rows cut into one contiguous block per
 * rank, the first total_rows % world blocks one row taller.  A shard of any other height is refused (DB2_EINVAL)
 * before a collective is issued. */
int db2_allgatherv_rows(db2_context *ctx, db2_matrix *local, int64_t total_rows, db2_matrix **full);

/* device-only matrix (DataObjectFactory::create<DenseMatrix<VT>>(rows, cols, zero, &alloc_desc)) */
int db2_matrix_create(db2_context *ctx, int dtype, int64_t rows, int64_t cols, int zero, db2_matrix **out);
/* matrix whose host placement is the caller's buffer (borrowed, must outlive the handle); the device placement is
 * created on first use by a kernel, with one asynchronous copy (pinned staging is the caller's choice). */
int db2_matrix_wrap_host(db2_context *ctx, int dtype, int64_t rows, int64_t cols, int64_t ld, void *host,
                         db2_matrix **out);
/* matrix whose device placement is the caller's device buffer (borrowed) */
int db2_matrix_wrap_device(db2_context *ctx, int dtype, int64_t rows, int64_t cols, int64_t ld, void *dptr,
                           db2_matrix **out);
/* zero-copy view of rows [r0, r1) (DenseMatrix view constructor, DenseMatrix.cpp:98-115) */
int db2_matrix_slice_rows(db2_matrix *m, int64_t r0, int64_t r1, db2_matrix **view);
/* zero-copy view of columns [c0, c1) (DenseMatrix view constructor with a column range, DenseMatrix.cpp:98-115):
 * the view keeps the parent's leading dimension, which every kernel honours */
int db2_matrix_slice_cols(db2_matrix *m, int64_t c0, int64_t c1, db2_matrix **view);
int db2_matrix_incref(db2_matrix *m);
int db2_matrix_decref(db2_matrix *m); /* frees at zero (DataObjectFactory::destroy) */
int db2_matrix_info(const db2_matrix *m, int *dtype, int64_t *rows, int64_t *cols);
/* device pointer of element (0,0) and leading dimension; makes the device placement current first */
int db2_matrix_device_ptr(db2_matrix *m, void **dptr, int64_t *ld);
/* copies the latest values into dst (rows x cols, leading dimension dst_ld); synchronises the stream */
int db2_matrix_to_host(db2_matrix *m, void *dst, int64_t dst_ld);
/* The same copy on the context's second stream, ordered after the work queued so far; returns without waiting, so that
 * the results of one pipeline run travel to the host while the input of the next travels to the device.  dst (pinned
 * for a true overlap) must stay valid until db2_context_side_sync, which waits for these copies.  The reference copies
 * results synchronously from pageable memory (src/runtime/local/datastructures/AllocationDescriptorCUDA.h:60-68). */
int db2_matrix_to_host_async(db2_matrix *m, void *dst, int64_t dst_ld);
int db2_context_side_sync(db2_context *ctx);

/* Operator calls.  *res == NULL on entry means "the kernel allocates the result" (the reference's convention,
 * e.g. kernels/CUDA/AggRow.cu:121-122); otherwise the given matrix is overwritten. */
int db2_ewBinaryMat(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs);
int db2_ewBinaryObjSca(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, const void *scalar);
int db2_ewUnaryMat(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg);
int db2_aggRow(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg);
int db2_aggCol(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg);
/* res_host: host pointer to one value of the matrix's value type; synchronises */
int db2_aggAll(db2_context *ctx, int op, void *res_host, db2_matrix *arg);
/* aggAll in two halves (f64): Start queues the reduction and returns, Wait blocks until its value has arrived.  Work
 * queued on the context between the two runs while the host waits, so a loop whose condition is a reduction
 * (components.daphne:21-26: while (sum(u != c) > 0)) can queue its next trip before it looks at the count of the
 * previous one.  slot is 0 or 1: two values may be outstanding.  db2_scalarStart does the same for a 1 x 1 matrix
 * that is already on the device (e.g. a count that was combined over the ranks). */
int db2_aggAllStart(db2_context *ctx, int op, db2_matrix *arg, int slot);
int db2_scalarStart(db2_context *ctx, db2_matrix *m, int slot);
int db2_scalarWait(db2_context *ctx, int slot, double *res);
int db2_matMul(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, int transa, int transb);
int db2_syrk(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int trans_left);
/* (For a large f64 argument with trans_left the result handle is returned before anything is computed: a db2_gemv on
 * the same argument that follows is computed in the same pass over it -- t(X) X and t(X) y of the normal equations,
 * lmDS_.daph:98-112 -- and any other use of the handle computes the product alone.) */
/* res (cols x 1) = t(mat) vec (Gemv<Dense,Dense,Dense>, src/runtime/local/kernels/Gemv.h:51-63) */
int db2_gemv(db2_context *ctx, db2_matrix **res, db2_matrix *mat, db2_matrix *vec);
int db2_solve(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs);
/* vectors are reshaped without moving data, like the reference (Transpose.h:57-58) */
int db2_transpose(db2_context *ctx, db2_matrix **res, db2_matrix *arg);
int db2_fill(db2_context *ctx, db2_matrix **res, int dtype, const void *value, int64_t rows, int64_t cols);
int db2_seq(db2_context *ctx, db2_matrix **res, int dtype, const void *start, const void *end, const void *inc);
int db2_diagMatrix(db2_context *ctx, db2_matrix **res, db2_matrix *arg);
/* lhs (m x 1) (op) rhs (1 x n) -> m x n; the reference's messages for other shapes (OuterBinary.h:56-59) */
int db2_outerBinary(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs);
/* the four Cond* kernels in one call: a NULL then_m / else_m means "use the scalar"; `dtype` is the value type of the
 * result, of the matrices and of the scalars; shape mismatches carry the reference's messages */
int db2_cond(db2_context *ctx, db2_matrix **res, int dtype, db2_matrix *cond, db2_matrix *then_m, const void *then_s,
             db2_matrix *else_m, const void *else_s);
/* cumulative SUM / PROD / MIN / MAX down the rows; any other opcode is the reference's "pure binary reduction" error
 * (AggCum.h:50-52) */
int db2_aggCum(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg);
/* info (1 x cols, int64): -1 keeps a column, 0 drops it, k > 0 expands it into k indicator columns; the reference's
 * messages for a bad info and for values outside their block (DB2_EDOMAIN; OneHot.h:57-101) */
int db2_oneHot(db2_context *ctx, db2_matrix **res, db2_matrix *arg, db2_matrix *info);
/* [lhs | rhs]; DB2_EINVAL with the reference's message when the row counts differ (ColBind.h:58-63) */
int db2_colBind(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs);
/* the columns of arg named by the int64 column matrix sel; negative positions count from the end, anything outside
 * [0, cols) is DB2_EDOMAIN with the reference's out_of_range message (ExtractCol.h:84-96) */
int db2_extractCol(db2_context *ctx, db2_matrix **res, db2_matrix *arg, db2_matrix *sel);
/* res_rows / res_cols < 0: derived from the largest coordinate (synchronises) */
int db2_ctable(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, double weight,
               int64_t res_rows, int64_t res_cols);
/* Row / column ranges as zero-copy views; negative bounds count from the end; DB2_EDOMAIN with the reference's
 * out_of_range message otherwise (src/runtime/local/kernels/SliceRow.h:45-82, SliceCol.h:52-86) */
int db2_sliceRow(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int64_t lowerIncl, int64_t upperExcl);
int db2_sliceCol(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int64_t lowerIncl, int64_t upperExcl);
/* rand(rows, cols, min, max, sparsity, seed) for double / float / int64 with the reference's stream: two
 * std::mt19937 engines (seed, seed * 3), values in row-major order with zeros redrawn, selection sampling of the
 * positions for sparsity < 1; seed -1 picks a random seed.  The walk is sequential and runs on the host, in row blocks
 * that are uploaded through pinned staging while the next block is generated.  min / max: host pointers to one value
 * of `dtype`.  Replaces RandMatrix<DenseMatrix<VT>, VT> (src/runtime/local/kernels/RandMatrix.h:82-161). */
int db2_randMatrix(db2_context *ctx, db2_matrix **res, int dtype, int64_t rows, int64_t cols, const void *min,
                   const void *max, double sparsity, int64_t seed);
/* value-type cast between f64 / i64 / u64 (CastObj, used for idxMin results feeding ctable) */
int db2_castObj(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int dtype);

/* ------------------------------------------------------------------------- */
/* row-partition scheduler                                                    */
/* ------------------------------------------------------------------------- */

/* The compiled body of a vectorized pipeline: a chain of operator calls on (row slices of) the inputs that leaves its
 * results in *outputs[i] (lowered `_vect_cudaN`, src/compiler/lowering/LowerToLLVMPass.cpp:575-726). */
typedef void (*db2_pipeline_fn)(db2_matrix ***outputs, db2_matrix **inputs, db2_context *ctx);

/* Runs `fun` over the row range of the ROWS-split inputs on this context's GPU and combines the results:
 * splits[i] = DB2_SPLIT_NONE / DB2_SPLIT_ROWS (a 1-row ROWS input is broadcast), combines[o] = DB2_COMBINE_ROWS /
 * COLS / ADD / MIN / MAX; scalar inputs travel in the pointer slot with isScalar[i] != 0; batch_rows <= 0 picks the
 * batch from the memory budget (normally the whole range).  ADD/MIN/MAX results are also combined over the row
 * shards of all ranks of the communicator.  Mirrors
 * _vectorizedPipeline__DenseMatrix_double_variadic__size_t__bool__Structure_variadic__size_t__int64_t__int64_t__
 * int64_t__int64_t__size_t__void_variadic (src/runtime/local/kernels/VectorizedPipeline.h:35-69 ->
 * vectorized/MTWrapper_dense.cpp:203-336, vectorized/TasksCUDA.cpp:21-123). */
int db2_vectorizedPipeline(db2_context *ctx, db2_matrix **outputs, size_t numOutputs, const int *isScalar,
                           db2_matrix **inputs, size_t numInputs, const int64_t *outRows, const int64_t *outCols,
                           const int64_t *splits, const int64_t *combines, db2_pipeline_fn fun, int64_t batch_rows);

/* ------------------------------------------------------------------------- */
/* several GPUs in one process                                                */
/* ------------------------------------------------------------------------- */

/* A device group: one context (stream, pooled memory) per listed device and, when the devices are distinct and NCCL
 * can be loaded, one communicator per device (ncclCommInitAll).  devices == NULL: the comma-separated list in the
 * environment variable DAPHNE_B200_DEVICES, default all visible devices.  The reference creates exactly one CUDA
 * context, for device 0 (src/runtime/local/kernels/CUDA/CreateCUDAContext.cpp:4-9), although its scheduler starts one
 * GPU worker per entry of DaphneContext::cuda_contexts (src/runtime/local/vectorized/MTWrapper.h:93-98,170-174).
 * A device may be listed more than once (several contexts share it; partials are then combined without NCCL). */
typedef struct db2_group db2_group;
int db2_group_create(const int *devices, int ndev, db2_group **out);
int db2_group_destroy(db2_group *g);
int db2_group_size(const db2_group *g, int *n);
int db2_group_context(db2_group *g, int index, db2_context **ctx); /* borrowed */
int db2_group_uses_nccl(const db2_group *g, int *yes);
int db2_group_sync(db2_group *g);

/* A matrix distributed over the devices of a group: contiguous row blocks (axis 0; the first rows % n devices hold one
 * more row), column blocks (axis 1, the COLS results of a pipeline) or one full copy per device (axis -1, broadcast
 * inputs and combined ADD/MIN/MAX results).  In the reference's data model this is a MetaDataObject with one
 * DataPlacement and Range per device (src/runtime/local/datastructures/MetaDataObject.h:39-57, DataPlacement.h:29-42),
 * which its local runtime never creates. */
typedef struct db2_dist db2_dist;
/* row blocks of a host buffer (borrowed): nothing is copied here, each device fetches its rows on first use */
int db2_dist_from_host(db2_group *g, int dtype, int64_t rows, int64_t cols, int64_t ld, void *host, db2_dist **out);
/* row blocks (replicate == 0) or full copies (replicate != 0) of a matrix of any context of this process */
int db2_dist_from_matrix(db2_group *g, db2_matrix *m, int replicate, db2_dist **out);
/* from one matrix per device (shards[i] on device i; references are taken): axis 0 / 1 / -1 as above */
int db2_dist_from_shards(db2_group *g, db2_matrix **shards, int axis, db2_dist **out);
int db2_dist_info(const db2_dist *d, int *dtype, int64_t *rows, int64_t *cols, int *axis);
/* the block held by device `index` (borrowed handle) and its first row / column */
int db2_dist_shard(db2_dist *d, int index, db2_matrix **shard, int64_t *offset);
int db2_dist_incref(db2_dist *d);
int db2_dist_decref(db2_dist *d);
/* every device copies its block into its rows / columns of dst (rows x cols, leading dimension dst_ld); synchronises */
int db2_dist_to_host(db2_dist *d, void *dst, int64_t dst_ld);
/* the whole matrix on device `index` of the group (new reference); other devices' blocks arrive by peer copies */
int db2_dist_gather(db2_dist *d, int index, db2_matrix **out);

/* Combine of one partial per device (ms[i] lives on device i of the group) with DB2_COMBINE_ADD / MIN / MAX; on return
 * ms[i] is the combined matrix on device i (a handle may have been replaced by a new one, the old one released).
 * The device-side twin of the host-side merge under a mutex in src/runtime/local/vectorized/Tasks.cpp:51-82. */
/* Elementwise chains that have no specialised kernel compiled into the library get one from the run-time compiler
 * (NVRTC), once per chain and process; until it is ready such chains are evaluated by a kernel that reads the chain at
 * run time.  DAPHNE has no counterpart (it launches one kernel per operator, e.g. src/runtime/local/kernels/CUDA/
 * EwBinaryMat.cu:97-263 for every binary step).  mode: 0 = never compile, 2 = compile on the calling thread when a
 * chain is first evaluated (0.4 - 0.8 s; the default), 1 = compile on a background thread while the run-time kernel
 * serves the calls (the process must not end while a compilation runs: db2_context_destroy and db2_rtc_wait wait
 * for it).  Environment: DB2_RTC=0 / async. */
int db2_rtc_set_mode(int mode);
/* returns when no compilation is running any more */
int db2_rtc_wait(void);
/* chains with a compiled kernel / being compiled / whose compilation failed (those stay with the run-time kernel) */
int db2_rtc_counts(int *ready, int *pending, int *failed);
/* compiles (and discards) the row-pass kernel of a chain: step i applies fused operation ops[i] (the order of
 * BinaryOpCode ADD SUB MUL DIV, then SQUARE EQ NEQ LT LE GT GE MIN MAX AND OR NEG ABS SIGN FLOOR CEIL ROUND ISNAN =
 * 0..21) with an operand of kinds[i] (0 matrix, 1 row vector, 2 column vector, 3 scalar, 4 none), operands swapped if
 * reversed[i]; row aggregation j of tap_kinds[j] (0 SUM 1 PROD 2 MIN 3 MAX 4 MEAN) sees the values after tap_after[j]
 * steps; ew bit 0: the final values are stored, bit 1: the form for rows that do not start on 16-byte boundaries; ntaps < 0: the kernel of the column sums of the chain instead.  Needs no
 * device.  *binary_bytes: size of the device binary. */
int db2_rtc_compile(const int *ops, const int *kinds, const int *reversed, int nsteps, const int *tap_after,
                    const int *tap_kinds, int ntaps, int ew, size_t *binary_bytes);
/* fn(device index, that device's context, user) on all devices of the group at once, each on its device's worker thread */
typedef int (*db2_group_fn)(int index, db2_context *ctx, void *user);
int db2_group_run(db2_group *g, db2_group_fn fn, void *user);
int db2_group_allreduce(db2_group *g, db2_matrix **ms, int combine);
/* a copy of src as a new matrix of ctx; any two contexts of this process (a peer copy when their devices differ) */
int db2_matrix_to_context(db2_context *ctx, db2_matrix *src, db2_matrix **out);
/* dst[r0 : r0 + src.rows, c0 : c0 + src.cols] = src; dst and src may live on different devices.  How the row blocks
 * of several devices are put into one result (the reference copies task results into the result at
 * rowSkip * rowStart, src/runtime/local/vectorized/TasksCUDA.cpp:77-102). */
int db2_matrix_copy_block(db2_matrix *dst, int64_t r0, int64_t c0, db2_matrix *src);

/* The row-partition scheduler over all devices of a group: device i runs db2_vectorizedPipeline on block i of the
 * ROWS-split inputs (which must share one row partition; broadcast inputs must be replicated) from its own host
 * thread; ROWS / COLS results stay distributed, ADD / MIN / MAX partials are combined over the devices -- one grouped
 * ncclAllReduce per result, or peer copies and a fold in device order -- and come back replicated.  Fewer rows than
 * devices is DB2_EUNSUPPORTED.  Extends VectorizedPipeline::apply -> MTWrapper::executeQueuePerDeviceType
 * (src/runtime/local/kernels/VectorizedPipeline.h:35-69, vectorized/MTWrapper_dense.cpp:204-336: "ToDo: multi-device
 * support" at :220) to the 8 GPUs of one box. */
int db2_vectorizedPipelineGroup(db2_group *g, db2_dist **outputs, size_t numOutputs, const int *isScalar,
                                db2_dist **inputs, size_t numInputs, const int64_t *outRows, const int64_t *outCols,
                                const int64_t *splits, const int64_t *combines, db2_pipeline_fn fun,
                                int64_t batch_rows);

/* ------------------------------------------------------------------------- */
/* Matrix files                                                               */
/* ------------------------------------------------------------------------- */
/* DAPHNE's binary matrix format (doc/BinaryFormat.md), dense matrices of double / float / int64 / uint64 in one dense
 * block.  Replaces ReadDaphne<DenseMatrix<VT>> (src/runtime/local/io/ReadDaphne.h:58-100) and
 * WriteDaphne<DenseMatrix<VT>> (src/runtime/local/io/WriteDaphne.h:62-80) for the device path: the file is streamed
 * through pinned staging buffers directly into (out of) the device placement; no pageable host copy is made. */
int db2_readDaphne(db2_context *ctx, db2_matrix **res, const char *path);
int db2_writeDaphne(db2_context *ctx, db2_matrix *m, const char *path);

/* ------------------------------------------------------------------------- */
/* CSR matrices                                                               */
/* ------------------------------------------------------------------------- */

/* A CSR matrix with a device placement (32-bit column indices where the column count allows, 64-bit row offsets)
 * and zero-copy row views.  The host layout handed in and out is the reference's: values[VT], colIdxs[size_t],
 * rowOffsets[size_t, rows + 1] (src/runtime/local/datastructures/CSRMatrix.h:70-72); the reference has no device
 * residency for CSRMatrix at all. */
typedef struct db2_csr db2_csr;

int db2_csr_wrap_host(db2_context *ctx, int dtype, int64_t rows, int64_t cols, const void *values,
                      const uint64_t *col_idx, const uint64_t *row_off, db2_csr **out);
/* rows [r0, r1) sharing the arrays (CSRMatrix view constructor, CSRMatrix.h:131-148) */
int db2_csr_slice_rows(db2_csr *m, int64_t r0, int64_t r1, db2_csr **view);
int db2_csr_incref(db2_csr *m);
int db2_csr_decref(db2_csr *m);
int db2_csr_info(db2_csr *m, int64_t *rows, int64_t *cols, int64_t *nnz);
int db2_csr_to_host(db2_csr *m, void *values, uint64_t *col_idx, uint64_t *row_off);
/* res = lhs (.) rhs, rhs of the same shape or a row/column vector; entries meeting an exactly zero rhs are dropped.
 * The product is deferred until its arrays are needed.  Replaces EwBinaryMat<CSR,CSR,Dense> for MUL
 * (src/runtime/local/kernels/EwBinaryMat.h:254-317; no CUDA twin in the reference). */
int db2_ewMulCsrDense(db2_context *ctx, db2_csr **res, db2_csr *lhs, db2_matrix *rhs);
/* SUM/PROD/MIN/MAX per row with the implicit zeros taking part where the reference lets them
 * (AggRow<Dense,CSR>, src/runtime/local/kernels/AggRow.h:178-238).  A deferred product is aggregated in one pass. */
int db2_aggRowCsr(db2_context *ctx, int op, db2_matrix **res, db2_csr *arg);
/* res = lhs @ rhs, dense rhs (Gemv<Dense,CSR,Dense>, src/runtime/local/kernels/Gemv.h:79-117) */
int db2_matMulCsrDense(db2_context *ctx, db2_matrix **res, db2_csr *lhs, db2_matrix *rhs);

/* ------------------------------------------------------------------------- */
/* the workloads' kernel-call sequences, issued natively                      */
/* ------------------------------------------------------------------------- */
/* What DAPHNE's JIT-compiled `main` does for a script: one call of the operator interface above per operator, in the
 * order the compiler emits them, with next to no host time between the calls.  Row-sharded when the context has a
 * communicator (every rank passes its row block; ADD partials are combined on the device). */
/* components.daphne (test/api/cli/algorithms/components.daphne:14-26); G = rows [row_lo, row_lo + G.rows) of the
 * n x n adjacency matrix; *labels = the labels of those rows */
int db2w_connected_components(db2_context *ctx, db2_csr *G, int64_t row_lo, int64_t maxi, db2_matrix **labels,
                              int64_t *iterations);
/* kmeans.daphne (test/api/cli/algorithms/kmeans.daphne:14-21): assignment (idxMin, ties to the lowest index) and
 * update (one-hot ctable, t(P) @ X) for `iterations` rounds */
int db2w_kmeans(db2_context *ctx, db2_matrix *X, db2_matrix *C0, int iterations, db2_matrix **C, db2_matrix **assign);
/* lmDS (scripts/algorithms/lmDS_.daph:98-112): A = t(X) @ X + lambda I (syrk), b = t(X) @ y (gemv), beta = solve(A, b) */
int db2w_normal_equations(db2_context *ctx, db2_matrix *X, db2_matrix *y, double lambda, db2_matrix **A,
                          db2_matrix **b, db2_matrix **beta);
/* The column standardisation + aggregation pipeline (cfg2) on one context; with a communicator on the context every
 * rank calls it on its row shard with n_total = the global row count.  *s_out is a 1 x 1 matrix on the device (the
 * sum over all shards).  ev_rows_begin / ev_rows_end: optional events recorded around the pass over X that produces
 * the three row results (for measurements). */
int db2w_standardise(db2_context *ctx, db2_matrix *X, int64_t n_total, db2_matrix **mu_out, db2_matrix **sd_out,
                     db2_matrix **r_out, db2_matrix **max_out, db2_matrix **idx_out, db2_matrix **s_out,
                     void *ev_rows_begin, void *ev_rows_end);
/* Column standardisation and aggregation over the devices of a group, in ONE process: three pipelines through
 * db2_vectorizedPipelineGroup (column sums: ADD; squared deviations from the global mean: ADD; the row results: ROWS,
 * and their sum: ADD) with compiled bodies that issue the operator calls of
 *   mu = mean(X, 1); sd = sqrt(var(X, 1)); Z = (X - mu) / sd; r = sum(Z ^ 2, 0); s = sum(r); m = aggMax(Z, 0);
 *   i = idxMax(Z, 0);
 * X: distributed by rows.  mu, sd, s come back replicated, r, row_max, row_idx_max distributed by rows. */
int db2w_standardise_group(db2_group *g, db2_dist *X, db2_dist **mu, db2_dist **sd, db2_dist **r, db2_dist **row_max,
                           db2_dist **row_idx_max, db2_dist **s);

#ifdef __cplusplus
}
#endif
#endif /* DAPHNE_B200_H */
