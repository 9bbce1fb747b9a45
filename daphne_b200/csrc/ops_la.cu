// Runtime operator calls for the contractions and the helper kernels (matMul, syrk, gemv, solve, transpose, fill,
// seq, diagMatrix, ctable, castObj): argument checks with the reference's messages, result allocation, scratch.
#include "fused.cuh"
#include "runtime.h"

#include <cmath>

namespace db2 {

template <typename TO, typename FROM>
__global__ void cast_kernel(const FROM *__restrict__ in, int64_t rows, int64_t cols, int64_t ld, TO *__restrict__ out,
                            int64_t out_ld) {
    const int64_t n = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[(i / cols) * out_ld + (i % cols)] = static_cast<TO>(in[(i / cols) * ld + (i % cols)]);
}

static void count(db2_context *ctx, uint64_t before) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load(std::memory_order_relaxed) - before;
}

// The f32 contraction (tensor-core kernel with bounded waits) leaves a status word at the start of its scratch area;
// bit 0 set means a wait expired and the result is not valid (bit 1: operands held inf / NaN and the
// product was recomputed by the plain kernel, which is not an error).
static int check_contraction_status(db2_context *ctx, int dtype, const void *scratch) {
    if (dtype != DB2_F32)
        return DB2_OK;
    int32_t st = 0;
    DB2_CUDA(cudaMemcpyAsync(&st, scratch, sizeof(st), cudaMemcpyDeviceToHost, ctx->stream));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    DB2_CHECK((st & 1) == 0, DB2_ETIMEOUT, "f32 contraction kernel gave up waiting (status %d); result discarded",
              (int)st);
    return DB2_OK;
}

// a deferred t(X) X that something other than the matching gemv needs: the product alone
int syrk_force(db2_matrix *m) {
    db2_context *ctx = m->ctx;
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    const Operand x = *m->syrk_of;
    m->dev = make_devbuf(ctx, (size_t)m->rows * m->cols * 8);
    m->dev_off = 0;
    m->dev_ld = m->cols;
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, db2k_syrk_scratch_bytes(DB2_F64, x.rows, x.cols, 1), &scratch));
    DB2_TRY(db2k_syrk(DB2_F64, x.ptr(8), x.rows, x.cols, x.ld, 1, m->dev_ptr(), m->dev_ld, scratch,
                      ctx->scratch_bytes, ctx->stream));
    m->dev_valid = true;
    m->syrk_of.reset();
    if (ctx->syrk_waiting == m)
        ctx->syrk_waiting = nullptr;
    count(ctx, before);
    return DB2_OK;
}

} // namespace db2

using namespace db2;

extern "C" {

int db2_matMul(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, int transa, int transb) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && lhs && rhs, DB2_EINVAL, "null argument");
    const int dt = lhs->dtype;
    DB2_CHECK((dt == DB2_F64 || dt == DB2_F32 || dt == DB2_I64 || dt == DB2_I32 || dt == DB2_U64 || dt == DB2_U32) &&
                  rhs->dtype == dt,
              DB2_EUNSUPPORTED, "matMul: operands of one value type (double, float or an integer type) on the device");
    const int64_t m = transa ? lhs->cols : lhs->rows, k = transa ? lhs->rows : lhs->cols;
    const int64_t k2 = transb ? rhs->cols : rhs->rows, n = transb ? rhs->rows : rhs->cols;
    DB2_CHECK(k == k2, DB2_EINVAL, "MatMul - #cols of lhs and #rows of rhs must be the same, but got%lldand%lld",
              (long long)k, (long long)k2);
    bind_device(ctx);
    {
        bool handled = false;
        DB2_TRY(onehot_try_matmul(ctx, res, lhs, rhs, transa, transb, &handled));
        if (handled)
            return DB2_OK;
        DB2_TRY(lazy_try_matmul(ctx, res, lhs, rhs, transa, transb, &handled));
        if (handled)
            return DB2_OK;
    }
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(lhs));
    DB2_TRY(ensure_device(rhs));
    DB2_TRY(prepare_result(ctx, res, dt, m, n));
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, db2k_matmul_scratch_bytes(dt, m, n, k), &scratch));
    DB2_TRY(db2k_matmul(dt, lhs->dev_ptr(), lhs->rows, lhs->cols, lhs->dev_ld, rhs->dev_ptr(), rhs->rows,
                        rhs->cols, rhs->dev_ld, transa, transb, (*res)->dev_ptr(), (*res)->dev_ld, scratch,
                        ctx->scratch_bytes, ctx->stream));
    count(ctx, before);
    return check_contraction_status(ctx, dt, scratch);
    DB2_API_END
}

int db2_syrk(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int trans_left) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    const int dt = arg->dtype;
    DB2_CHECK(dt == DB2_F64 || dt == DB2_F32, DB2_EUNSUPPORTED, "syrk: double or float on the device");
    const int64_t n = trans_left ? arg->cols : arg->rows;
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(arg));
    // t(X) X of a large X whose result nobody has looked at yet: the normal equations ask for t(X) y next
    // (lmDS_.daph:98-112; one pipeline with two ADD results under --vec), and both come out of one pass over X
    if (dt == DB2_F64 && trans_left && *res == nullptr && !ctx->eager && arg->rows * arg->cols >= ((int64_t)1 << 22) &&
        db2k_syrk_gemv_supported(arg->rows, arg->cols)) {
        auto x = std::make_shared<Operand>();
        x->buf = arg->dev;
        x->off = arg->dev_off;
        x->ld = arg->dev_ld;
        x->rows = arg->rows;
        x->cols = arg->cols;
        db2_matrix *r = new db2_matrix(); // no placement yet
        r->ctx = ctx;
        r->dtype = DB2_F64;
        r->rows = r->cols = n;
        r->syrk_of = x;
        if (ctx->syrk_waiting && ctx->syrk_waiting->syrk_of) // one at a time: the older one is computed now
            DB2_TRY(syrk_force(ctx->syrk_waiting));
        ctx->syrk_waiting = r;
        *res = r;
        return DB2_OK;
    }
    DB2_TRY(prepare_result(ctx, res, dt, n, n));
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, db2k_syrk_scratch_bytes(dt, arg->rows, arg->cols, trans_left), &scratch));
    DB2_TRY(db2k_syrk(dt, arg->dev_ptr(), arg->rows, arg->cols, arg->dev_ld, trans_left, (*res)->dev_ptr(),
                      (*res)->dev_ld, scratch, ctx->scratch_bytes, ctx->stream));
    count(ctx, before);
    return check_contraction_status(ctx, dt, scratch);
    DB2_API_END
}

int db2_gemv(db2_context *ctx, db2_matrix **res, db2_matrix *mat, db2_matrix *vec) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && mat && vec, DB2_EINVAL, "null argument");
    if (ctx->syrk_waiting && mat->dtype == DB2_F64 && vec->dtype == DB2_F64 && mat->dev_valid) {
        // t(X) X of this very X is waiting: one pass over X gives both
        db2_matrix *w = ctx->syrk_waiting;
        const Operand &x = *w->syrk_of;
        if (x.buf == mat->dev && x.off == mat->dev_off && x.ld == mat->dev_ld && x.rows == mat->rows &&
            x.cols == mat->cols && vec->rows == mat->rows && vec->cols == 1) {
            bind_device(ctx);
            const uint64_t before = g_launches.load();
            DB2_TRY(ensure_device(vec));
            if (vec->dev_ld == 1 && aligned16(vec->dev_ptr())) {
                DB2_TRY(prepare_result(ctx, res, DB2_F64, mat->cols, 1));
                if ((*res)->dev_ld == 1) {
                    w->dev = make_devbuf(ctx, (size_t)w->rows * w->cols * 8);
                    w->dev_off = 0;
                    w->dev_ld = w->cols;
                    void *scratch = nullptr;
                    DB2_TRY(ctx_scratch(ctx, db2k_syrk_gemv_scratch_bytes(mat->rows, mat->cols), &scratch));
                    DB2_TRY(db2k_syrk_gemv(mat->dev_ptr(), mat->rows, mat->cols, mat->dev_ld, vec->dev_ptr(),
                                           w->dev_ptr(), w->dev_ld, (*res)->dev_ptr(), scratch, ctx->scratch_bytes,
                                           ctx->stream));
                    w->dev_valid = true;
                    w->syrk_of.reset();
                    ctx->syrk_waiting = nullptr;
                    count(ctx, before);
                    return DB2_OK;
                }
            }
        }
    }
    if (mat->dtype == DB2_F32 && vec->dtype == DB2_F32) {
        // f32: t(mat) @ vec as a tensor-core product with one result column (Gemv.h:51-63 calls cblas_sgemv)
        DB2_CHECK(vec->rows == mat->rows && vec->cols == 1, DB2_EINVAL,
                  "Gemv - vec must be a column vector with as many rows as mat (%lld), got (%lld x %lld)",
                  (long long)mat->rows, (long long)vec->rows, (long long)vec->cols);
        return db2_matMul(ctx, res, mat, vec, 1, 0);
    }
    DB2_CHECK(mat->dtype == DB2_F64 && vec->dtype == DB2_F64, DB2_EUNSUPPORTED,
              "gemv: double or float operands of one type on the device");
    DB2_CHECK(vec->rows == mat->rows && vec->cols == 1, DB2_EINVAL,
              "Gemv - vec must be a column vector with as many rows as mat (%lld), got (%lld x %lld)",
              (long long)mat->rows, (long long)vec->rows, (long long)vec->cols);
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(mat));
    DB2_TRY(ensure_device(vec));
    DB2_TRY(prepare_result(ctx, res, DB2_F64, mat->cols, 1));
    db2_matrix *r = *res;
    if (mat->cols == 0)
        return DB2_OK;
    // t(mat) vec = column sums of (mat .* vec): one fused column pass over mat (HBM-bound, mat is read once)
    FusedProgram P;
    memset(&P, 0, sizeof(P));
    P.base = mat->dev_ptr();
    P.base_ld = mat->dev_ld;
    P.rows = mat->rows;
    P.cols = mat->cols;
    P.nsteps = 1;
    P.steps[0].kind = FK_COLVEC;
    P.steps[0].op = FO_MUL;
    P.steps[0].smem_off = -1;
    P.steps[0].ptr = vec->dev_ptr();
    P.steps[0].ld = vec->dev_ld;
    if (mat->rows == 0) {
        DB2_CUDA(cudaMemsetAsync(r->dev_ptr(), 0, (size_t)mat->cols * 8, ctx->stream));
        return DB2_OK;
    }
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, fused_col_scratch_bytes(mat->cols), &scratch));
    if (r->dev_ld == 1) {
        int rc = DB2_OK;
        if (!fused_col_pass_ct(P, "MUL.C#", DB2_AGG_SUM, r->dev_ptr(), scratch, ctx->scratch_bytes, ctx->stream, &rc))
            rc = fused_col_pass_f64(P, DB2_AGG_SUM, r->dev_ptr(), scratch, ctx->scratch_bytes, ctx->stream);
        DB2_TRY(rc);
    } else {
        return set_error(DB2_EUNSUPPORTED, "gemv into a strided result view");
    }
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_solve(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && lhs && rhs, DB2_EINVAL, "null argument");
    if (lhs->dtype == DB2_F32 && rhs->dtype == DB2_F32) {
        // float systems (LAPACKE_sgesv in the reference, Solve.h:66-84) are solved in double and the solution is
        // rounded once: every float is a double, so this is the same system, solved at least as accurately
        db2_matrix *l64 = nullptr, *r64 = nullptr, *x64 = nullptr;
        int rc = db2_castObj(ctx, &l64, lhs, DB2_F64);
        if (rc == DB2_OK)
            rc = db2_castObj(ctx, &r64, rhs, DB2_F64);
        if (rc == DB2_OK)
            rc = db2_solve(ctx, &x64, l64, r64);
        if (rc == DB2_OK)
            rc = db2_castObj(ctx, res, x64, DB2_F32);
        for (db2_matrix *m : {l64, r64, x64})
            if (m)
                db2_matrix_decref(m);
        return rc;
    }
    DB2_CHECK(lhs->dtype == DB2_F64 && rhs->dtype == DB2_F64, DB2_EUNSUPPORTED,
              "solve: double or float operands of one type on the device");
    // checks and messages of Solve.h:90-99
    DB2_CHECK(lhs->rows == rhs->rows, DB2_EINVAL, "#rows of lhs and #rows of rhs must be the same");
    DB2_CHECK(lhs->rows == lhs->cols, DB2_EINVAL, "#rows and #cols of lhs must be the same");
    DB2_CHECK(rhs->cols == 1, DB2_EINVAL, "#cols of rhs must be 1");
    const int64_t n = lhs->rows;
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(lhs));
    DB2_TRY(ensure_device(rhs));
    DB2_TRY(prepare_result(ctx, res, DB2_F64, n, 1));
    db2_matrix *r = *res;
    DB2_CHECK(r->dev_ld == 1, DB2_EUNSUPPORTED, "solve into a strided result view");
    if (n == 0)
        return DB2_OK;
    auto work = make_devbuf(ctx, (size_t)n * n * 8);
    DB2_CUDA(cudaMemcpy2DAsync(work->ptr, (size_t)n * 8, lhs->dev_ptr(), (size_t)lhs->dev_ld * 8, (size_t)n * 8,
                               (size_t)n, cudaMemcpyDeviceToDevice, ctx->stream));
    DB2_CUDA(cudaMemcpy2DAsync(r->dev_ptr(), 8, rhs->dev_ptr(), (size_t)rhs->dev_ld * 8, 8, (size_t)n,
                               cudaMemcpyDeviceToDevice, ctx->stream));
    auto pivots = make_devbuf(ctx, db2k_solve_scratch_bytes(n));
    DB2_TRY(db2k_solve(DB2_F64, work->ptr, n, r->dev_ptr(), ctx->dev_status + 8, pivots->ptr, pivots->bytes,
                       ctx->stream));
    count(ctx, before);
    // the reference throws from inside the call when a pivot is exactly zero: check synchronously
    DB2_CUDA(cudaMemcpyAsync(ctx->host_status + 8, ctx->dev_status + 8, sizeof(int32_t), cudaMemcpyDeviceToHost,
                             ctx->stream));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    if (ctx->host_status[8] != 0)
        return set_error(DB2_EINVAL, "A factor Ui is exactly singular, so the solution could not be computed");
    return DB2_OK;
    DB2_API_END
}

int db2_transpose(db2_context *ctx, db2_matrix **res, db2_matrix *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(arg));
    if (*res == nullptr && (arg->rows == 1 || (arg->cols == 1 && arg->dev_ld == 1))) {
        // a contiguous vector is reshaped, sharing the buffer (Transpose.h:57-58)
        db2_matrix *r = new db2_matrix();
        r->ctx = ctx;
        r->dtype = arg->dtype;
        r->rows = arg->cols;
        r->cols = arg->rows;
        r->dev = arg->dev;
        r->dev_off = arg->dev_off;
        r->dev_ld = r->cols;
        r->dev_valid = true;
        r->is_view = true;
        *res = r;
        return DB2_OK;
    }
    DB2_TRY(prepare_result(ctx, res, arg->dtype, arg->cols, arg->rows));
    DB2_TRY(db2k_transpose(arg->dtype, arg->dev_ptr(), arg->rows, arg->cols, arg->dev_ld, (*res)->dev_ptr(),
                           (*res)->dev_ld, ctx->stream));
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_fill(db2_context *ctx, db2_matrix **res, int dtype, const void *value, int64_t rows, int64_t cols) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && value, DB2_EINVAL, "null argument");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(prepare_result(ctx, res, dtype, rows, cols));
    DB2_TRY(db2k_fill(dtype, (*res)->dev_ptr(), rows, cols, (*res)->dev_ld, value, ctx->stream));
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_seq(db2_context *ctx, db2_matrix **res, int dtype, const void *start_p, const void *end_p, const void *inc_p) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && start_p && end_p && inc_p, DB2_EINVAL, "null argument");
    DB2_CHECK(dtype == DB2_F64 || dtype == DB2_I64, DB2_EUNSUPPORTED, "seq: double and int64 only");
    double start, end, inc;
    if (dtype == DB2_F64) {
        start = *static_cast<const double *>(start_p);
        end = *static_cast<const double *>(end_p);
        inc = *static_cast<const double *>(inc_p);
    } else {
        start = (double)*static_cast<const int64_t *>(start_p);
        end = (double)*static_cast<const int64_t *>(end_p);
        inc = (double)*static_cast<const int64_t *>(inc_p);
    }
    // argument checks and row count of Seq.h:51-72,89-98
    DB2_CHECK(!std::isnan(inc), DB2_EINVAL, "inc cannot be NaN");
    DB2_CHECK(!std::isnan(start), DB2_EINVAL, "start cannot be NaN");
    DB2_CHECK(!std::isnan(end), DB2_EINVAL, "end cannot be NaN");
    DB2_CHECK(inc != 0, DB2_EINVAL, "inc should not be zero");
    int64_t n = 0;
    if (!((start < end && inc < 0) || (start > end && inc > 0))) {
        n = (int64_t)std::ceil(std::fabs(end - start) / std::fabs(inc)) + 1;
        const double last = start + (double)(n - 1) * inc;
        const double eps = 1.0e-13;
        if ((end < start && end - last > eps) || (end > start && last - end > eps))
            n--;
    }
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(prepare_result(ctx, res, dtype, n, 1));
    DB2_TRY(db2k_seq(dtype, (*res)->dev_ptr(), n, start_p, inc_p, ctx->stream));
    if (dtype == DB2_I64 && !(*res)->is_view) {
        (*res)->is_seq = true;
        (*res)->seq_start = *static_cast<const int64_t *>(start_p);
        (*res)->seq_inc = *static_cast<const int64_t *>(inc_p);
    }
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_diagMatrix(db2_context *ctx, db2_matrix **res, db2_matrix *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    DB2_CHECK(arg->cols == 1, DB2_EINVAL, "DiagMatrix.h - parameter arg must be a column-matrix");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(arg));
    DB2_TRY(prepare_result(ctx, res, arg->dtype, arg->rows, arg->rows));
    DB2_TRY(db2k_diag_matrix(arg->dtype, arg->dev_ptr(), arg->dev_ld, arg->rows, (*res)->dev_ptr(), (*res)->dev_ld,
                             ctx->stream));
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_ctable(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, double weight, int64_t res_rows,
               int64_t res_cols) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && lhs && rhs, DB2_EINVAL, "null argument");
    DB2_CHECK(lhs->dtype == DB2_I64 && rhs->dtype == DB2_I64, DB2_EUNSUPPORTED, "ctable: int64 coordinates only");
    DB2_CHECK(lhs->cols == 1 && rhs->cols == 1, DB2_EINVAL, "ctable: lhs and rhs must have only one column");
    DB2_CHECK(lhs->rows == rhs->rows, DB2_EINVAL, "ctable: lhs and rhs must have the same number of rows");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(lhs));
    DB2_TRY(ensure_device(rhs));
    const int64_t n = lhs->rows;
    // lhs = seq(0, n - 1): exactly one entry per row, in row order.  The result is kept as (rhs, weight) and written
    // out only if something other than t(P) @ X or sum(P, 1) asks for its values.
    if (*res == nullptr && !ctx->eager && lhs->is_seq && lhs->seq_start == 0 && lhs->seq_inc == 1 && n > 0 &&
        (res_rows == n || res_rows < 0) && res_cols > 0) {
        db2_matrix *r = new db2_matrix();
        r->ctx = ctx;
        r->dtype = DB2_F64;
        r->rows = n;
        r->cols = res_cols;
        auto oh = std::make_shared<OneHot>();
        oh->idx.buf = rhs->dev;
        oh->idx.off = rhs->dev_off;
        oh->idx.ld = rhs->dev_ld;
        oh->idx.rows = n;
        oh->idx.cols = 1;
        oh->weight = weight;
        r->onehot = oh;
        *res = r;
        return DB2_OK;
    }
    if (res_rows < 0 || res_cols < 0) {
        DB2_CHECK(n > 0, DB2_EINVAL, "ctable: cannot derive the result shape from empty coordinate vectors");
        long long *dmax = reinterpret_cast<long long *>(ctx->dev_status + 16);
        long long *hmax = reinterpret_cast<long long *>(ctx->host_status + 16);
        if (res_rows < 0) {
            DB2_TRY(db2k_max_i64(lhs->dev_ptr(), lhs->dev_ld, n, dmax, ctx->stream));
            DB2_CUDA(cudaMemcpyAsync(hmax, dmax, 8, cudaMemcpyDeviceToHost, ctx->stream));
            DB2_CUDA(cudaStreamSynchronize(ctx->stream));
            res_rows = *hmax + 1;
        }
        if (res_cols < 0) {
            DB2_TRY(db2k_max_i64(rhs->dev_ptr(), rhs->dev_ld, n, dmax, ctx->stream));
            DB2_CUDA(cudaMemcpyAsync(hmax, dmax, 8, cudaMemcpyDeviceToHost, ctx->stream));
            DB2_CUDA(cudaStreamSynchronize(ctx->stream));
            res_cols = *hmax + 1;
        }
    }
    DB2_TRY(prepare_result(ctx, res, DB2_F64, res_rows, res_cols));
    DB2_TRY(db2k_ctable(lhs->dev_ptr(), lhs->dev_ld, rhs->dev_ptr(), rhs->dev_ld, n, weight, (*res)->dev_ptr(),
                        res_rows, res_cols, (*res)->dev_ld, 0, ctx->stream));
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_castObj(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int dtype) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(arg));
    // The two 64-bit integer types hold the same bits (the conversion wraps): the result is a second handle on the
    // same device buffer.  A later write through either handle gets a buffer of its own (prepare_result), so the two
    // matrices stay independent values.  K-means casts a million row positions per iteration this way.
    if (*res == nullptr && arg->dev && arg->dev_valid && !arg->is_view &&
        ((arg->dtype == DB2_U64 && dtype == DB2_I64) || (arg->dtype == DB2_I64 && dtype == DB2_U64))) {
        db2_matrix *r = new db2_matrix();
        r->ctx = ctx;
        r->dtype = dtype;
        r->rows = arg->rows;
        r->cols = arg->cols;
        r->dev = arg->dev;
        r->dev_off = arg->dev_off;
        r->dev_ld = arg->dev_ld;
        r->dev_valid = true;
        *res = r;
        return DB2_OK;
    }
    DB2_TRY(prepare_result(ctx, res, dtype, arg->rows, arg->cols));
    db2_matrix *r = *res;
    const int64_t n = arg->rows * arg->cols;
    if (n == 0)
        return DB2_OK;
    int64_t want = (n + 255) / 256;
    const int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(want < cap ? want : cap);
#define DB2_CAST(FROM_CODE, FROM_T, TO_CODE, TO_T)                                                                     \
    if (arg->dtype == FROM_CODE && dtype == TO_CODE) {                                                                 \
        cast_kernel<TO_T, FROM_T><<<grid, 256, 0, ctx->stream>>>(static_cast<const FROM_T *>(arg->dev_ptr()),          \
                                                                 arg->rows, arg->cols, arg->dev_ld,                    \
                                                                 static_cast<TO_T *>(r->dev_ptr()), r->dev_ld);        \
        DB2_TRY(after_launch("cast_kernel"));                                                                          \
        count(ctx, before);                                                                                            \
        return DB2_OK;                                                                                                 \
    }
    DB2_CAST(DB2_U64, uint64_t, DB2_I64, int64_t)
    DB2_CAST(DB2_U64, uint64_t, DB2_F64, double)
    DB2_CAST(DB2_I64, int64_t, DB2_F64, double)
    DB2_CAST(DB2_I64, int64_t, DB2_U64, uint64_t)
    DB2_CAST(DB2_F64, double, DB2_I64, int64_t)
    DB2_CAST(DB2_F64, double, DB2_U64, uint64_t)
    DB2_CAST(DB2_F64, double, DB2_F32, float)
    DB2_CAST(DB2_F32, float, DB2_F64, double)
    DB2_CAST(DB2_F64, double, DB2_F64, double)
    DB2_CAST(DB2_I64, int64_t, DB2_I64, int64_t)
    DB2_CAST(DB2_U64, uint64_t, DB2_U64, uint64_t)
#undef DB2_CAST
    return set_error(DB2_EUNSUPPORTED, "castObj from value type %d to %d", arg->dtype, dtype);
    DB2_API_END
}

} // extern "C"
