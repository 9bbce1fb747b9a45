// Reorganisation kernels: ColBind, ExtractCol, the conditional select (Cond*) and OneHot.
//
// Both are pure copies (16 bytes of traffic per 8-byte element), so the only thing that matters is that every warp
// moves whole rows with its lanes side by side (coalesced on both ends) and has several rows in flight:
//   ColBind     res = [lhs | rhs]                 (src/runtime/local/kernels/ColBind.h:54-88; CUDA twin CUDA/ColBind.cu:24-44,
//                                                  one element per thread with a 32-bit index)
//   ExtractCol  res[:, c] = arg[:, sel[c]]        (src/runtime/local/kernels/ExtractCol.h:64-105; CUDA twin
//                                                  CUDA/ExtractCol.cu:22-30)
// A warp owns rows r, r + W, ... (W = warps in the grid) and walks four of them at a time; lane l copies the columns
// l, l + 32, ...  The column selection of ExtractCol is validated on the host (negative positions count from the end,
// anything outside [0, cols) is the reference's out_of_range error) and handed to the kernel as resolved positions.
#include "runtime.h"

#include <string>
#include <vector>

namespace db2 {

constexpr int RG_THREADS = 256, RG_ROWS = 4;

template <typename VT>
__global__ void __launch_bounds__(RG_THREADS)
    col_bind_kernel(const VT *__restrict__ lhs, int64_t ld_l, int64_t cols_l, const VT *__restrict__ rhs, int64_t ld_r,
                    int64_t cols_r, int64_t rows, VT *__restrict__ res, int64_t ld_o) {
    const int lane = threadIdx.x % 32;
    const int64_t warp = ((int64_t)blockIdx.x * RG_THREADS + threadIdx.x) / 32;
    const int64_t nwarps = (int64_t)gridDim.x * (RG_THREADS / 32);
    const int64_t cols = cols_l + cols_r;
    for (int64_t r0 = warp * RG_ROWS; r0 < rows; r0 += nwarps * RG_ROWS) {
        for (int64_t c = lane; c < cols; c += 32) {
            VT v[RG_ROWS];
#pragma unroll
            for (int u = 0; u < RG_ROWS; u++)
                if (r0 + u < rows)
                    v[u] = c < cols_l ? lhs[(r0 + u) * ld_l + c] : rhs[(r0 + u) * ld_r + (c - cols_l)];
#pragma unroll
            for (int u = 0; u < RG_ROWS; u++)
                if (r0 + u < rows)
                    res[(r0 + u) * ld_o + c] = v[u];
        }
    }
}

template <typename VT>
__global__ void __launch_bounds__(RG_THREADS)
    extract_col_kernel(const VT *__restrict__ arg, int64_t ld, int64_t rows, const int64_t *__restrict__ pos,
                       int64_t nsel, VT *__restrict__ res, int64_t ld_o) {
    const int lane = threadIdx.x % 32;
    const int64_t warp = ((int64_t)blockIdx.x * RG_THREADS + threadIdx.x) / 32;
    const int64_t nwarps = (int64_t)gridDim.x * (RG_THREADS / 32);
    for (int64_t r0 = warp * RG_ROWS; r0 < rows; r0 += nwarps * RG_ROWS) {
        for (int64_t c = lane; c < nsel; c += 32) {
            const int64_t p = pos[c];
            VT v[RG_ROWS];
#pragma unroll
            for (int u = 0; u < RG_ROWS; u++)
                if (r0 + u < rows)
                    v[u] = arg[(r0 + u) * ld + p];
#pragma unroll
            for (int u = 0; u < RG_ROWS; u++)
                if (r0 + u < rows)
                    res[(r0 + u) * ld_o + c] = v[u];
        }
    }
}

// res = cond ? then : else, element by element; `then` / `else` are matrices of the shape of cond or immediates
// (CondMatMatMat.h, CondMatMatSca.h, CondMatScaMat.h, CondMatScaSca.h: static_cast<bool>(cond) picks, so a NaN
// condition is true).  Same warp-per-row walk as the copies above.
template <typename VT, typename CT>
__global__ void __launch_bounds__(RG_THREADS)
    cond_kernel(const CT *__restrict__ cond, int64_t ld_c, const VT *__restrict__ then_m, int64_t ld_t, VT then_s,
                const VT *__restrict__ else_m, int64_t ld_e, VT else_s, int64_t rows, int64_t cols,
                VT *__restrict__ res, int64_t ld_o) {
    const int lane = threadIdx.x % 32;
    const int64_t warp = ((int64_t)blockIdx.x * RG_THREADS + threadIdx.x) / 32;
    const int64_t nwarps = (int64_t)gridDim.x * (RG_THREADS / 32);
    for (int64_t r0 = warp * RG_ROWS; r0 < rows; r0 += nwarps * RG_ROWS) {
        for (int64_t c = lane; c < cols; c += 32) {
            CT k[RG_ROWS];
            VT t[RG_ROWS], e[RG_ROWS];
#pragma unroll
            for (int u = 0; u < RG_ROWS; u++)
                if (r0 + u < rows) {
                    k[u] = cond[(r0 + u) * ld_c + c];
                    t[u] = then_m ? then_m[(r0 + u) * ld_t + c] : then_s;
                    e[u] = else_m ? else_m[(r0 + u) * ld_e + c] : else_s;
                }
#pragma unroll
            for (int u = 0; u < RG_ROWS; u++)
                if (r0 + u < rows)
                    res[(r0 + u) * ld_o + c] = (k[u] != (CT)0) ? t[u] : e[u];
        }
    }
}

// One-hot encoding (src/runtime/local/kernels/OneHot.h:54-110): result column j either copies argument column
// src[j] (hot[j] < 0) or is 1 where the argument value, cut to an integer, equals hot[j] and 0 elsewhere.  `width[j]`
// is the size of the block column j belongs to (only read where hot[j] == 0: that lane checks the value's range and
// raises *status, the reference's out_of_range).
template <typename VT>
__global__ void __launch_bounds__(RG_THREADS)
    one_hot_kernel(const VT *__restrict__ arg, int64_t ld, int64_t rows, const int64_t *__restrict__ src,
                   const int64_t *__restrict__ hot, const int64_t *__restrict__ width, int64_t cols_res,
                   VT *__restrict__ res, int64_t ld_o, int32_t *__restrict__ status) {
    const int lane = threadIdx.x % 32;
    const int64_t warp = ((int64_t)blockIdx.x * RG_THREADS + threadIdx.x) / 32;
    const int64_t nwarps = (int64_t)gridDim.x * (RG_THREADS / 32);
    bool bad = false;
    for (int64_t r0 = warp * RG_ROWS; r0 < rows; r0 += nwarps * RG_ROWS) {
        for (int64_t c = lane; c < cols_res; c += 32) {
            const int64_t s = src[c], h = hot[c];
            const int64_t w = h == 0 ? width[c] : 0;
#pragma unroll
            for (int u = 0; u < RG_ROWS; u++)
                if (r0 + u < rows) {
                    const VT v = arg[(r0 + u) * ld + s];
                    VT out = v;
                    if (h >= 0) {
                        // the reference converts to size_t: negative values and NaN cannot name a position
                        const bool in_range = v >= (VT)0 && v < (VT)9.2e18;
                        const int64_t k = in_range ? (int64_t)v : -1;
                        out = (k == h) ? (VT)1 : (VT)0;
                        if (h == 0 && (k < 0 || k >= w))
                            bad = true;
                    }
                    res[(r0 + u) * ld_o + c] = out;
                }
        }
    }
    if (bad)
        atomicExch(status, 1);
}

static void count(db2_context *ctx, uint64_t before) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load(std::memory_order_relaxed) - before;
}

static int reorg_grid(int64_t rows) {
    const int64_t want = (rows + (RG_THREADS / 32) * RG_ROWS - 1) / ((RG_THREADS / 32) * RG_ROWS);
    const int64_t cap = (int64_t)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

} // namespace db2

using namespace db2;

extern "C" {

int db2k_col_bind(int dtype, const void *lhs, int64_t lhs_ld, int64_t lhs_cols, const void *rhs, int64_t rhs_ld,
                  int64_t rhs_cols, int64_t rows, void *res, int64_t res_ld, void *stream) {
    DB2_CHECK(rows >= 0 && lhs_cols >= 0 && rhs_cols >= 0, DB2_EINVAL, "negative shape");
    if (rows == 0 || lhs_cols + rhs_cols == 0)
        return DB2_OK;
    const int grid = reorg_grid(rows);
    DB2_DISPATCH_DTYPE(dtype, VT,
                       (col_bind_kernel<VT><<<grid, RG_THREADS, 0, as_stream(stream)>>>(
                           static_cast<const VT *>(lhs), lhs_ld, lhs_cols, static_cast<const VT *>(rhs), rhs_ld,
                           rhs_cols, rows, static_cast<VT *>(res), res_ld)));
    return after_launch("col_bind_kernel");
}

int db2k_extract_col(int dtype, const void *arg, int64_t ld, int64_t rows, const void *dev_positions, int64_t nsel,
                     void *res, int64_t res_ld, void *stream) {
    DB2_CHECK(rows >= 0 && nsel >= 0, DB2_EINVAL, "negative shape");
    if (rows == 0 || nsel == 0)
        return DB2_OK;
    const int grid = reorg_grid(rows);
    DB2_DISPATCH_DTYPE(dtype, VT,
                       (extract_col_kernel<VT><<<grid, RG_THREADS, 0, as_stream(stream)>>>(
                           static_cast<const VT *>(arg), ld, rows, static_cast<const int64_t *>(dev_positions), nsel,
                           static_cast<VT *>(res), res_ld)));
    return after_launch("extract_col_kernel");
}

int db2k_cond(int dtype, int cond_dtype, const void *cond, int64_t cond_ld, const void *then_m, int64_t then_ld,
              const void *then_s, const void *else_m, int64_t else_ld, const void *else_s, int64_t rows, int64_t cols,
              void *res, int64_t res_ld, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative shape");
    DB2_CHECK((then_m || then_s) && (else_m || else_s), DB2_EINVAL, "then / else need a matrix or a scalar");
    if (rows == 0 || cols == 0)
        return DB2_OK;
    const int grid = reorg_grid(rows);
    DB2_DISPATCH_DTYPE(
        dtype, VT,
        DB2_DISPATCH_DTYPE(cond_dtype, CT,
                           (cond_kernel<VT, CT><<<grid, RG_THREADS, 0, as_stream(stream)>>>(
                               static_cast<const CT *>(cond), cond_ld, static_cast<const VT *>(then_m), then_ld,
                               then_m ? (VT)0 : *static_cast<const VT *>(then_s), static_cast<const VT *>(else_m),
                               else_ld, else_m ? (VT)0 : *static_cast<const VT *>(else_s), rows, cols,
                               static_cast<VT *>(res), res_ld))));
    return after_launch("cond_kernel");
}

int db2_cond(db2_context *ctx, db2_matrix **res, int dtype, db2_matrix *cond, db2_matrix *then_m, const void *then_s,
             db2_matrix *else_m, const void *else_s) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && cond, DB2_EINVAL, "null argument");
    DB2_CHECK((then_m || then_s) && (else_m || else_s), DB2_EINVAL, "cond: then / else need a matrix or a scalar");
    const char *name = then_m ? (else_m ? "CondMatMatMat" : "CondMatMatSca") : (else_m ? "CondMatScaMat" : "CondMatScaSca");
    const char *what = then_m ? (else_m ? "condition/then/else" : "condition/then") : "condition/else";
    DB2_CHECK((!then_m || (then_m->rows == cond->rows && then_m->cols == cond->cols)) &&
                  (!else_m || (else_m->rows == cond->rows && else_m->cols == cond->cols)),
              DB2_EINVAL, "%s: %s matrices must have the same shape", name, what);
    DB2_CHECK((!then_m || then_m->dtype == dtype) && (!else_m || else_m->dtype == dtype), DB2_EUNSUPPORTED,
              "cond: then / else are not of the result's value type");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(cond));
    if (then_m)
        DB2_TRY(ensure_device(then_m));
    if (else_m)
        DB2_TRY(ensure_device(else_m));
    DB2_TRY(prepare_result(ctx, res, dtype, cond->rows, cond->cols));
    DB2_TRY(db2k_cond(dtype, cond->dtype, cond->dev_ptr(), cond->dev_ld, then_m ? then_m->dev_ptr() : nullptr,
                      then_m ? then_m->dev_ld : 0, then_s, else_m ? else_m->dev_ptr() : nullptr,
                      else_m ? else_m->dev_ld : 0, else_s, cond->rows, cond->cols, (*res)->dev_ptr(), (*res)->dev_ld,
                      ctx->stream));
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2k_one_hot(int dtype, const void *arg, int64_t ld, int64_t rows, const void *dev_src, const void *dev_hot,
                 const void *dev_width, int64_t cols_res, void *res, int64_t res_ld, void *dev_status, void *stream) {
    DB2_CHECK(rows >= 0 && cols_res >= 0, DB2_EINVAL, "negative shape");
    DB2_CHECK(dtype == DB2_F64 || dtype == DB2_I64, DB2_EUNSUPPORTED, "OneHot: double and int64 values only");
    if (rows == 0 || cols_res == 0)
        return DB2_OK;
    const int grid = reorg_grid(rows);
    if (dtype == DB2_F64)
        one_hot_kernel<double><<<grid, RG_THREADS, 0, as_stream(stream)>>>(
            static_cast<const double *>(arg), ld, rows, static_cast<const int64_t *>(dev_src),
            static_cast<const int64_t *>(dev_hot), static_cast<const int64_t *>(dev_width), cols_res,
            static_cast<double *>(res), res_ld, static_cast<int32_t *>(dev_status));
    else
        one_hot_kernel<int64_t><<<grid, RG_THREADS, 0, as_stream(stream)>>>(
            static_cast<const int64_t *>(arg), ld, rows, static_cast<const int64_t *>(dev_src),
            static_cast<const int64_t *>(dev_hot), static_cast<const int64_t *>(dev_width), cols_res,
            static_cast<int64_t *>(res), res_ld, static_cast<int32_t *>(dev_status));
    return after_launch("one_hot_kernel");
}

int db2_oneHot(db2_context *ctx, db2_matrix **res, db2_matrix *arg, db2_matrix *info) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg && info, DB2_EINVAL, "null argument");
    DB2_CHECK(info->dtype == DB2_I64, DB2_EUNSUPPORTED, "OneHot: parameter 'info' must be an int64 matrix");
    DB2_CHECK(info->rows == 1, DB2_EINVAL, "OneHot - parameter 'info' must be a row matrix");
    DB2_CHECK(info->cols == arg->cols, DB2_EINVAL,
              "OneHot - parameter 'info' must provide information for each column of parameter arg");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    std::vector<int64_t> inf((size_t)info->cols);
    if (info->cols > 0)
        DB2_TRY(db2_matrix_to_host(info, inf.data(), info->cols));
    std::vector<int64_t> table; // [src | hot | width], cols_res entries each
    std::vector<int64_t> src, hot, width;
    for (int64_t c = 0; c < arg->cols; c++) {
        const int64_t n = inf[(size_t)c];
        DB2_CHECK(n >= -1, DB2_EINVAL, "OneHot: parameter 'info' must be an integer greater or equal than -1");
        if (n == -1) {
            src.push_back(c), hot.push_back(-1), width.push_back(0);
        } else {
            DB2_CHECK((int64_t)src.size() + n <= ((int64_t)1 << 31), DB2_EUNSUPPORTED, "OneHot: result too wide");
            for (int64_t k = 0; k < n; k++)
                src.push_back(c), hot.push_back(k), width.push_back(n);
        }
    }
    const int64_t cols_res = (int64_t)src.size();
    DB2_CHECK(cols_res > 0, DB2_EINVAL, "OneHot: parameter 'info' must contain at least one non-zero entry");
    DB2_TRY(ensure_device(arg));
    DB2_TRY(prepare_result(ctx, res, arg->dtype, arg->rows, cols_res));
    if (arg->rows > 0) {
        table.reserve((size_t)cols_res * 3);
        table.insert(table.end(), src.begin(), src.end());
        table.insert(table.end(), hot.begin(), hot.end());
        table.insert(table.end(), width.begin(), width.end());
        void *dev = nullptr;
        const size_t tb = (size_t)cols_res * 3 * 8;
        DB2_TRY(ctx_scratch(ctx, tb + 16, &dev));
        int32_t *status = reinterpret_cast<int32_t *>(static_cast<char *>(dev) + tb);
        DB2_CUDA(cudaMemcpyAsync(dev, table.data(), tb, cudaMemcpyHostToDevice, ctx->stream));
        DB2_CUDA(cudaMemsetAsync(status, 0, 4, ctx->stream));
        const int64_t *t = static_cast<const int64_t *>(dev);
        DB2_TRY(db2k_one_hot(arg->dtype, arg->dev_ptr(), arg->dev_ld, arg->rows, t, t + cols_res, t + 2 * cols_res,
                             cols_res, (*res)->dev_ptr(), (*res)->dev_ld, status, ctx->stream));
        int32_t flag = 0; // the reference throws on a value outside its block: the status is read before returning
        DB2_CUDA(cudaMemcpyAsync(&flag, status, 4, cudaMemcpyDeviceToHost, ctx->stream));
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
        DB2_CHECK(flag == 0, DB2_EDOMAIN,
                  "OneHot: arg values that are encoded (info value != -1) must be positive and smaller than the "
                  "corresponding info value");
    }
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_colBind(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && lhs && rhs, DB2_EINVAL, "null argument");
    DB2_CHECK(lhs->dtype == rhs->dtype, DB2_EUNSUPPORTED, "ColBind: operands of different value types");
    DB2_CHECK(lhs->rows == rhs->rows, DB2_EINVAL,
              "ColBind - the two operands must have the same number of rows, but lhs has %lld and rhs has %lld rows",
              (long long)lhs->rows, (long long)rhs->rows);
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(lhs));
    DB2_TRY(ensure_device(rhs));
    DB2_TRY(prepare_result(ctx, res, lhs->dtype, lhs->rows, lhs->cols + rhs->cols));
    DB2_TRY(db2k_col_bind(lhs->dtype, lhs->dev_ptr(), lhs->dev_ld, lhs->cols, rhs->dev_ptr(), rhs->dev_ld, rhs->cols,
                          lhs->rows, (*res)->dev_ptr(), (*res)->dev_ld, ctx->stream));
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_extractCol(db2_context *ctx, db2_matrix **res, db2_matrix *arg, db2_matrix *sel) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg && sel, DB2_EINVAL, "null argument");
    DB2_CHECK(sel->dtype == DB2_I64, DB2_EUNSUPPORTED, "ExtractCol: the column selection must be an int64 matrix");
    DB2_CHECK(sel->cols == 1, DB2_EINVAL,
              "invalid argument passed to ExtractCol: column selection must be given as column matrix but has '%lld' "
              "columns instead of one",
              (long long)sel->cols);
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    // the selection is small: it is validated on the host, with the reference's rules and message
    const int64_t nsel = sel->rows;
    std::vector<int64_t> pos((size_t)nsel);
    if (nsel > 0)
        DB2_TRY(db2_matrix_to_host(sel, pos.data(), 1));
    for (int64_t c = 0; c < nsel; c++) {
        const int64_t given = pos[(size_t)c];
        int64_t p = given;
        if (p < 0)
            p += arg->cols;
        DB2_CHECK(p >= 0 && p < arg->cols, DB2_EDOMAIN,
                  "invalid argument '%lld' passed to ExtractCol: out of bounds for dense matrix with column boundaries "
                  "'[0, %lld)'",
                  (long long)given, (long long)arg->cols);
        pos[(size_t)c] = p;
    }
    DB2_TRY(ensure_device(arg));
    DB2_TRY(prepare_result(ctx, res, arg->dtype, arg->rows, nsel));
    if (arg->rows > 0 && nsel > 0) {
        void *dev_pos = nullptr;
        DB2_TRY(ctx_scratch(ctx, (size_t)nsel * 8, &dev_pos));
        DB2_CUDA(cudaMemcpyAsync(dev_pos, pos.data(), (size_t)nsel * 8, cudaMemcpyHostToDevice, ctx->stream));
        DB2_TRY(db2k_extract_col(arg->dtype, arg->dev_ptr(), arg->dev_ld, arg->rows, dev_pos, nsel, (*res)->dev_ptr(),
                                 (*res)->dev_ld, ctx->stream));
        // `pos` is pageable host memory: the copy above has consumed it when the call returns
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
