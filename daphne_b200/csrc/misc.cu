// Small helper kernels called between the hot operators: transpose, fill, seq, diagMatrix, ctable.
#include "common.cuh"

namespace db2 {

// ---------------------------------------------------------------------------
// transpose: 32 x 32 tiles through shared memory (both sides coalesced)
// ---------------------------------------------------------------------------
template <typename VT>
__global__ void transpose_kernel(const VT *__restrict__ in, int64_t rows, int64_t cols, int64_t ld,
                                 VT *__restrict__ out, int64_t out_ld) {
    __shared__ VT tile[32][33];
    const int64_t tiles_c = (cols + 31) / 32;
    const int64_t ntiles = ((rows + 31) / 32) * tiles_c;
    for (int64_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
        const int64_t r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
        for (int y = threadIdx.y; y < 32; y += blockDim.y) {
            const int64_t r = r0 + y, c = c0 + threadIdx.x;
            if (r < rows && c < cols)
                tile[y][threadIdx.x] = in[r * ld + c];
        }
        __syncthreads();
        for (int y = threadIdx.y; y < 32; y += blockDim.y) {
            const int64_t c = c0 + y, r = r0 + threadIdx.x;
            if (r < rows && c < cols)
                out[c * out_ld + r] = tile[threadIdx.x][y];
        }
        __syncthreads();
    }
}

template <typename VT> __global__ void fill_kernel(VT *out, int64_t rows, int64_t cols, int64_t ld, VT value) {
    const int64_t n = rows * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[(i / cols) * ld + (i % cols)] = value;
}

// seq(start, end, inc): element i is start + i * inc (the reference accumulates by repeated addition; the closed form
// is exact for the integer-valued sequences used as vertex ids and row indices)
template <typename VT> __global__ void seq_kernel(VT *out, int64_t n, VT start, VT inc) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = start + (VT)i * inc;
}

// diagMatrix: n x n with the vector on the diagonal
template <typename VT>
__global__ void diag_kernel(const VT *__restrict__ vec, int64_t vec_ld, int64_t n, VT *__restrict__ out, int64_t ld) {
    const int64_t total = n * n;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / n, c = i % n;
        out[r * ld + c] = (r == c) ? vec[r * vec_ld] : (VT)0;
    }
}

// ctable (dense result): res[lhs[i], rhs[i]] += weight.  The additions to one cell are all the same value, so their
// order does not matter and atomics give the exact result of the reference's serial scatter for integer-valued
// weights; out-of-range coordinates are ignored when the result shape was given (CTable.h:98-103).
__global__ void ctable_kernel(const int64_t *__restrict__ lhs, int64_t lhs_ld, const int64_t *__restrict__ rhs,
                              int64_t rhs_ld, int64_t n, double weight, double *__restrict__ out, int64_t rows,
                              int64_t cols, int64_t ld) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = lhs[i * lhs_ld], c = rhs[i * rhs_ld];
        if (r >= 0 && c >= 0 && r < rows && c < cols)
            atomicAdd(out + r * ld + c, weight);
    }
}
// row-major one-hot form used when every row index occurs once in order (lhs = seq(0, n-1)): no atomics, pure store
__global__ void ctable_onehot_kernel(const int64_t *__restrict__ rhs, int64_t rhs_ld, int64_t n, double weight,
                                     double *__restrict__ out, int64_t cols, int64_t ld) {
    const int64_t total = n * cols;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / cols, c = i % cols;
        out[r * ld + c] = (rhs[r * rhs_ld] == c) ? weight : 0.0;
    }
}

__global__ void max_i64_kernel(const int64_t *__restrict__ v, int64_t ld, int64_t n, long long *out) {
    long long m = INT64_MIN;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        m = max(m, (long long)v[i * ld]);
    for (int o = 16; o >= 1; o >>= 1)
        m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (threadIdx.x % 32 == 0)
        atomicMax(out, m);
}

static int grid_for(int64_t n, int threads) {
    int64_t want = (n + threads - 1) / threads;
    const int64_t cap = (int64_t)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

} // namespace db2

using namespace db2;

extern "C" int db2k_transpose(int dtype, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                              int64_t res_ld, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    if (rows * cols == 0)
        return DB2_OK;
    const int64_t ntiles = ((rows + 31) / 32) * ((cols + 31) / 32);
    const int64_t cap = (int64_t)sm_count() * 8;
    const int grid = (int)(ntiles < cap ? ntiles : cap);
    if (dtype_size(dtype) == 8)
        transpose_kernel<uint64_t><<<grid, dim3(32, 8), 0, as_stream(stream)>>>(
            static_cast<const uint64_t *>(arg), rows, cols, ld, static_cast<uint64_t *>(res), res_ld);
    else
        transpose_kernel<uint32_t><<<grid, dim3(32, 8), 0, as_stream(stream)>>>(
            static_cast<const uint32_t *>(arg), rows, cols, ld, static_cast<uint32_t *>(res), res_ld);
    return after_launch("transpose_kernel");
}

extern "C" int db2k_fill(int dtype, void *res, int64_t rows, int64_t cols, int64_t ld, const void *value,
                         void *stream) {
    DB2_CHECK(value, DB2_EINVAL, "null value");
    if (rows * cols == 0)
        return DB2_OK;
    const int grid = grid_for(rows * cols, 256);
    if (dtype_size(dtype) == 1)
        fill_kernel<uint8_t><<<grid, 256, 0, as_stream(stream)>>>(static_cast<uint8_t *>(res), rows, cols, ld,
                                                                 *static_cast<const uint8_t *>(value));
    else if (dtype_size(dtype) == 8)
        fill_kernel<uint64_t><<<grid, 256, 0, as_stream(stream)>>>(static_cast<uint64_t *>(res), rows, cols, ld,
                                                                  *static_cast<const uint64_t *>(value));
    else
        fill_kernel<uint32_t><<<grid, 256, 0, as_stream(stream)>>>(static_cast<uint32_t *>(res), rows, cols, ld,
                                                                  *static_cast<const uint32_t *>(value));
    return after_launch("fill_kernel");
}

extern "C" int db2k_seq(int dtype, void *res, int64_t n, const void *start, const void *inc, void *stream) {
    DB2_CHECK(start && inc, DB2_EINVAL, "null argument");
    if (n == 0)
        return DB2_OK;
    const int grid = grid_for(n, 256);
    DB2_DISPATCH_DTYPE(dtype, VT,
                       (seq_kernel<VT><<<grid, 256, 0, as_stream(stream)>>>(static_cast<VT *>(res), n,
                                                                            *static_cast<const VT *>(start),
                                                                            *static_cast<const VT *>(inc))));
    return after_launch("seq_kernel");
}

extern "C" int db2k_diag_matrix(int dtype, const void *vec, int64_t vec_ld, int64_t n, void *res, int64_t res_ld,
                                void *stream) {
    if (n == 0)
        return DB2_OK;
    const int grid = grid_for(n * n, 256);
    DB2_DISPATCH_DTYPE(dtype, VT,
                       (diag_kernel<VT><<<grid, 256, 0, as_stream(stream)>>>(static_cast<const VT *>(vec), vec_ld, n,
                                                                             static_cast<VT *>(res), res_ld)));
    return after_launch("diag_kernel");
}

extern "C" int db2k_max_i64(const void *vec, int64_t ld, int64_t n, void *dev_out, void *stream) {
    DB2_CHECK(n > 0, DB2_EINVAL, "empty vector");
    const long long init = INT64_MIN;
    DB2_CUDA(cudaMemcpyAsync(dev_out, &init, 8, cudaMemcpyHostToDevice, as_stream(stream)));
    max_i64_kernel<<<grid_for(n, 256), 256, 0, as_stream(stream)>>>(static_cast<const int64_t *>(vec), ld, n,
                                                                   static_cast<long long *>(dev_out));
    return after_launch("max_i64_kernel");
}

extern "C" int db2k_ctable(const void *lhs, int64_t lhs_ld, const void *rhs, int64_t rhs_ld, int64_t n, double weight,
                           void *res, int64_t res_rows, int64_t res_cols, int64_t res_ld, int lhs_is_row_index,
                           void *stream) {
    DB2_CHECK(res_rows >= 0 && res_cols >= 0, DB2_EINVAL, "negative result shape");
    if (res_rows * res_cols == 0)
        return DB2_OK;
    cudaStream_t st = as_stream(stream);
    if (lhs_is_row_index && res_rows == n) {
        ctable_onehot_kernel<<<grid_for(n * res_cols, 256), 256, 0, st>>>(static_cast<const int64_t *>(rhs), rhs_ld, n,
                                                                         weight, static_cast<double *>(res), res_cols,
                                                                         res_ld);
        return after_launch("ctable_onehot_kernel");
    }
    if (res_ld == res_cols)
        DB2_CUDA(cudaMemsetAsync(res, 0, (size_t)res_rows * res_cols * 8, st));
    else
        DB2_CUDA(cudaMemset2DAsync(res, (size_t)res_ld * 8, 0, (size_t)res_cols * 8, (size_t)res_rows, st));
    if (n > 0) {
        ctable_kernel<<<grid_for(n, 256), 256, 0, st>>>(static_cast<const int64_t *>(lhs), lhs_ld,
                                                       static_cast<const int64_t *>(rhs), rhs_ld, n, weight,
                                                       static_cast<double *>(res), res_rows, res_cols, res_ld);
        return after_launch("ctable_kernel");
    }
    return DB2_OK;
}
