// Elementwise kernels: matrix (op) matrix with row/column-vector broadcast, matrix (op) scalar, unary.
//
// All three are HBM-bound: per result element one or two loads and one store.  Layout of the work:
//   * contiguous operands without broadcast are treated as one flat array: every thread moves 16-byte packets
//     (2 x f64 / 4 x f32), UNROLL packets in flight per thread, grid = a multiple of the SM count, grid-stride loop;
//   * broadcast or strided (ld != cols) operands use a 2-D mapping: threadIdx.x walks the packets of a row,
//     threadIdx.y walks rows, so no per-element division or modulo is ever computed and the broadcast vector is
//     read from registers/L1 (row vector) or once per row (column vector).
// Indexing is 64-bit throughout.
#include "ops.cuh"

namespace db2 {

constexpr int EW_THREADS = 256;
constexpr int EW_UNROLL = 4;

// ---------------------------------------------------------------------------
// flat kernels
// ---------------------------------------------------------------------------
template <int OP, typename VT>
__global__ void __launch_bounds__(EW_THREADS)
    ew_bin_flat_kernel(const VT *__restrict__ lhs, const VT *__restrict__ rhs, VT *__restrict__ res, int64_t n) {
    constexpr int N = Pack<VT>::N;
    const int64_t npk = n / N;
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
    int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    for (; i + (EW_UNROLL - 1) * stride < npk; i += EW_UNROLL * stride) {
        Pack<VT> a[EW_UNROLL], b[EW_UNROLL];
#pragma unroll
        for (int u = 0; u < EW_UNROLL; u++) {
            a[u] = ld_pack_stream(lhs + (i + u * stride) * N);
            b[u] = ld_pack_stream(rhs + (i + u * stride) * N);
        }
#pragma unroll
        for (int u = 0; u < EW_UNROLL; u++) {
            Pack<VT> r;
#pragma unroll
            for (int k = 0; k < N; k++)
                r.v[k] = binary_op<OP>(a[u].v[k], b[u].v[k]);
            st_pack_stream(res + (i + u * stride) * N, r);
        }
    }
    for (; i < npk; i += stride) {
        Pack<VT> a = ld_pack_stream(lhs + i * N), b = ld_pack_stream(rhs + i * N), r;
#pragma unroll
        for (int k = 0; k < N; k++)
            r.v[k] = binary_op<OP>(a.v[k], b.v[k]);
        st_pack_stream(res + i * N, r);
    }
    // tail elements (n % N)
    const int64_t t = npk * N + (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    if (t < n)
        res[t] = binary_op<OP>(lhs[t], rhs[t]);
}

template <int OP, typename VT>
__global__ void __launch_bounds__(EW_THREADS)
    ew_sca_flat_kernel(const VT *__restrict__ lhs, VT s, VT *__restrict__ res, int64_t n) {
    constexpr int N = Pack<VT>::N;
    const int64_t npk = n / N;
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
    int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    for (; i + (EW_UNROLL - 1) * stride < npk; i += EW_UNROLL * stride) {
        Pack<VT> a[EW_UNROLL];
#pragma unroll
        for (int u = 0; u < EW_UNROLL; u++)
            a[u] = ld_pack_stream(lhs + (i + u * stride) * N);
#pragma unroll
        for (int u = 0; u < EW_UNROLL; u++) {
            Pack<VT> r;
#pragma unroll
            for (int k = 0; k < N; k++)
                r.v[k] = binary_op<OP>(a[u].v[k], s);
            st_pack_stream(res + (i + u * stride) * N, r);
        }
    }
    for (; i < npk; i += stride) {
        Pack<VT> a = ld_pack_stream(lhs + i * N), r;
#pragma unroll
        for (int k = 0; k < N; k++)
            r.v[k] = binary_op<OP>(a.v[k], s);
        st_pack_stream(res + i * N, r);
    }
    const int64_t t = npk * N + (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    if (t < n)
        res[t] = binary_op<OP>(lhs[t], s);
}

template <int OP, typename VT>
__global__ void __launch_bounds__(EW_THREADS)
    ew_un_flat_kernel(const VT *__restrict__ arg, VT *__restrict__ res, int64_t n, int32_t *status) {
    constexpr int N = Pack<VT>::N;
    const int64_t npk = n / N;
    const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
    bool bad = false;
    int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    for (; i + (EW_UNROLL - 1) * stride < npk; i += EW_UNROLL * stride) {
        Pack<VT> a[EW_UNROLL];
#pragma unroll
        for (int u = 0; u < EW_UNROLL; u++)
            a[u] = ld_pack_stream(arg + (i + u * stride) * N);
#pragma unroll
        for (int u = 0; u < EW_UNROLL; u++) {
            Pack<VT> r;
#pragma unroll
            for (int k = 0; k < N; k++)
                r.v[k] = unary_op<OP>(a[u].v[k], bad);
            st_pack_stream(res + (i + u * stride) * N, r);
        }
    }
    for (; i < npk; i += stride) {
        Pack<VT> a = ld_pack_stream(arg + i * N), r;
#pragma unroll
        for (int k = 0; k < N; k++)
            r.v[k] = unary_op<OP>(a.v[k], bad);
        st_pack_stream(res + i * N, r);
    }
    const int64_t t = npk * N + (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
    if (t < n)
        res[t] = unary_op<OP>(arg[t], bad);
    if (bad && status)
        atomicExch(status, 1);
}

// ---------------------------------------------------------------------------
// 2-D kernels (broadcast / strided).  blockDim = (TX, EW_THREADS / TX); TX = power of two <= 256 covering the
// packets of one row.  MODE: 0 = same shape, 1 = rhs is a row vector, 2 = rhs is a column vector, 3 = rhs scalar,
// 4 = unary.  VEC = elements per access (Pack<VT>::N when all row starts are 16-byte aligned, else 1).
// ---------------------------------------------------------------------------
template <int OP, typename VT, int MODE, int VEC>
__global__ void __launch_bounds__(EW_THREADS)
    ew_2d_kernel(const VT *__restrict__ lhs, int64_t lld, const VT *__restrict__ rhs, int64_t rld, VT s,
                 VT *__restrict__ res, int64_t res_ld, int64_t rows, int64_t cols, int32_t *status) {
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t row_stride = (int64_t)gridDim.x * blockDim.y;
    const int64_t col_stride = (int64_t)blockDim.x * VEC;
    bool bad = false;
    for (int64_t c0 = (int64_t)tx * VEC; c0 < cols; c0 += col_stride) {
        const int nv = (cols - c0 < VEC) ? (int)(cols - c0) : VEC; // ragged last packet (only when VEC == 1 or tail)
        VT rv[VEC];
        if constexpr (MODE == 1) {
#pragma unroll
            for (int k = 0; k < VEC; k++)
                rv[k] = (k < nv) ? rhs[c0 + k] : (VT)0;
        }
        for (int64_t r = (int64_t)blockIdx.x * blockDim.y + ty; r < rows; r += row_stride) {
            const VT *lp = lhs + r * lld + c0;
            VT *rp = res + r * res_ld + c0;
            VT a[VEC], b[VEC], o[VEC];
            if (nv == VEC) {
                if constexpr (VEC > 1) {
                    Pack<VT> pa = ld_pack_stream(lp);
#pragma unroll
                    for (int k = 0; k < VEC; k++)
                        a[k] = pa.v[k];
                } else
                    a[0] = lp[0];
            } else {
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    a[k] = (k < nv) ? lp[k] : (VT)0;
            }
            if constexpr (MODE == 0) {
                const VT *bp = rhs + r * rld + c0;
                if (nv == VEC && VEC > 1) {
                    Pack<VT> pb = ld_pack_stream(bp);
#pragma unroll
                    for (int k = 0; k < VEC; k++)
                        b[k] = pb.v[k];
                } else {
#pragma unroll
                    for (int k = 0; k < VEC; k++)
                        b[k] = (k < nv) ? bp[k] : (VT)0;
                }
            } else if constexpr (MODE == 1) {
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    b[k] = rv[k];
            } else if constexpr (MODE == 2) {
                const VT x = rhs[r * rld];
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    b[k] = x;
            } else {
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    b[k] = s;
            }
#pragma unroll
            for (int k = 0; k < VEC; k++) {
                if constexpr (MODE == 4)
                    o[k] = (k < nv) ? unary_op<OP>(a[k], bad) : (VT)0;
                else
                    o[k] = binary_op<OP>(a[k], b[k]);
            }
            if (nv == VEC) {
                if constexpr (VEC > 1) {
                    Pack<VT> po;
#pragma unroll
                    for (int k = 0; k < VEC; k++)
                        po.v[k] = o[k];
                    st_pack_stream(rp, po);
                } else
                    rp[0] = o[0];
            } else {
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    if (k < nv)
                        rp[k] = o[k];
            }
        }
    }
    if constexpr (MODE == 4) {
        if (bad && status)
            atomicExch(status, 1);
    }
}

static int flat_grid(int64_t npk) {
    const int64_t per_block = (int64_t)EW_THREADS * EW_UNROLL;
    int64_t want = (npk + per_block - 1) / per_block;
    const int64_t cap = (int64_t)sm_count() * 8; // 8 resident CTAs of 256 threads per SM
    if (want > cap)
        want = cap;
    if (want < 1)
        want = 1;
    return (int)want;
}

struct Grid2D {
    dim3 block;
    int grid;
};
static Grid2D grid_2d(int64_t rows, int64_t cols, int vec) {
    const int64_t packets = (cols + vec - 1) / vec;
    int tx = next_pow2(packets);
    if (tx > EW_THREADS)
        tx = EW_THREADS;
    const int ty = EW_THREADS / tx;
    int64_t want = (rows + ty - 1) / ty;
    const int64_t cap = (int64_t)sm_count() * 8;
    // keep at least 4 rows per thread-row in flight when there is enough work
    if (want > cap)
        want = cap;
    if (want < 1)
        want = 1;
    return {dim3(tx, ty, 1), (int)want};
}

template <typename VT> static bool rows_aligned(const void *p, int64_t ld) {
    return aligned16(p) && ((ld * (int64_t)sizeof(VT)) % 16 == 0);
}

template <int OP, typename VT, int MODE>
static int launch_2d(const VT *lhs, int64_t lld, const VT *rhs, int64_t rld, VT s, VT *res, int64_t res_ld,
                     int64_t rows, int64_t cols, int32_t *status, cudaStream_t st) {
    constexpr int N = Pack<VT>::N;
    bool vec_ok = rows_aligned<VT>(lhs, lld) && rows_aligned<VT>(res, res_ld) && (cols % N == 0);
    if (MODE == 0)
        vec_ok = vec_ok && rows_aligned<VT>(rhs, rld);
    if (vec_ok) {
        Grid2D g = grid_2d(rows, cols, N);
        ew_2d_kernel<OP, VT, MODE, N><<<g.grid, g.block, 0, st>>>(lhs, lld, rhs, rld, s, res, res_ld, rows, cols,
                                                                     status);
    } else {
        Grid2D g = grid_2d(rows, cols, 1);
        ew_2d_kernel<OP, VT, MODE, 1><<<g.grid, g.block, 0, st>>>(lhs, lld, rhs, rld, s, res, res_ld, rows, cols,
                                                                     status);
    }
    return after_launch("ew_2d_kernel");
}

template <int OP, typename VT>
static int ew_binary_impl(const VT *lhs, int64_t lr, int64_t lc, int64_t lld, const VT *rhs, int64_t rr, int64_t rc,
                          int64_t rld, VT *res, int64_t res_ld, cudaStream_t st) {
    if (lr == 0 || lc == 0)
        return DB2_OK;
    // shape cases in the order the reference tests them (EwBinaryMat.h:72-107)
    if (lr == rr && lc == rc) {
        const bool contiguous = (lld == lc && rld == rc && res_ld == lc) || lr == 1;
        if (contiguous && aligned16(lhs) && aligned16(rhs) && aligned16(res)) {
            const int64_t n = lr * lc;
            ew_bin_flat_kernel<OP, VT><<<flat_grid(n / Pack<VT>::N), EW_THREADS, 0, st>>>(lhs, rhs, res, n);
            return after_launch("ew_bin_flat_kernel");
        }
        return launch_2d<OP, VT, 0>(lhs, lld, rhs, rld, (VT)0, res, res_ld, lr, lc, nullptr, st);
    } else if (lc == rc && (rr == 1 || lr == 1)) {
        return launch_2d<OP, VT, 1>(lhs, lld, rhs, rld, (VT)0, res, res_ld, lr, lc, nullptr, st);
    } else if (lr == rr && (rc == 1 || lc == 1)) {
        return launch_2d<OP, VT, 2>(lhs, lld, rhs, rld, (VT)0, res, res_ld, lr, lc, nullptr, st);
    }
    return set_error(DB2_EINVAL,
                     "EwBinaryMat(Dense) - lhs and rhs must either have the same dimensions, or one of them must be "
                     "a row/column vector with the width/height of the other, but lhs has shape (%lld x %lld) and "
                     "rhs has shape (%lld x %lld)",
                     (long long)lr, (long long)lc, (long long)rr, (long long)rc);
}

// res[r][c] = lhs[r] (op) rhs[c]: a warp writes whole rows (coalesced), four rows in flight; nothing but the two
// vectors is read, so the pass is bound by the write stream
template <int OP, typename VT>
__global__ void __launch_bounds__(EW_THREADS)
    ew_outer_kernel(const VT *__restrict__ lhs, int64_t lld, const VT *__restrict__ rhs, VT *__restrict__ res,
                    int64_t res_ld, int64_t rows, int64_t cols) {
    const int lane = threadIdx.x % 32;
    const int64_t warp = ((int64_t)blockIdx.x * EW_THREADS + threadIdx.x) / 32;
    const int64_t nwarps = (int64_t)gridDim.x * (EW_THREADS / 32);
    for (int64_t r0 = warp * 4; r0 < rows; r0 += nwarps * 4) {
        VT a[4];
#pragma unroll
        for (int u = 0; u < 4; u++)
            a[u] = r0 + u < rows ? lhs[(r0 + u) * lld] : (VT)0;
        for (int64_t c = lane; c < cols; c += 32) {
            const VT b = rhs[c];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (r0 + u < rows)
                    res[(r0 + u) * res_ld + c] = binary_op<OP>(a[u], b);
        }
    }
}

template <int OP, typename VT>
static int ew_outer_impl(const VT *lhs, int64_t lld, const VT *rhs, VT *res, int64_t res_ld, int64_t rows,
                         int64_t cols, cudaStream_t st) {
    const int64_t want = (rows + 31) / 32, cap = (int64_t)sm_count() * 8;
    const int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    ew_outer_kernel<OP, VT><<<grid, EW_THREADS, 0, st>>>(lhs, lld, rhs, res, res_ld, rows, cols);
    return after_launch("ew_outer_kernel");
}

} // namespace db2

using namespace db2;

extern "C" int db2k_outer_binary(int dtype, int op, const void *lhs, int64_t lhs_ld, int64_t rows, const void *rhs,
                                 int64_t cols, void *res, int64_t res_ld, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    if (rows == 0 || cols == 0)
        return DB2_OK;
    DB2_CHECK(lhs && rhs && res, DB2_EINVAL, "null operand");
    DB2_DISPATCH_DTYPE(dtype, VT, DB2_DISPATCH_BINOP(op, OP, return (ew_outer_impl<OP, VT>(
                                                                 (const VT *)lhs, lhs_ld, (const VT *)rhs, (VT *)res,
                                                                 res_ld, rows, cols, as_stream(stream)))));
    return DB2_OK;
}

extern "C" int db2k_ew_binary(int dtype, int op, const void *lhs, int64_t lhs_rows, int64_t lhs_cols,
                              int64_t lhs_ld, const void *rhs, int64_t rhs_rows, int64_t rhs_cols, int64_t rhs_ld,
                              void *res, int64_t res_ld, void *stream) {
    DB2_CHECK(lhs_rows >= 0 && lhs_cols >= 0 && rhs_rows >= 0 && rhs_cols >= 0, DB2_EINVAL, "negative dimension");
    DB2_CHECK((lhs && rhs && res) || lhs_rows * lhs_cols == 0, DB2_EINVAL, "null operand");
    DB2_DISPATCH_DTYPE_EW(dtype, VT, DB2_DISPATCH_BINOP(op, OP, return (ew_binary_impl<OP, VT>(
                                                                 (const VT *)lhs, lhs_rows, lhs_cols, lhs_ld,
                                                                 (const VT *)rhs, rhs_rows, rhs_cols, rhs_ld, (VT *)res,
                                                                 res_ld, as_stream(stream)))));
    return DB2_OK;
}

template <int OP, typename VT>
static int ew_sca_impl(const VT *lhs, int64_t rows, int64_t cols, int64_t ld, VT s, VT *res, int64_t res_ld,
                       cudaStream_t st) {
    if (rows == 0 || cols == 0)
        return DB2_OK;
    const bool contiguous = (ld == cols && res_ld == cols) || rows == 1;
    if (contiguous && aligned16(lhs) && aligned16(res)) {
        const int64_t n = rows * cols;
        ew_sca_flat_kernel<OP, VT><<<flat_grid(n / Pack<VT>::N), EW_THREADS, 0, st>>>(lhs, s, res, n);
        return after_launch("ew_sca_flat_kernel");
    }
    return launch_2d<OP, VT, 3>(lhs, ld, nullptr, 0, s, res, res_ld, rows, cols, nullptr, st);
}

extern "C" int db2k_ew_binary_sca(int dtype, int op, const void *lhs, int64_t rows, int64_t cols, int64_t ld,
                                  const void *scalar, void *res, int64_t res_ld, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    DB2_CHECK(scalar != nullptr, DB2_EINVAL, "null scalar");
    DB2_CHECK((lhs && res) || rows * cols == 0, DB2_EINVAL, "null operand");
    DB2_DISPATCH_DTYPE_EW(dtype, VT,
                       DB2_DISPATCH_BINOP(op, OP, return (ew_sca_impl<OP, VT>((const VT *)lhs, rows, cols, ld,
                                                                              *(const VT *)scalar, (VT *)res, res_ld,
                                                                              as_stream(stream)))));
    return DB2_OK;
}

template <int OP, typename VT>
static int ew_un_impl(const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, int64_t res_ld, int32_t *status,
                      cudaStream_t st) {
    if (rows == 0 || cols == 0)
        return DB2_OK;
    const bool contiguous = (ld == cols && res_ld == cols) || rows == 1;
    if (contiguous && aligned16(arg) && aligned16(res)) {
        const int64_t n = rows * cols;
        ew_un_flat_kernel<OP, VT><<<flat_grid(n / Pack<VT>::N), EW_THREADS, 0, st>>>(arg, res, n, status);
        return after_launch("ew_un_flat_kernel");
    }
    return launch_2d<OP, VT, 4>(arg, ld, nullptr, 0, (VT)0, res, res_ld, rows, cols, status, st);
}

extern "C" int db2k_ew_unary(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                             int64_t res_ld, int32_t *dev_status, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    DB2_CHECK((arg && res) || rows * cols == 0, DB2_EINVAL, "null operand");
    DB2_DISPATCH_DTYPE(dtype, VT,
                       DB2_DISPATCH_UNOP(op, OP, return (ew_un_impl<OP, VT>((const VT *)arg, rows, cols, ld, (VT *)res,
                                                                            res_ld, dev_status, as_stream(stream)))));
    return DB2_OK;
}
