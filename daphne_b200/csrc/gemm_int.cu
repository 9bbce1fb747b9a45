// MatMul for the integer value types (int64_t, int32_t): res = op(lhs) @ op(rhs).
//
// The reference sends these to Eigen (src/runtime/local/kernels/MatMul.cpp:40-57 dot, :78-134 gemv, gemm below them;
// Eigen is a third-party dependency that is not part of the reference tree).  Integer addition and multiplication
// wrap and are associative, so every summation order gives the same bits: parity is bit-exact against the plain
// triple loop.  The arithmetic is done on the unsigned type (two's complement wrap without signed overflow).
//
// 64 x 64 result tile per CTA of 256 threads, 4 x 4 results per thread, the operands staged through shared memory in
// slices of 16 along the contraction index; a transposed operand is read through swapped strides, so none of the four
// combinations needs a copy.
#include "common.cuh"

namespace db2 {

constexpr int IT_M = 64, IT_N = 64, IT_K = 16;

template <typename U>
__global__ void __launch_bounds__(256)
    gemm_int_kernel(const U *__restrict__ A, int64_t a_rs, int64_t a_cs, const U *__restrict__ B, int64_t b_rs,
                    int64_t b_cs, U *__restrict__ C, int64_t ldc, int64_t M, int64_t N, int64_t K) {
    // op(A)(i, l) = A[i * a_rs + l * a_cs], op(B)(l, j) = B[l * b_rs + j * b_cs]
    __shared__ U sa[IT_K][IT_M + 1], sb[IT_K][IT_N + 1];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int64_t i0 = (int64_t)blockIdx.y * IT_M, j0 = (int64_t)blockIdx.x * IT_N;
    U acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++)
            acc[a][b] = 0;
    for (int64_t l0 = 0; l0 < K; l0 += IT_K) {
        // 16 x 64 elements per operand and slice, 4 per thread; the faster-running index follows the unit stride
        for (int e = tid; e < IT_K * IT_M; e += 256) {
            const int l = a_cs == 1 ? e % IT_K : e / IT_M, i = a_cs == 1 ? e / IT_K : e % IT_M;
            sa[l][i] = (i0 + i < M && l0 + l < K) ? A[(i0 + i) * a_rs + (l0 + l) * a_cs] : (U)0;
        }
        for (int e = tid; e < IT_K * IT_N; e += 256) {
            const int l = b_cs == 1 ? e / IT_N : e % IT_K, j = b_cs == 1 ? e % IT_N : e / IT_K;
            sb[l][j] = (j0 + j < N && l0 + l < K) ? B[(l0 + l) * b_rs + (j0 + j) * b_cs] : (U)0;
        }
        __syncthreads();
#pragma unroll
        for (int l = 0; l < IT_K; l++) {
            U av[4], bv[4];
#pragma unroll
            for (int a = 0; a < 4; a++)
                av[a] = sa[l][ty * 4 + a];
#pragma unroll
            for (int b = 0; b < 4; b++)
                bv[b] = sb[l][tx * 4 + b];
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++)
                    acc[a][b] += av[a] * bv[b];
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int64_t i = i0 + ty * 4 + a, j = j0 + tx * 4 + b;
            if (i < M && j < N)
                C[i * ldc + j] = acc[a][b];
        }
}

template <typename U>
static int launch_gemm_int(const void *lhs, int64_t lhs_ld, bool ta, const void *rhs, int64_t rhs_ld, bool tb, void *res,
                           int64_t ldc, int64_t m, int64_t n, int64_t k, cudaStream_t st) {
    if (m == 0 || n == 0)
        return DB2_OK;
    DB2_CHECK((m + IT_M - 1) / IT_M <= 65535, DB2_EUNSUPPORTED, "integer matMul: more than 4,194,240 result rows");
    dim3 grid((unsigned)((n + IT_N - 1) / IT_N), (unsigned)((m + IT_M - 1) / IT_M));
    gemm_int_kernel<U><<<grid, 256, 0, st>>>(static_cast<const U *>(lhs), ta ? 1 : lhs_ld, ta ? lhs_ld : 1,
                                             static_cast<const U *>(rhs), tb ? 1 : rhs_ld, tb ? rhs_ld : 1,
                                             static_cast<U *>(res), ldc, m, n, k);
    return after_launch("gemm_int_kernel");
}

int gemm_int(int dtype, const void *lhs, int64_t lhs_ld, bool ta, const void *rhs, int64_t rhs_ld, bool tb, void *res,
             int64_t ldc, int64_t m, int64_t n, int64_t k, cudaStream_t st) {
    if (dtype == DB2_I64 || dtype == DB2_U64)
        return launch_gemm_int<unsigned long long>(lhs, lhs_ld, ta, rhs, rhs_ld, tb, res, ldc, m, n, k, st);
    return launch_gemm_int<unsigned int>(lhs, lhs_ld, ta, rhs, rhs_ld, tb, res, ldc, m, n, k, st);
}

} // namespace db2
