// Blocked LU with partial pivoting for solve(A, b), one right-hand side (the systems of the normal equations are
// d x d with d = 100 .. 512; LAPACKE_dgesv in the reference, src/runtime/local/kernels/Solve.h:86-116).
//
// Right-looking, panel width NB: (1) the current panel (all remaining rows x NB columns) is factorised by ONE CTA in
// shared memory -- pivot search (first largest |a|, like idamax), row exchange, scaling, rank-1 updates; (2) the row
// exchanges are applied to the other columns and to b, and the block row is solved against the unit lower triangle
// (one thread per column); (3) the trailing matrix and b get the rank-NB update from 32 x 32 tiles.  A final kernel
// does the back substitution.  About 3 launches per 32 columns instead of a single CTA walking the whole trailing
// matrix through L2 for every column (23 ms for d = 512 before, about 1.5 ms now).
#include "common.cuh"

namespace db2 {

constexpr int LU_THREADS = 1024;

// Panel rows k0..n-1, columns k0..k0+nb-1 in shared memory, row pitch nb + 1.
__global__ void __launch_bounds__(LU_THREADS)
    lu_panel_kernel(double *__restrict__ A, int64_t n, int64_t k0, int nb, int *__restrict__ piv,
                    int32_t *__restrict__ status) {
    extern __shared__ double P[];
    __shared__ double s_val[32];
    __shared__ int s_idx[32];
    __shared__ int s_p;
    const int tid = threadIdx.x, nt = blockDim.x;
    const int m = (int)(n - k0), pitch = nb + 1;
    for (int e = tid; e < m * nb; e += nt)
        P[(e / nb) * pitch + e % nb] = A[(k0 + e / nb) * n + k0 + e % nb];
    __syncthreads();
    for (int j = 0; j < nb; j++) {
        double best = -1.0;
        int bi = m;
        for (int i = j + tid; i < m; i += nt) {
            const double v = fabs(P[i * pitch + j]);
            if (v > best || (v == best && i < bi)) {
                best = v;
                bi = i;
            }
        }
        for (int o = 16; o >= 1; o >>= 1) {
            const double ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (tid % 32 == 0) {
            s_val[tid / 32] = best;
            s_idx[tid / 32] = bi;
        }
        __syncthreads();
        if (tid == 0) {
            double b = s_val[0];
            int ix = s_idx[0];
            for (int w = 1; w < nt / 32; w++)
                if (s_val[w] > b || (s_val[w] == b && s_idx[w] < ix)) {
                    b = s_val[w];
                    ix = s_idx[w];
                }
            if (ix >= m) // no candidate was accepted (every remaining entry of the column is NaN): keep row j
                ix = j;
            s_p = ix;
            piv[k0 + j] = (int)k0 + ix;
            if (!(b > 0.0) && *status == 0)
                *status = (int32_t)(k0 + j + 1); // exactly singular (or NaN) pivot
        }
        __syncthreads();
        const int p = s_p;
        if (p != j && p < m)
            for (int c = tid; c < nb; c += nt) {
                const double t = P[j * pitch + c];
                P[j * pitch + c] = P[p * pitch + c];
                P[p * pitch + c] = t;
            }
        __syncthreads();
        const double d = P[j * pitch + j];
        for (int i = j + 1 + tid; i < m; i += nt)
            P[i * pitch + j] = __ddiv_rn(P[i * pitch + j], d);
        __syncthreads();
        const int w = nb - j - 1;
        if (w > 0)
            for (int e = tid; e < (m - j - 1) * w; e += nt) {
                const int i = j + 1 + e / w, c = j + 1 + e % w;
                P[i * pitch + c] = __fma_rn(-P[i * pitch + j], P[j * pitch + c], P[i * pitch + c]);
            }
        __syncthreads();
    }
    for (int e = tid; e < m * nb; e += nt)
        A[(k0 + e / nb) * n + k0 + e % nb] = P[(e / nb) * pitch + e % nb];
}

// The same factorisation for panels of at most 512 rows: one thread per ROW, the row's 32 panel entries in registers.
// Per column: block-wide argmax of |a[j]| (shuffles + one barrier), exchange of the pivot row and row j through shared
// memory (one barrier), then every thread below the diagonal scales its a[j] and updates its remaining entries from
// the broadcast pivot row -- two barriers per column instead of five, no shared-memory traffic for the updates.
constexpr int LU_NB = 32, LU_REG_ROWS = 512;
__global__ void __launch_bounds__(LU_REG_ROWS)
    lu_panel_reg_kernel(double *__restrict__ A, int64_t n, int64_t k0, int nb, int *__restrict__ piv,
                        int32_t *__restrict__ status) {
    // ONE barrier per column: before it every warp publishes its best pivot candidate TOGETHER WITH that candidate's
    // row, and the owner of row j publishes row j; after it every thread folds the warps' candidates to the same
    // pivot p and finds both rows it may need.  The buffers alternate with the column parity, so the writes of column
    // j + 1 cannot overtake the reads of column j - 1 (a thread writes them only after the barrier of column j, which
    // every thread reaches after its reads of column j - 1).
    __shared__ double cand_row[2][LU_REG_ROWS / 32][LU_NB]; // [parity][warp][entries]: row of the warp's candidate
    __shared__ double row_j[2][LU_NB];                      // [parity][entries]: row j before the exchange
    __shared__ double s_val[2][LU_REG_ROWS / 32];
    __shared__ int s_idx[2][LU_REG_ROWS / 32];
    const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32, nwarps = blockDim.x / 32;
    const int m = (int)(n - k0);
    double a[LU_NB];
#pragma unroll
    for (int c = 0; c < LU_NB; c++)
        a[c] = (tid < m && c < nb) ? A[(k0 + tid) * n + k0 + c] : 0.0;
#pragma unroll
    for (int j = 0; j < LU_NB; j++) {
        if (j >= nb)
            break;
        const int par = j & 1;
        // first largest |a[j]| among the rows j .. m-1 (idamax)
        const bool cand = tid >= j && tid < m;
        double best = cand ? fabs(a[j]) : -1.0;
        int bi = cand ? tid : 0x7fffffff;
        if (best != best) // a NaN pivot candidate: treated as "not larger" like the comparison of the scan
            best = -1.0;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const double ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        if (tid == bi) { // this warp's candidate publishes its row
#pragma unroll
            for (int c = 0; c < LU_NB; c++)
                cand_row[par][warp][c] = a[c];
        }
        if (lane == 0) {
            s_val[par][warp] = best;
            s_idx[par][warp] = bi;
        }
        if (tid == j) {
#pragma unroll
            for (int c = 0; c < LU_NB; c++)
                row_j[par][c] = a[c];
        }
        __syncthreads();
        best = lane < nwarps ? s_val[par][lane] : -1.0;
        bi = lane < nwarps ? s_idx[par][lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) {
            const double ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) {
                best = ov;
                bi = oi;
            }
        }
        const int p = bi; // every thread has the same answer; always a row in [j, m): row j is a candidate
        const double *prow = cand_row[par][p / 32];
        if (tid == 0) {
            piv[k0 + j] = (int)k0 + p;
            if (!(best > 0.0) && *status == 0)
                *status = (int32_t)(k0 + j + 1); // exactly singular (or NaN) pivot
        }
        if (p != j) { // the two rows change places
            if (tid == j) {
#pragma unroll
                for (int c = 0; c < LU_NB; c++)
                    a[c] = prow[c];
            } else if (tid == p) {
#pragma unroll
                for (int c = 0; c < LU_NB; c++)
                    a[c] = row_j[par][c];
            }
        }
        if (tid > j && tid < m) {
            const double l = __ddiv_rn(a[j], prow[j]);
            a[j] = l;
#pragma unroll
            for (int c = j + 1; c < LU_NB; c++)
                a[c] = __fma_rn(-l, prow[c], a[c]);
        }
    }
    if (tid < m)
#pragma unroll
        for (int c = 0; c < LU_NB; c++)
            if (c < nb)
                A[(k0 + tid) * n + k0 + c] = a[c];
}

// One thread per column outside the panel (column index n stands for the right-hand side): row exchanges of the
// panel, then -- right of the panel and for b -- the forward substitution with the panel's unit lower triangle.
// The column's entries of the block row live in shared memory while this happens (one column of a [32][threads] tile
// per thread) and the triangle is staged once per block: the 32 exchanges and 496 updates of a column touch global
// memory only for its 32 entries and for pivot rows below the block row.  (Keeping them in global memory cost a
// dependent L2 round trip per update: 2 ms of the 2.4 ms a 512 x 512 solve took.)
constexpr int TRSM_THREADS = 128;
__global__ void __launch_bounds__(TRSM_THREADS)
    lu_swap_trsm_kernel(double *__restrict__ A, double *__restrict__ x, int64_t n, int64_t k0, int nb,
                        const int *__restrict__ piv) {
    __shared__ double V[LU_NB][TRSM_THREADS + 1];
    __shared__ double L[LU_NB][LU_NB + 1];
    __shared__ int P[LU_NB];
    const int t = threadIdx.x;
    for (int e = t; e < nb * nb; e += TRSM_THREADS)
        L[e / nb][e % nb] = A[(k0 + e / nb) * n + k0 + e % nb];
    if (t < nb)
        P[t] = piv[k0 + t];
    __syncthreads();
    const int64_t c = (int64_t)blockIdx.x * TRSM_THREADS + t;
    if (c > n || (c >= k0 && c < k0 + nb))
        return;
    const bool rhs = (c == n);
    double *col = rhs ? x : A + c;
    const int64_t st = rhs ? 1 : n;
    for (int j = 0; j < nb; j++)
        V[j][t] = col[(k0 + j) * st];
    for (int j = 0; j < nb; j++) {
        const int64_t p = P[j];
        if (p > k0 + j && p < n) { // a pivot row lies below row k0 + j and inside the matrix; anything else is no exchange
            const double v = V[j][t];
            if (p < k0 + nb) {
                V[j][t] = V[p - k0][t];
                V[p - k0][t] = v;
            } else {
                V[j][t] = col[p * st];
                col[p * st] = v;
            }
        }
    }
    if (rhs || c >= k0 + nb)
        for (int j = 0; j < nb; j++) {
            const double v = V[j][t];
            for (int i = j + 1; i < nb; i++)
                V[i][t] = __fma_rn(-L[i][j], v, V[i][t]);
        }
    for (int j = 0; j < nb; j++)
        col[(k0 + j) * st] = V[j][t];
}

// A22 -= L21 U12 (and b2 -= L21 b1 as one more column): 32 x 32 tiles
__global__ void __launch_bounds__(256)
    lu_update_kernel(double *__restrict__ A, double *__restrict__ x, int64_t n, int64_t k0, int nb) {
    __shared__ double L[32][33], U[32][33];
    const int64_t r0 = k0 + nb + (int64_t)blockIdx.y * 32, c0 = k0 + nb + (int64_t)blockIdx.x * 32;
    const int tx = threadIdx.x % 32, ty = threadIdx.x / 32; // 32 x 8
    for (int i = ty; i < 32; i += 8) {
        const int64_t r = r0 + i;
        L[i][tx] = (r < n && tx < nb) ? A[r * n + k0 + tx] : 0.0;
        const int64_t c = c0 + tx; // column n = right-hand side
        double u = 0.0;
        if (i < nb && c <= n)
            u = (c == n) ? x[k0 + i] : A[(k0 + i) * n + c];
        U[i][tx] = u;
    }
    __syncthreads();
    const int64_t c = c0 + tx;
    if (c > n)
        return;
    for (int i = ty; i < 32; i += 8) {
        const int64_t r = r0 + i;
        if (r >= n)
            continue;
        double acc = (c == n) ? x[r] : A[r * n + c];
        for (int p = 0; p < nb; p++)
            acc = __fma_rn(-L[i][p], U[p][tx], acc);
        if (c == n)
            x[r] = acc;
        else
            A[r * n + c] = acc;
    }
}

// Back substitution in blocks of 32 unknowns: warp 0 solves the 32 x 32 triangle on the diagonal (its tile sits in
// shared memory, the unknowns in registers, one shuffle per unknown), then all threads subtract the block's
// contribution from the rows above, each reading 32 consecutive entries of its row.  Every unknown sees the same
// operations in the same order as in the column-by-column loop (x_k /= U_kk; x_i -= U_ik x_k for k descending), so the
// result has the same bits; what changes is that the loop no longer pays two block-wide barriers and a strided pass
// through L2 per unknown.
__global__ void __launch_bounds__(LU_THREADS)
    lu_backsolve_kernel(const double *__restrict__ A, double *__restrict__ x, int64_t n) {
    extern __shared__ double xs[];
    __shared__ double T[32][33];
    const int tid = threadIdx.x, nt = blockDim.x, lane = tid % 32;
    for (int64_t i = tid; i < n; i += nt)
        xs[i] = x[i];
    for (int64_t k1 = n; k1 > 0; k1 -= 32) {
        const int64_t k0 = k1 >= 32 ? k1 - 32 : 0;
        const int w = (int)(k1 - k0);
        for (int e = tid; e < w * w; e += nt)
            T[e / w][e % w] = A[(k0 + e / w) * n + k0 + e % w];
        __syncthreads();
        if (tid < 32) {
            double xi = lane < w ? xs[k0 + lane] : 0.0;
            for (int j = w - 1; j >= 0; j--) {
                const double xj = __ddiv_rn(__shfl_sync(0xffffffffu, xi, j), T[j][j]);
                if (lane == j)
                    xi = xj;
                else if (lane < j)
                    xi = __fma_rn(-T[lane][j], xj, xi);
            }
            if (lane < w)
                xs[k0 + lane] = xi;
        }
        __syncthreads();
        for (int64_t i = tid; i < k0; i += nt) {
            double acc = xs[i];
            const double *row = A + i * n + k0;
            for (int c = w - 1; c >= 0; c--)
                acc = __fma_rn(-row[c], xs[k0 + c], acc);
            xs[i] = acc;
        }
        __syncthreads();
    }
    for (int64_t i = tid; i < n; i += nt)
        x[i] = xs[i];
}

} // namespace db2

using namespace db2;

extern "C" size_t db2k_solve_scratch_bytes(int64_t n) { return (size_t)(n > 0 ? n : 1) * sizeof(int) + 64; }

extern "C" int db2k_solve(int dtype, void *a_work, int64_t n, void *x_inout, int32_t *dev_status, void *scratch,
                          size_t scratch_bytes, void *stream) {
    DB2_CHECK(dtype == DB2_F64, DB2_EUNSUPPORTED, "solve: only double is implemented on the device");
    DB2_CHECK(a_work && x_inout && dev_status, DB2_EINVAL, "null argument");
    DB2_CHECK(scratch && scratch_bytes >= db2k_solve_scratch_bytes(n), DB2_EINVAL, "solve scratch too small");
    if (n == 0)
        return DB2_OK;
    DB2_CHECK(n <= 12800, DB2_EUNSUPPORTED, "solve: systems larger than 12800 unknowns are not supported");
    cudaStream_t st = as_stream(stream);
    double *A = static_cast<double *>(a_work), *x = static_cast<double *>(x_inout);
    int *piv = static_cast<int *>(scratch);
    DB2_CUDA(cudaMemsetAsync(dev_status, 0, sizeof(int32_t), st));
    // widest panel whose rows fit 200 KB of shared memory
    int nb = 32;
    while (nb > 1 && (size_t)n * (nb + 1) * 8 > 200 * 1024)
        nb /= 2;
    static PerDeviceOnce attr;
    if (attr.need()) {
        DB2_CUDA(cudaFuncSetAttribute(lu_panel_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        DB2_CUDA(cudaFuncSetAttribute(lu_backsolve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr.mark();
    }
    for (int64_t k0 = 0; k0 < n; k0 += nb) {
        const int w = (int)((n - k0 < nb) ? (n - k0) : nb);
        const int64_t m = n - k0;
        const int threads = m * w >= 4096 ? LU_THREADS : 256;
        if (m <= LU_REG_ROWS && w <= LU_NB) {
            const int rows32 = (int)((m + 31) / 32 * 32);
            lu_panel_reg_kernel<<<1, rows32, 0, st>>>(A, n, k0, w, piv, dev_status);
            DB2_TRY(after_launch("lu_panel_reg_kernel"));
        } else {
            lu_panel_kernel<<<1, threads, (size_t)m * (w + 1) * 8, st>>>(A, n, k0, w, piv, dev_status);
            DB2_TRY(after_launch("lu_panel_kernel"));
        }
        lu_swap_trsm_kernel<<<(unsigned)((n + 1 + TRSM_THREADS - 1) / TRSM_THREADS), TRSM_THREADS, 0, st>>>(A, x, n, k0, w,
                                                                                                        piv);
        DB2_TRY(after_launch("lu_swap_trsm_kernel"));
        const int64_t rest = n - k0 - w;
        if (rest > 0) {
            dim3 grid((unsigned)((rest + 1 + 31) / 32), (unsigned)((rest + 31) / 32));
            lu_update_kernel<<<grid, 256, 0, st>>>(A, x, n, k0, w);
            DB2_TRY(after_launch("lu_update_kernel"));
        }
    }
    lu_backsolve_kernel<<<1, n >= 256 ? LU_THREADS : 256, (size_t)n * 8, st>>>(A, x, n);
    return after_launch("lu_backsolve_kernel");
}
