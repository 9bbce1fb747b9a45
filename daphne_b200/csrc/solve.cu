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
#include "fused_step.cuh"

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
// Per column: block-wide argmax of |a[j]|, exchange of the pivot row and row j through shared memory, then every
// thread below the diagonal scales its a[j] and updates its remaining entries from the broadcast pivot row -- one
// barrier per column, no shared-memory traffic for the updates.
//
// What bounds the kernel is the chain of dependent operations per column, so that chain is kept short:
//   * |a| is compared as an integer (the bit pattern of a non-negative double orders like its value), which lets the
//     argmax run on the warp-reduce instructions: three of them per level (high word, low word, lowest row among the
//     equals) instead of five rounds of 64-bit shuffles and FP64 compares;
//   * the division by the pivot is a / p exactly (correctly rounded), but computed from the pivot's reciprocal, which
//     every candidate row prepares for its own entry BEFORE the search -- off the critical path -- and the winner
//     publishes with its row; after the barrier a multiplication and two fused multiply-adds remain (fast_div).
constexpr int LU_NB = 32, LU_REG_ROWS = 512;

// order of |a| as an integer: 0 for "no candidate" and for a NaN (which the scan's comparison never prefers),
// 1 + bits(|a|) for a candidate
__device__ __forceinline__ unsigned long long pivot_key(double a, bool cand) {
    const unsigned long long bits = (unsigned long long)__double_as_longlong(fabs(a));
    return (cand && bits <= 0x7ff0000000000000ull) ? bits + 1ull : 0ull;
}
// the largest key of the warp and the lowest row that has it
__device__ __forceinline__ void warp_first_largest(unsigned long long key, int row, unsigned long long &kmax, int &rmin) {
    const unsigned hi = (unsigned)(key >> 32);
    const unsigned mh = __reduce_max_sync(0xffffffffu, hi);
    const unsigned lo = hi == mh ? (unsigned)key : 0u;
    const unsigned ml = __reduce_max_sync(0xffffffffu, lo);
    const bool top = hi == mh && lo == ml;
    rmin = (int)__reduce_min_sync(0xffffffffu, top ? (unsigned)row : 0x7fffffffu);
    kmax = ((unsigned long long)mh << 32) | ml;
}

// Layout of the dynamic shared memory of lu_panel_reg_kernel (doubles): the multipliers every row has collected,
// [LU_REG_ROWS][LU_NB + 1]; the pivot rows, [LU_NB][LU_NB]; the candidates' rows, [2][LU_REG_ROWS / 32][LU_NB]
constexpr int LU_PANEL_SMEM = (LU_REG_ROWS * (LU_NB + 1) + LU_NB * LU_NB + 2 * (LU_REG_ROWS / 32) * LU_NB) * 8;

__global__ void __launch_bounds__(LU_REG_ROWS)
    lu_panel_reg_kernel(double *__restrict__ A, int64_t n, int64_t k0, int nb, int *__restrict__ piv,
                        int32_t *__restrict__ status) {
    // The loop over the columns is a REAL loop: the part of the row that is still being eliminated lives in
    // a[0 .. 31 - j] -- the update of column j writes entry c to a[c - 1] -- so the code of every column is the same
    // and stays in the instruction cache.  (Unrolled over the columns, with fixed register positions, the kernel was
    // 32 different pieces of code that each ran once: it waited for instruction fetches more than for anything
    // else.)  Rows are not exchanged either: a thread keeps its row and only the row's POSITION changes hands.  A row
    // that becomes a pivot row leaves its remaining entries in `urow`, every other row notes its multiplier in
    // `lmul`; the rows are written to their final positions at the end.
    //
    // ONE barrier per column: before it every warp publishes its best pivot candidate TOGETHER WITH that candidate's
    // row; after it every thread folds the warps' candidates to the same pivot.  The buffers alternate with the column
    // parity, so the writes of column j + 1 cannot overtake the reads of column j - 1.
    extern __shared__ double lu_sm[];
    double(*lmul)[LU_NB + 1] = reinterpret_cast<double(*)[LU_NB + 1]>(lu_sm);
    double(*urow)[LU_NB] = reinterpret_cast<double(*)[LU_NB]>(lu_sm + LU_REG_ROWS * (LU_NB + 1));
    double(*cand_row)[LU_REG_ROWS / 32][LU_NB] =
        reinterpret_cast<double(*)[LU_REG_ROWS / 32][LU_NB]>(lu_sm + LU_REG_ROWS * (LU_NB + 1) + LU_NB * LU_NB);
    __shared__ double cand_rcp[2][LU_REG_ROWS / 32]; // reciprocal of the candidate's entry (0: none usable)
    __shared__ unsigned long long s_key[2][LU_REG_ROWS / 32];
    __shared__ int s_pos[2][LU_REG_ROWS / 32];
    const int tid = threadIdx.x, lane = tid % 32, warp = tid / 32, nwarps = blockDim.x / 32;
    const int m = (int)(n - k0);
    double a[LU_NB];
#pragma unroll
    for (int c = 0; c < LU_NB; c++)
        a[c] = (tid < m && c < nb) ? A[(k0 + tid) * n + k0 + c] : 0.0;
    int pos = tid;      // the position (row of the panel) this thread's row holds at the moment
    int pivoted_at = -1; // the column at which it became the pivot row
#pragma unroll 1
    for (int j = 0; j < nb; j++) {
        const int par = j & 1;
        // first largest |a| of column j among the rows at positions j .. m-1 (idamax)
        const bool cand = pivoted_at < 0 && tid < m;
        const double rcp = cand ? div_helper(a[0]) : 0.0;
        unsigned long long key;
        int bp;
        warp_first_largest(pivot_key(a[0], cand), cand ? pos : 0x7fffffff, key, bp);
        if (cand && pos == bp) { // this warp's candidate publishes its row
#pragma unroll
            for (int c = 0; c < LU_NB; c++)
                cand_row[par][warp][c] = a[c];
            cand_rcp[par][warp] = rcp;
        }
        if (lane == 0) {
            s_key[par][warp] = key;
            s_pos[par][warp] = bp;
        }
        __syncthreads();
        const int wpos = lane < nwarps ? s_pos[par][lane] : 0x7fffffff;
        warp_first_largest(lane < nwarps ? s_key[par][lane] : 0ull, wpos, key, bp);
        const int p = bp; // the same in every thread; always a position in [j, m): the row at position j is a candidate
        const int pw = __ffs(__ballot_sync(0xffffffffu, wpos == p)) - 1; // the warp whose candidate it is
        const double *prow = cand_row[par][pw];
        if (tid == 0) {
            piv[k0 + j] = (int)k0 + p;
            if (key <= 1ull && *status == 0)
                *status = (int32_t)(k0 + j + 1); // exactly singular (or NaN) pivot
        }
        if (tid < LU_NB)
            urow[j][tid] = prow[tid]; // entries j .. of the pivot row (entry j + c at index c)
        if (cand) {
            if (pos == p) { // this row is the pivot row: it moves to position j and is finished
                pos = j;
                pivoted_at = j;
            } else {
                if (pos == j)
                    pos = p; // the row that sat at position j takes the pivot row's place
                const double l = fast_div(a[0], prow[0], cand_rcp[par][pw]);
                lmul[tid][j] = l;
#pragma unroll
                for (int c = 1; c < LU_NB; c++)
                    a[c - 1] = __fma_rn(-l, prow[c], a[c]);
                a[LU_NB - 1] = 0.0;
            }
        }
    }
    __syncthreads(); // urow is complete
    if (tid < m) {
        double *dst = A + (k0 + pos) * n + k0;
        const int from_pivot_row = pivoted_at >= 0 ? pivoted_at : nb; // the first column that is not a multiplier
        for (int c = 0; c < from_pivot_row; c++)
            dst[c] = lmul[tid][c];
        for (int c = from_pivot_row; c < nb; c++)
            dst[c] = urow[pivoted_at][c - pivoted_at];
    }
}

// One thread per column right of the panel (column index n stands for the right-hand side): row exchanges of the
// panel, then the forward substitution with the panel's unit lower triangle.  (Columns left of the panel hold
// multipliers that nothing reads again -- the right-hand side is carried along as a column -- so they are left alone.)
//
// The 32 exchanges of a panel are one permutation.  Warp 0 composes it once per block -- lane j follows which original
// row ends up in row k0 + j of the block row, and the lanes also keep the list of rows below the block row that
// receive a row -- so every thread can fetch all its sources with INDEPENDENT loads and then write the displaced rows,
// instead of 32 dependent read-modify-write round trips through L2.  The column's 32 entries of the block row stay
// in registers through the substitution; the triangle is staged in shared memory once per block.
constexpr int TRSM_THREADS = 128;
__global__ void __launch_bounds__(TRSM_THREADS)
    lu_swap_trsm_kernel(double *__restrict__ A, double *__restrict__ x, int64_t n, int64_t k0, int nb,
                        const int *__restrict__ piv) {
    __shared__ double L[2 * LU_NB][LU_NB + 1]; // rows nb .. stay zero: the substitution loop needs no bounds
    __shared__ int src_blk[LU_NB];               // original row whose entry ends up in row k0 + j
    __shared__ int out_row[LU_NB], out_src[LU_NB]; // rows below the block row that receive original row out_src
    __shared__ int out_cnt;
    const int t = threadIdx.x;
    if (t < 32) {
        // lane j: cur = original row now in position k0 + j; lane e < cnt: (orow, osrc) of the e-th outside row
        int cur = (int)k0 + t, orow = -1, osrc = -1, cnt = 0;
        for (int j = 0; j < nb; j++) {
            const int p = piv[k0 + j];
            if (p > k0 + j && p < n) { // a pivot row below row k0 + j and inside the matrix; anything else: no exchange
                const int cj = __shfl_sync(0xffffffffu, cur, j);
                if (p < k0 + nb) {
                    const int cp = __shfl_sync(0xffffffffu, cur, p - (int)k0);
                    if (t == j)
                        cur = cp;
                    else if (t == p - (int)k0)
                        cur = cj;
                } else {
                    const unsigned hit = __ballot_sync(0xffffffffu, t < cnt && orow == p);
                    int e = hit ? __ffs(hit) - 1 : cnt;
                    const int prev = hit ? __shfl_sync(0xffffffffu, osrc, e) : p; // what row p holds right now
                    if (!hit) {
                        if (t == cnt)
                            orow = p;
                        cnt++;
                    }
                    if (t == e)
                        osrc = cj;
                    if (t == j)
                        cur = prev;
                }
            }
        }
        src_blk[t] = cur;
        out_row[t] = orow;
        out_src[t] = osrc;
        if (t == 0)
            out_cnt = cnt;
    }
    for (int e = t; e < 2 * LU_NB * LU_NB; e += TRSM_THREADS) {
        const int i = e / LU_NB, j = e % LU_NB;
        L[i][j] = (i < nb && j < nb) ? A[(k0 + i) * n + k0 + j] : 0.0;
    }
    __syncthreads();
    const int64_t c0 = (int64_t)blockIdx.x * TRSM_THREADS + t;
    const int64_t c = k0 + nb + c0; // columns k0 + nb .. n - 1, then the right-hand side
    if (c > n)
        return;
    const bool rhs = (c == n);
    double *col = rhs ? x : A + c;
    const int64_t st = rhs ? 1 : n;
    const int cnt = out_cnt;
    double v[LU_NB], w[LU_NB];
#pragma unroll
    for (int j = 0; j < LU_NB; j++)
        v[j] = j < nb ? col[(int64_t)src_blk[j] * st] : 0.0;
#pragma unroll
    for (int e = 0; e < LU_NB; e++)
        w[e] = e < cnt ? col[(int64_t)out_src[e] * st] : 0.0;
#pragma unroll
    for (int e = 0; e < LU_NB; e++)
        if (e < cnt)
            col[(int64_t)out_row[e] * st] = w[e];
    // forward substitution as a loop with one body: the entries still to be updated move down one register per
    // column (entry j + i sits in v[i]), so that x_j is always v[0]
#pragma unroll 1
    for (int j = 0; j < nb; j++) {
        const double xj = v[0];
        col[(k0 + j) * st] = xj;
#pragma unroll
        for (int i = 1; i < LU_NB; i++)
            v[i - 1] = __fma_rn(-L[j + i][j], xj, v[i]);
        v[LU_NB - 1] = 0.0;
    }
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
            // x_j / U_jj is the exact quotient, taken from the diagonal's reciprocal (prepared by all lanes at once,
            // ahead of the dependent chain of the 32 unknowns)
            const double dg = lane < w ? T[lane][lane] : 1.0, ry = div_helper(dg);
            for (int j = w - 1; j >= 0; j--) {
                const double xj = fast_div(__shfl_sync(0xffffffffu, xi, j), __shfl_sync(0xffffffffu, dg, j),
                                           __shfl_sync(0xffffffffu, ry, j));
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
            double rv[32]; // the row's 32 entries are fetched together, then used in the order of the column loop
#pragma unroll
            for (int c = 0; c < 32; c++)
                rv[c] = c < w ? row[c] : 0.0;
#pragma unroll
            for (int c = 31; c >= 0; c--)
                if (c < w)
                    acc = __fma_rn(-rv[c], xs[k0 + c], acc);
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
        DB2_CUDA(cudaFuncSetAttribute(lu_panel_reg_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      LU_PANEL_SMEM));
        DB2_CUDA(cudaFuncSetAttribute(lu_backsolve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr.mark();
    }
    for (int64_t k0 = 0; k0 < n; k0 += nb) {
        const int w = (int)((n - k0 < nb) ? (n - k0) : nb);
        const int64_t m = n - k0;
        const int threads = m * w >= 4096 ? LU_THREADS : 256;
        if (m <= LU_REG_ROWS && w <= LU_NB) {
            const int rows32 = (int)((m + 31) / 32 * 32);
            lu_panel_reg_kernel<<<1, rows32, LU_PANEL_SMEM, st>>>(A, n, k0, w, piv, dev_status);
            DB2_TRY(after_launch("lu_panel_reg_kernel"));
        } else {
            lu_panel_kernel<<<1, threads, (size_t)m * (w + 1) * 8, st>>>(A, n, k0, w, piv, dev_status);
            DB2_TRY(after_launch("lu_panel_kernel"));
        }
        const int64_t right = n - k0 - w + 1; // columns right of the panel and the right-hand side
        lu_swap_trsm_kernel<<<(unsigned)((right + TRSM_THREADS - 1) / TRSM_THREADS), TRSM_THREADS, 0, st>>>(A, x, n, k0, w,
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
