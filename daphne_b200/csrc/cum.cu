// AggCum: cumulative SUM / PROD / MIN / MAX down the rows of every column
// (src/runtime/local/kernels/AggCum.h:48-86: row 0 is copied, row r = f(result row r - 1, argument row r); no CUDA twin).
//
// The scan is blocked over the rows; every block of rows is read ONCE:
//   pass 1  each CTA folds its contiguous range of rows into one value per column           (8 B/elem read)
//   pass 2  one thread per column turns the CTAs' values into exclusive prefixes              (tiny)
//   pass 3  each CTA walks its range again in chunks of TY x 16 rows: a thread loads its 16 rows of one column into
//           registers, folds them, the chunk's TY partial values are scanned through shared memory on top of the
//           running carry, and the thread writes its 16 results from the registers            (8 B read + 8 B written)
// Threads of a warp lie along the columns (coalesced rows) for matrices of 32 and more columns; narrower matrices put
// several row groups into a warp: contiguous ones of a power-of-two width go through shared memory (see STAGE), the
// others rely on L1 (every line is used completely by the 16 loads of a chunk).
// Folding is f(running, x) started from the operation's identity: -0.0 for SUM (so that the first row is a copy
// even of -0.0), 1 for PROD, +-inf / the integer limits for MIN / MAX.  MIN / MAX follow the reference's comparisons
// (std::min / std::max: a NaN argument never replaces the running value, a NaN in row 0 stays for the whole column).
// Floating-point sums and products are blocked, i.e. rounded in a different order than the reference's sequential
// loop; MIN, MAX and the integer types are exact.
#include "runtime.h"

#include <limits>

namespace db2 {

constexpr int CUM_THREADS = 256, CUM_LS = 16;
enum { CUM_SUM = 0, CUM_PROD = 1, CUM_MIN = 2, CUM_MAX = 3 };

template <typename VT, int KIND> struct CumOp {
    __device__ static VT identity() {
        if constexpr (KIND == CUM_SUM)
            return std::is_floating_point<VT>::value ? (VT)-0.0 : (VT)0;
        else if constexpr (KIND == CUM_PROD)
            return (VT)1;
        else if constexpr (std::is_floating_point<VT>::value)
            return KIND == CUM_MIN ? (VT)INFINITY : (VT)-INFINITY;
        else
            return KIND == CUM_MIN ? std::numeric_limits<VT>::max() : std::numeric_limits<VT>::lowest();
    }
    __device__ static VT nan() {
        if constexpr (std::is_floating_point<VT>::value)
            return (VT)NAN;
        else
            return (VT)0; // never used: only floating-point columns can start with a NaN
    }
    __device__ static VT apply(VT run, VT x) {
        if constexpr (KIND == CUM_SUM) {
            if constexpr (std::is_same<VT, double>::value)
                return __dadd_rn(run, x);
            else if constexpr (std::is_same<VT, float>::value)
                return __fadd_rn(run, x);
            else
                return run + x;
        } else if constexpr (KIND == CUM_PROD) {
            if constexpr (std::is_same<VT, double>::value)
                return __dmul_rn(run, x);
            else if constexpr (std::is_same<VT, float>::value)
                return __fmul_rn(run, x);
            else
                return run * x;
        } else if constexpr (KIND == CUM_MIN)
            return (x < run) ? x : run;
        else
            return (run < x) ? x : run;
    }
};

// WRITE = false: part[b][c] = fold of CTA b's rows.  WRITE = true: results, starting from the prefixes in part.
// STAGE: the matrix is contiguous and its width is the power of two tx_n < 32.  A chunk (CUM_THREADS * CUM_LS
// consecutive elements) then goes through shared memory, so that global loads and stores are consecutive per lane
// while every thread still owns CUM_LS consecutive rows of its column (one padding slot per thread's run keeps the
// strided shared accesses conflict free).
template <typename VT, int KIND, bool WRITE, bool STAGE>
__global__ void __launch_bounds__(CUM_THREADS)
    agg_cum_kernel(const VT *__restrict__ arg, int64_t rows, int64_t cols, int64_t ld, int64_t rows_per_cta, int tx_n,
                   VT *__restrict__ part, VT *__restrict__ res, int64_t res_ld) {
    using Op = CumOp<VT, KIND>;
    __shared__ VT agg[CUM_THREADS];
    __shared__ VT carry[32];
    __shared__ VT stage[STAGE ? CUM_THREADS * CUM_LS + CUM_THREADS : 1];
    auto padded = [&](int e) { return e + e / (CUM_LS * tx_n); };
    const int ty_n = CUM_THREADS / tx_n, tx = threadIdx.x % tx_n, ty = threadIdx.x / tx_n;
    const int64_t r_begin = (int64_t)blockIdx.x * rows_per_cta;
    const int64_t r_end = r_begin + rows_per_cta < rows ? r_begin + rows_per_cta : rows;
    for (int64_t c0 = 0; c0 < cols; c0 += tx_n) {
        const int64_t c = c0 + tx;
        const bool col_ok = c < cols;
        __syncthreads(); // the previous column group is done with carry[]
        if (ty == 0)
            carry[tx] = (WRITE && col_ok) ? part[(int64_t)blockIdx.x * cols + c] : Op::identity();
        bool poison = false; // MIN / MAX of a column whose first value is a NaN
        if constexpr (WRITE && std::is_floating_point<VT>::value && (KIND == CUM_MIN || KIND == CUM_MAX)) {
            if (col_ok) {
                const VT first = arg[c];
                poison = first != first;
            }
        }
        for (int64_t r0 = r_begin; r0 < r_end; r0 += (int64_t)ty_n * CUM_LS) {
            const int64_t my = r0 + (int64_t)ty * CUM_LS;
            VT x[CUM_LS];
            if constexpr (STAGE) {
                const VT *base = arg + r0 * ld; // ld == cols == tx_n: the chunk is one run of elements
                const int64_t left = (r_end - r0) * tx_n;
#pragma unroll
                for (int i = 0; i < CUM_LS; i++) {
                    const int e = i * CUM_THREADS + threadIdx.x;
                    stage[padded(e)] = e < left ? base[e] : Op::identity();
                }
                __syncthreads();
#pragma unroll
                for (int i = 0; i < CUM_LS; i++)
                    x[i] = stage[padded((ty * CUM_LS + i) * tx_n + tx)];
            } else {
#pragma unroll
                for (int i = 0; i < CUM_LS; i++)
                    x[i] = (col_ok && my + i < r_end) ? arg[(my + i) * ld + c] : Op::identity();
            }
            VT local = Op::identity();
#pragma unroll
            for (int i = 0; i < CUM_LS; i++)
                local = Op::apply(local, x[i]);
            agg[ty * tx_n + tx] = local;
            __syncthreads();
            VT pre = carry[tx];
            for (int j = 0; j < ty; j++)
                pre = Op::apply(pre, agg[j * tx_n + tx]);
            if constexpr (WRITE && STAGE) {
                VT run = pre;
#pragma unroll
                for (int i = 0; i < CUM_LS; i++) {
                    run = Op::apply(run, x[i]);
                    stage[padded((ty * CUM_LS + i) * tx_n + tx)] = poison ? Op::nan() : run;
                }
                __syncthreads();
                VT *out = res + r0 * res_ld;
                const int64_t left = (r_end - r0) * tx_n;
#pragma unroll
                for (int i = 0; i < CUM_LS; i++) {
                    const int e = i * CUM_THREADS + threadIdx.x;
                    if (e < left)
                        out[e] = stage[padded(e)];
                }
            } else if constexpr (WRITE) {
                VT run = pre;
#pragma unroll
                for (int i = 0; i < CUM_LS; i++) {
                    run = Op::apply(run, x[i]);
                    if (col_ok && my + i < r_end)
                        res[(my + i) * res_ld + c] = poison ? Op::nan() : run;
                }
            }
            __syncthreads(); // everybody has read carry[], agg[] and the staged chunk
            if (ty == ty_n - 1)
                carry[tx] = Op::apply(pre, local);
            // the next turn's barrier (after agg[] is written) orders this store before its readers
        }
        __syncthreads();
        if constexpr (!WRITE) {
            if (ty == 0 && col_ok)
                part[(int64_t)blockIdx.x * cols + c] = carry[tx];
        }
    }
}

// part[b][c] (fold of CTA b) -> exclusive prefix over b, in place.  One block per column: thread t owns a run of
// consecutive b (loaded at once), the runs' folds are scanned through shared memory, then every thread writes the
// prefixes of its run.  (A single thread walking all b would pay one global round trip per step.)
template <typename VT, int KIND>
__global__ void __launch_bounds__(256) agg_cum_prefix_kernel(VT *__restrict__ part, int nb, int64_t cols) {
    using Op = CumOp<VT, KIND>;
    constexpr int MAXS = 8; // nb <= 8 * 148 CTAs of the scan kernels: at most 5 per thread; more are walked in turns
    __shared__ VT fold[256];
    __shared__ VT carry;
    const int64_t c = blockIdx.x;
    const int t = threadIdx.x;
    if (t == 0)
        carry = Op::identity();
    for (int b0 = 0; b0 < nb; b0 += 256 * MAXS) {
        const int left = nb - b0 < 256 * MAXS ? nb - b0 : 256 * MAXS;
        const int per = (left + 255) / 256;
        VT v[MAXS];
        VT local = Op::identity();
#pragma unroll
        for (int i = 0; i < MAXS; i++) {
            const int b = b0 + t * per + i;
            v[i] = (i < per && t * per + i < left) ? part[(int64_t)b * cols + c] : Op::identity();
        }
#pragma unroll
        for (int i = 0; i < MAXS; i++)
            local = Op::apply(local, v[i]);
        fold[t] = local;
        __syncthreads();
        VT run = carry;
        for (int j = 0; j < t; j++)
            run = Op::apply(run, fold[j]);
#pragma unroll
        for (int i = 0; i < MAXS; i++) {
            const int b = b0 + t * per + i;
            if (i < per && t * per + i < left)
                part[(int64_t)b * cols + c] = run;
            run = Op::apply(run, v[i]);
        }
        __syncthreads();
        if (t == 255)
            carry = run;
        __syncthreads();
    }
}

struct CumPlan {
    int tx_n, nb;
    int64_t rows_per_cta;
};
static CumPlan cum_plan(int64_t rows, int64_t cols) {
    CumPlan p;
    p.tx_n = (int)next_pow2(cols < 32 ? cols : 32);
    if (p.tx_n < 1)
        p.tx_n = 1;
    const int64_t chunk = (int64_t)(CUM_THREADS / p.tx_n) * CUM_LS; // rows per CTA turn
    int64_t nb = (rows + chunk - 1) / chunk;
    const int64_t cap = (int64_t)sm_count() * 8;
    if (nb > cap)
        nb = cap;
    if (nb < 1)
        nb = 1;
    p.rows_per_cta = ((rows + nb - 1) / nb + chunk - 1) / chunk * chunk;
    p.nb = (int)((rows + p.rows_per_cta - 1) / p.rows_per_cta);
    if (p.nb < 1)
        p.nb = 1;
    return p;
}

template <typename VT, int KIND>
static int agg_cum_impl(const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, int64_t res_ld, VT *part,
                        cudaStream_t st) {
    const CumPlan p = cum_plan(rows, cols);
    const bool stage = p.tx_n < 32 && cols == p.tx_n && ld == cols && res_ld == cols;
    if (stage)
        agg_cum_kernel<VT, KIND, false, true><<<p.nb, CUM_THREADS, 0, st>>>(arg, rows, cols, ld, p.rows_per_cta, p.tx_n,
                                                                             part, nullptr, 0);
    else
        agg_cum_kernel<VT, KIND, false, false><<<p.nb, CUM_THREADS, 0, st>>>(arg, rows, cols, ld, p.rows_per_cta,
                                                                              p.tx_n, part, nullptr, 0);
    DB2_TRY(after_launch("agg_cum_kernel"));
    agg_cum_prefix_kernel<VT, KIND><<<(unsigned)cols, 256, 0, st>>>(part, p.nb, cols);
    DB2_TRY(after_launch("agg_cum_prefix_kernel"));
    if (stage)
        agg_cum_kernel<VT, KIND, true, true><<<p.nb, CUM_THREADS, 0, st>>>(arg, rows, cols, ld, p.rows_per_cta, p.tx_n,
                                                                            part, res, res_ld);
    else
        agg_cum_kernel<VT, KIND, true, false><<<p.nb, CUM_THREADS, 0, st>>>(arg, rows, cols, ld, p.rows_per_cta, p.tx_n,
                                                                             part, res, res_ld);
    return after_launch("agg_cum_kernel");
}

static void count(db2_context *ctx, uint64_t before) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load(std::memory_order_relaxed) - before;
}

} // namespace db2

using namespace db2;

extern "C" {

size_t db2k_agg_cum_scratch_bytes(int64_t rows, int64_t cols) {
    if (rows <= 0 || cols <= 0)
        return 0;
    return (size_t)cum_plan(rows, cols).nb * (size_t)cols * 8;
}

int db2k_agg_cum(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res, int64_t res_ld,
                 void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(op >= CUM_SUM && op <= CUM_MAX, DB2_EINVAL,
              "the aggregation function used in aggCum must be a pure binary reduction");
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative shape");
    if (rows == 0 || cols == 0)
        return DB2_OK;
    DB2_CHECK(arg && res && scratch && scratch_bytes >= db2k_agg_cum_scratch_bytes(rows, cols), DB2_EINVAL,
              "aggCum: null operand or scratch smaller than db2k_agg_cum_scratch_bytes");
#define DB2_CUM(KIND)                                                                                                  \
    DB2_DISPATCH_DTYPE(dtype, VT,                                                                                      \
                       return (agg_cum_impl<VT, KIND>(static_cast<const VT *>(arg), rows, cols, ld,                    \
                                                      static_cast<VT *>(res), res_ld, static_cast<VT *>(scratch),     \
                                                      as_stream(stream))))
    switch (op) {
    case CUM_SUM: DB2_CUM(CUM_SUM); break;
    case CUM_PROD: DB2_CUM(CUM_PROD); break;
    case CUM_MIN: DB2_CUM(CUM_MIN); break;
    default: DB2_CUM(CUM_MAX); break;
    }
#undef DB2_CUM
    return DB2_OK;
}

int db2_aggCum(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    DB2_CHECK(op >= CUM_SUM && op <= CUM_MAX, DB2_EINVAL,
              "the aggregation function used in aggCum must be a pure binary reduction");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(arg));
    DB2_TRY(prepare_result(ctx, res, arg->dtype, arg->rows, arg->cols));
    if (arg->rows > 0 && arg->cols > 0) {
        void *scratch = nullptr;
        const size_t sb = db2k_agg_cum_scratch_bytes(arg->rows, arg->cols);
        DB2_TRY(ctx_scratch(ctx, sb, &scratch));
        DB2_TRY(db2k_agg_cum(arg->dtype, op, arg->dev_ptr(), arg->rows, arg->cols, arg->dev_ld, (*res)->dev_ptr(),
                             (*res)->dev_ld, scratch, sb, ctx->stream));
    }
    count(ctx, before);
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
