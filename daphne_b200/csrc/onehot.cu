// One-hot matrices that are never written out.
//
// K-means builds the assignment matrix  P = ctable(seq(0, n-1), a, 1.0, n, k)  (CTable.h:55-106: one entry per row) only
// to multiply it,  t(P) @ X  (MatMul.cpp:284-288: a dense 50 x 1M by 1M x 64 dgemm in the reference), and to count its
// columns,  sum(P, 1)  (AggCol.h:135-141).  Written out, P is n x k doubles (400 MB for n = 1M, k = 50) that are
// produced once and read twice per iteration.  Here the result of such a ctable call keeps only (a, weight): a matrix
// with db2_matrix::onehot set has no placement until something else needs its values (then the dense rows are
// written by the ordinary ctable kernel).  The two consumers above run directly on the index vector:
//   t(P) @ X   = per-cluster sums of the rows of X: every warp keeps private k x d accumulators in shared memory and
//                adds its rows to them (no atomics, fixed row order), warps and CTAs are summed in a fixed order;
//   sum(P, 1)  = histogram of a (integer counts, exact).
#include "runtime.h"

namespace db2 {

constexpr int SEG_MAX_WARPS = 8;
constexpr size_t SEG_SMEM_LIMIT = 216 * 1024;

// accumulators acc[warp][cluster][column]
__global__ void __launch_bounds__(SEG_MAX_WARPS * 32)
    onehot_segsum_kernel(const int64_t *__restrict__ idx, int64_t idx_ld, const double *__restrict__ X, int64_t ldx,
                         int64_t n, int d, int k, int vec, double *__restrict__ partials) {
    extern __shared__ double acc[];
    const int warps = blockDim.x / 32, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int kd = k * d;
    for (int e = threadIdx.x; e < warps * kd; e += blockDim.x)
        acc[e] = 0.0;
    __syncthreads();
    double *mine = acc + warp * kd;
    // every warp owns a contiguous run of rows and walks it in order, 32 rows per batch: one coalesced load of the 32
    // cluster numbers (the next batch's is issued before this batch is processed), then 16 rows of X in flight
    const int64_t total_warps = (int64_t)gridDim.x * warps, gw = (int64_t)blockIdx.x * warps + warp;
    const int64_t per = (n + total_warps - 1) / total_warps;
    const int64_t lo = gw * per, hi = lo + per < n ? lo + per : n;
    constexpr int U = 16;
    int64_t c_next = (lo + lane < hi) ? idx[(lo + lane) * idx_ld] : -1;
    for (int64_t b0 = lo; b0 < hi; b0 += 32) {
        const int64_t c_mine = c_next;
        c_next = (b0 + 32 + lane < hi) ? idx[(b0 + 32 + lane) * idx_ld] : -1;
#pragma unroll
        for (int h = 0; h < 32; h += U) {
            if (b0 + h >= hi)
                break;
            if (vec && d == 64) {
                // one row = 32 lanes x 16 bytes
                double2 x[U];
                int cu[U];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const long long c = __shfl_sync(0xffffffffu, (long long)c_mine, h + u);
                    cu[u] = (c >= 0 && c < k) ? (int)c : -1;
                    x[u] = cu[u] >= 0 ? __ldcs(reinterpret_cast<const double2 *>(X + (b0 + h + u) * ldx) + lane)
                                      : make_double2(0.0, 0.0);
                }
#pragma unroll
                for (int u = 0; u < U; u++)
                    if (cu[u] >= 0) {
                        double2 *a = reinterpret_cast<double2 *>(mine + cu[u] * d) + lane;
                        double2 t = *a;
                        t.x = __dadd_rn(t.x, x[u].x);
                        t.y = __dadd_rn(t.y, x[u].y);
                        *a = t;
                    }
            } else {
#pragma unroll 1
                for (int u = 0; u < U; u++) {
                    const long long c = __shfl_sync(0xffffffffu, (long long)c_mine, h + u);
                    if (c >= 0 && c < k)
                        for (int j = lane; j < d; j += 32)
                            mine[c * d + j] = __dadd_rn(mine[c * d + j], X[(b0 + h + u) * ldx + j]);
                }
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < kd; e += blockDim.x) {
        double t = acc[e];
        for (int w = 1; w < warps; w++)
            t = __dadd_rn(t, acc[w * kd + e]);
        partials[(int64_t)blockIdx.x * kd + e] = t;
    }
}

// The same sums for d = 64 columns of 16-byte aligned rows (one row = 32 lanes x 16 bytes), written for latency:
//  * 32 rows of X per warp (16 KB) are on their way at any time: a row's registers are refilled with the row 32
//    further on as soon as the row has been added, so the loads are spread evenly over the additions (with two
//    register sets filled in turns -- 8 rows each: 108 us for 1 M rows, 16 rows each: 124 us -- no load is issued
//    while a whole set is being added; this form: 101 us with 16 rows, 96 us with 32).  Eight warps per SM keep
//    128 KB in flight; the block is alone on its SM, so the 158 registers cost nothing;
//  * two rows are added at a time: when their clusters differ the two read-modify-write chains on shared memory are
//    independent and overlap, when they agree the accumulator is read and written once for both.  The order of the
//    additions into any accumulator is the row order, as in the general kernel;
//  * rows without a valid cluster number (and the rows past the end of a warp's range) are added to a spare
//    accumulator row, so nothing in the loop is conditional.
__global__ void __launch_bounds__(SEG_MAX_WARPS * 32)
    onehot_segsum64_kernel(const int64_t *__restrict__ idx, int64_t idx_ld, const double *__restrict__ X, int64_t ldx,
                           int64_t n, int k, double *__restrict__ partials) {
    extern __shared__ __align__(16) double acc[];
    constexpr int D = 64, U = 32;
    const int warps = blockDim.x / 32, warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int slots = (k + 1) * D; // per warp; row k is the spare one
    for (int e = threadIdx.x; e < warps * slots; e += blockDim.x)
        acc[e] = 0.0;
    __syncthreads();
    const unsigned mine_s = (unsigned)__cvta_generic_to_shared(acc + warp * slots) + (unsigned)(lane * 16);
    const int64_t total_warps = (int64_t)gridDim.x * warps, gw = (int64_t)blockIdx.x * warps + warp;
    const int64_t per = ((n + total_warps - 1) / total_warps + 31) / 32 * 32;
    const int64_t lo = gw * per, hi = lo + per < n ? lo + per : n;
    if (lo < hi) {
        const double2 *xl = reinterpret_cast<const double2 *>(X) + lane;
        const int64_t ld2 = ldx / 2;
        // x[u]: the next row of this warp whose number is u modulo U; a row's register pair is refilled with the
        // row U further on as soon as the row has been added
        double2 x[U];
        auto ldrow = [&](int64_t r) { return (r < hi) ? __ldcs(xl + r * ld2) : make_double2(0.0, 0.0); };
        auto lds = [](unsigned a) {
            double2 v;
            asm volatile("ld.shared.v2.f64 {%0, %1}, [%2];\n" : "=d"(v.x), "=d"(v.y) : "r"(a) : "memory");
            return v;
        };
        auto sts = [](unsigned a, double2 v) {
            asm volatile("st.shared.v2.f64 [%0], {%1, %2};\n" ::"r"(a), "d"(v.x), "d"(v.y) : "memory");
        };
#pragma unroll
        for (int u = 0; u < U; u++)
            x[u] = ldrow(lo + u);
        int64_t c_next = (lo + lane < hi) ? idx[(lo + lane) * idx_ld] : -1;
        for (int64_t b0 = lo; b0 < hi; b0 += 32) {
            const int ci = (c_next >= 0 && c_next < k) ? (int)c_next : k;
            c_next = (b0 + 32 + lane < hi) ? idx[(b0 + 32 + lane) * idx_ld] : -1;
#pragma unroll
            for (int h = 0; h < 32; h += U) {
#pragma unroll
                for (int u = 0; u < U; u += 2) {
                    const int c0 = __shfl_sync(0xffffffffu, ci, h + u), c1 = __shfl_sync(0xffffffffu, ci, h + u + 1);
                    const unsigned a0 = mine_s + (unsigned)(c0 * D * 8), a1 = mine_s + (unsigned)(c1 * D * 8);
                    if (c0 != c1) {
                        double2 t0 = lds(a0), t1 = lds(a1);
                        t0.x = __dadd_rn(t0.x, x[u].x);
                        t0.y = __dadd_rn(t0.y, x[u].y);
                        t1.x = __dadd_rn(t1.x, x[u + 1].x);
                        t1.y = __dadd_rn(t1.y, x[u + 1].y);
                        sts(a0, t0);
                        sts(a1, t1);
                    } else {
                        double2 t0 = lds(a0);
                        t0.x = __dadd_rn(__dadd_rn(t0.x, x[u].x), x[u + 1].x);
                        t0.y = __dadd_rn(__dadd_rn(t0.y, x[u].y), x[u + 1].y);
                        sts(a0, t0);
                    }
                    x[u] = ldrow(b0 + h + u + U);
                    x[u + 1] = ldrow(b0 + h + u + 1 + U);
                }
            }
        }
    }
    __syncthreads();
    const int kd = k * D;
    for (int e = threadIdx.x; e < kd; e += blockDim.x) {
        double t = acc[e];
        for (int w = 1; w < warps; w++)
            t = __dadd_rn(t, acc[w * slots + e]);
        partials[(int64_t)blockIdx.x * kd + e] = t;
    }
}

// out = sum over the CTAs' partial sums in a fixed order: 32 elements per CTA, 8 thread groups each adding every 8th
// partial, then the 8 group sums in order
__global__ void __launch_bounds__(256)
    onehot_segsum_final_kernel(const double *__restrict__ partials, int parts, int kd, int d, double *__restrict__ out,
                               int64_t ldo) {
    __shared__ double sh[8][32];
    const int e = blockIdx.x * 32 + threadIdx.x % 32, grp = threadIdx.x / 32;
    double t = 0.0;
    if (e < kd)
        for (int p = grp; p < parts; p += 8)
            t = __dadd_rn(t, partials[(int64_t)p * kd + e]);
    sh[grp][threadIdx.x % 32] = t;
    __syncthreads();
    if (grp == 0 && e < kd) {
        for (int q = 1; q < 8; q++)
            t = __dadd_rn(t, sh[q][threadIdx.x]);
        out[(int64_t)(e / d) * ldo + e % d] = t;
    }
}

__global__ void onehot_hist_kernel(const int64_t *__restrict__ idx, int64_t idx_ld, int64_t n, int k,
                                   unsigned long long *__restrict__ counts) {
    extern __shared__ unsigned int h[];
    for (int e = threadIdx.x; e < k; e += blockDim.x)
        h[e] = 0u;
    __syncthreads();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t c = idx[i * idx_ld];
        if (c >= 0 && c < k)
            atomicAdd(h + c, 1u);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < k; e += blockDim.x)
        if (h[e])
            atomicAdd(counts + e, (unsigned long long)h[e]);
}
__global__ void onehot_hist_final_kernel(const unsigned long long *__restrict__ counts, int k, double *__restrict__ out) {
    for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < k; e += gridDim.x * blockDim.x)
        out[e] = (double)counts[e];
}

static void count(db2_context *ctx, uint64_t before) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load(std::memory_order_relaxed) - before;
}

// writes the dense rows of a one-hot matrix (someone needs its values after all)
int onehot_force(db2_matrix *m) {
    db2_context *ctx = m->ctx;
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    std::shared_ptr<const OneHot> oh = m->onehot;
    m->dev = make_devbuf(ctx, (size_t)m->rows * m->cols * 8);
    m->dev_off = 0;
    m->dev_ld = m->cols;
    DB2_TRY(db2k_ctable(nullptr, 1, oh->idx.ptr(8), oh->idx.ld, m->rows, oh->weight, m->dev->ptr, m->rows, m->cols,
                        m->dev_ld, 1, ctx->stream));
    m->dev_valid = true;
    m->onehot.reset();
    count(ctx, before);
    return DB2_OK;
}

// t(P) @ X for a one-hot P (weight 1): *handled stays false when the shapes do not fit the kernel
int onehot_try_matmul(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, int transa, int transb,
                      bool *handled) {
    *handled = false;
    if (!lhs->onehot || lhs->dev_valid || !transa || transb || rhs->dtype != DB2_F64 || lhs->onehot->weight != 1.0)
        return DB2_OK;
    const int64_t n = lhs->rows, k = lhs->cols, d = rhs->cols;
    if (rhs->rows != n || k < 1 || d < 1 || (size_t)k * d * 8 > SEG_SMEM_LIMIT || n < 1)
        return DB2_OK;
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(rhs));
    const double *X = static_cast<const double *>(rhs->dev_ptr());
    const int vec = aligned16(X) && rhs->dev_ld % 2 == 0;
    const bool k64 = vec && d == 64 && (size_t)(k + 1) * d * 8 <= SEG_SMEM_LIMIT; // the latency-tuned kernel
    const int64_t acc_rows = k64 ? k + 1 : k;
    int warps = SEG_MAX_WARPS;
    while ((size_t)warps * acc_rows * d * 8 > SEG_SMEM_LIMIT)
        warps /= 2;
    DB2_TRY(prepare_result(ctx, res, DB2_F64, k, d));
    const int grid = sm_count();
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, (size_t)grid * k * d * 8, &scratch));
    const size_t smem = (size_t)warps * acc_rows * d * 8;
    static PerDeviceOnce attr;
    if (attr.need()) {
        DB2_CUDA(cudaFuncSetAttribute(onehot_segsum_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)SEG_SMEM_LIMIT));
        DB2_CUDA(cudaFuncSetAttribute(onehot_segsum64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)SEG_SMEM_LIMIT));
        attr.mark();
    }
    std::shared_ptr<const OneHot> oh = lhs->onehot;
    if (k64)
        onehot_segsum64_kernel<<<grid, warps * 32, smem, ctx->stream>>>(static_cast<const int64_t *>(oh->idx.ptr(8)),
                                                                        oh->idx.ld, X, rhs->dev_ld, n, (int)k,
                                                                        static_cast<double *>(scratch));
    else
        onehot_segsum_kernel<<<grid, warps * 32, smem, ctx->stream>>>(static_cast<const int64_t *>(oh->idx.ptr(8)),
                                                                      oh->idx.ld, X, rhs->dev_ld, n, (int)d, (int)k, vec,
                                                                      static_cast<double *>(scratch));
    DB2_TRY(after_launch("onehot_segsum_kernel"));
    const int kd = (int)(k * d);
    onehot_segsum_final_kernel<<<(kd + 31) / 32, 256, 0, ctx->stream>>>(
        static_cast<const double *>(scratch), grid, kd, (int)d, static_cast<double *>((*res)->dev_ptr()),
        (*res)->dev_ld);
    DB2_TRY(after_launch("onehot_segsum_final_kernel"));
    count(ctx, before);
    *handled = true;
    return DB2_OK;
}

// sum(P, 1) for a one-hot P (weight 1): the histogram of the index vector
int onehot_try_agg_col(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled) {
    *handled = false;
    if (!arg->onehot || arg->dev_valid || op != DB2_AGG_SUM || arg->onehot->weight != 1.0 || arg->cols > 8192 ||
        arg->rows >= (int64_t)1 << 53)
        return DB2_OK;
    const uint64_t before = g_launches.load();
    const int k = (int)arg->cols;
    DB2_TRY(prepare_result(ctx, res, DB2_F64, 1, k));
    DB2_CHECK((*res)->dev_ld >= 1, DB2_EINVAL, "bad result");
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, (size_t)k * 8, &scratch));
    DB2_CUDA(cudaMemsetAsync(scratch, 0, (size_t)k * 8, ctx->stream));
    std::shared_ptr<const OneHot> oh = arg->onehot;
    if (arg->rows > 0) {
        int64_t want = (arg->rows + 255) / 256;
        const int64_t cap = (int64_t)sm_count() * 8;
        onehot_hist_kernel<<<(unsigned)(want < cap ? want : cap), 256, (size_t)k * 4, ctx->stream>>>(
            static_cast<const int64_t *>(oh->idx.ptr(8)), oh->idx.ld, arg->rows, k,
            static_cast<unsigned long long *>(scratch));
        DB2_TRY(after_launch("onehot_hist_kernel"));
    }
    onehot_hist_final_kernel<<<(k + 255) / 256, 256, 0, ctx->stream>>>(
        static_cast<const unsigned long long *>(scratch), k, static_cast<double *>((*res)->dev_ptr()));
    DB2_TRY(after_launch("onehot_hist_final_kernel"));
    count(ctx, before);
    *handled = true;
    return DB2_OK;
}

} // namespace db2
