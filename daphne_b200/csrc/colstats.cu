// Column statistics in one pass over a large f64 matrix.
//
// The standardisation workload asks for  mean(X, 1)  and then  var(X, 1)  (or, row-sharded, for the column sums of X
// and of (X - mu)^2).  The reference's AggCol reads X once for the mean and once more for the squared deviations
// (src/runtime/local/kernels/AggCol.h:146-173).  Here the pass that produces the column sums also accumulates, per
// column c and relative to a pivot K_c (the first row's value),
//        S1_c = sum_r (x_rc - K_c),      S2_c = sum_r (x_rc - K_c)^2,
// and keeps (K, S1, S2) beside the matrix.  A later request for  sum_r (x_rc - mu_c)^2  on the same, unchanged buffer is
// then answered without touching X:
//        sum_r (x - mu)^2  =  S2 - 2 d S1 + n d^2,     d = mu - K.
// This is algebra, not the reference's summation order; it stays inside the 1e-12 relative tolerance of f64
// reductions as long as the pivot is not far from the data (d^2 not >> the variance).  The answer kernel checks that
// condition per column and raises a flag instead of answering when it fails; the caller then runs the ordinary pass.
#include "fused.cuh"
#include "runtime.h"

namespace db2 {

constexpr int CS_THREADS = 256; // block = TX column pairs x TY row lanes, TX = 1 .. 32 by the column count

// partials [blockIdx.x][3][cols]: sum x, S1, S2 over the rows blockIdx.x * TY + ty, + gridDim.x * TY, ...
__global__ void __launch_bounds__(CS_THREADS)
    col_stats_partial_kernel(const double *__restrict__ X, int64_t rows, int64_t cols, int64_t ld, int vec,
                             double *__restrict__ part) {
    __shared__ double sh[3][CS_THREADS * 2]; // [statistic][(ty * TX + tx) * 2 + k]
    const int tx = threadIdx.x, ty = threadIdx.y, CS_TX = blockDim.x, CS_TY = blockDim.y;
    const int64_t c0 = ((int64_t)blockIdx.y * CS_TX + tx) * 2;
    double s0[2] = {0.0, 0.0}, s1[2] = {0.0, 0.0}, s2[2] = {0.0, 0.0}, piv[2] = {0.0, 0.0};
    const bool has0 = c0 < cols, has1 = c0 + 1 < cols;
    if (has0)
        piv[0] = X[c0];
    if (has1)
        piv[1] = X[c0 + 1];
    const int64_t stride = (int64_t)gridDim.x * CS_TY;
    if (vec && has1) {
        int64_t r = (int64_t)blockIdx.x * CS_TY + ty;
        for (; r + stride < rows; r += 2 * stride) { // two rows in flight per thread
            const double2 a = __ldcs(reinterpret_cast<const double2 *>(X + r * ld + c0));
            const double2 b = __ldcs(reinterpret_cast<const double2 *>(X + (r + stride) * ld + c0));
            double d;
            s0[0] = __dadd_rn(s0[0], a.x); d = __dsub_rn(a.x, piv[0]); s1[0] = __dadd_rn(s1[0], d); s2[0] = __fma_rn(d, d, s2[0]);
            s0[1] = __dadd_rn(s0[1], a.y); d = __dsub_rn(a.y, piv[1]); s1[1] = __dadd_rn(s1[1], d); s2[1] = __fma_rn(d, d, s2[1]);
            s0[0] = __dadd_rn(s0[0], b.x); d = __dsub_rn(b.x, piv[0]); s1[0] = __dadd_rn(s1[0], d); s2[0] = __fma_rn(d, d, s2[0]);
            s0[1] = __dadd_rn(s0[1], b.y); d = __dsub_rn(b.y, piv[1]); s1[1] = __dadd_rn(s1[1], d); s2[1] = __fma_rn(d, d, s2[1]);
        }
        for (; r < rows; r += stride) {
            const double2 a = __ldcs(reinterpret_cast<const double2 *>(X + r * ld + c0));
            double d;
            s0[0] = __dadd_rn(s0[0], a.x); d = __dsub_rn(a.x, piv[0]); s1[0] = __dadd_rn(s1[0], d); s2[0] = __fma_rn(d, d, s2[0]);
            s0[1] = __dadd_rn(s0[1], a.y); d = __dsub_rn(a.y, piv[1]); s1[1] = __dadd_rn(s1[1], d); s2[1] = __fma_rn(d, d, s2[1]);
        }
    } else if (has0) {
        for (int64_t r = (int64_t)blockIdx.x * CS_TY + ty; r < rows; r += stride)
            for (int k = 0; k < 2; k++)
                if (c0 + k < cols) {
                    const double x = X[r * ld + c0 + k], d = __dsub_rn(x, piv[k]);
                    s0[k] = __dadd_rn(s0[k], x);
                    s1[k] = __dadd_rn(s1[k], d);
                    s2[k] = __fma_rn(d, d, s2[k]);
                }
    }
    for (int k = 0; k < 2; k++) {
        sh[0][(ty * CS_TX + tx) * 2 + k] = s0[k];
        sh[1][(ty * CS_TX + tx) * 2 + k] = s1[k];
        sh[2][(ty * CS_TX + tx) * 2 + k] = s2[k];
    }
    __syncthreads();
    // thread (tx, ty) with ty < 6 finishes statistic ty / 2 of column c0 + ty % 2, adding the row lanes in order
    if (ty < 6) {
        const int q = ty / 2, k = ty % 2;
        if (c0 + k < cols) {
            double t = sh[q][tx * 2 + k];
            for (int y = 1; y < CS_TY; y++)
                t = __dadd_rn(t, sh[q][(y * CS_TX + tx) * 2 + k]);
            part[((int64_t)blockIdx.x * 3 + q) * cols + c0 + k] = t;
        }
    }
}

// one warp per (statistic, column): lanes add every 32nd partial, then a shuffle tree (fixed order)
// out: the column sums (out_mode 0) or means (1);  stats: [pivot | S1 | S2][cols]
__global__ void col_stats_final_kernel(const double *__restrict__ part, int parts, int64_t cols, int64_t rows,
                                       const double *__restrict__ X, int out_mode, double *__restrict__ out,
                                       double *__restrict__ stats) {
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    const int lane = threadIdx.x % 32;
    if (w >= 3 * cols)
        return;
    const int q = (int)(w / cols);
    const int64_t c = w % cols;
    double t = 0.0;
    for (int p = lane; p < parts; p += 32)
        t = __dadd_rn(t, part[((int64_t)p * 3 + q) * cols + c]);
    for (int m = 16; m >= 1; m >>= 1)
        t = __dadd_rn(t, shfl_xor(t, m));
    if (lane == 0) {
        if (q == 0) {
            out[c] = out_mode == 1 ? __ddiv_rn(t, (double)rows) : t;
            stats[c] = X[c]; // the pivot
        } else {
            stats[q * cols + c] = t;
        }
    }
}

// kind 0: out = sum (x - mu)^2;  1: population variance (mu = own mean);  2: standard deviation
// *flag is raised (and nothing usable is written) when a column's pivot is too far from the data for the identity
__global__ void col_stats_answer_kernel(const double *__restrict__ stats, int64_t cols, int64_t rows,
                                        const double *__restrict__ mu, int kind, double *__restrict__ out,
                                        int32_t *__restrict__ flag) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols)
        return;
    const double n = (double)rows, K = stats[c], S1 = stats[cols + c], S2 = stats[2 * cols + c];
    const double m = kind == 0 ? mu[c] : __dadd_rn(K, __ddiv_rn(S1, n));
    const double d = __dsub_rn(m, K);
    // S2 - 2 d S1 + n d^2
    const double r = __fma_rn(__dmul_rn(n, d), d, __fma_rn(__dmul_rn(-2.0, d), S1, S2));
    if (!(S2 <= 1000.0 * r) && S2 != 0.0)
        atomicExch(flag, 1);
    double v = r;
    if (kind >= 1)
        v = __ddiv_rn(r, n);
    if (kind == 2)
        v = __dsqrt_rn(v);
    out[c] = v;
}

// ---- row-sharded runs: statistics of all ranks ----
// packet of one rank: [rows | pivot (cols) | S1 (cols) | S2 (cols) | column sums (cols)]
__global__ void col_stats_pack_kernel(const double *__restrict__ stats, const double *__restrict__ sums, int64_t cols,
                                      int64_t rows, double *__restrict__ pkt) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i == 0)
        pkt[0] = (double)rows;
    if (i < 3 * cols)
        pkt[1 + i] = stats[i];
    if (i < cols)
        pkt[1 + 3 * cols + i] = sums[i];
}
// the column sums over all ranks, added in rank order (the same bits on every rank)
__global__ void col_stats_fold_kernel(const double *__restrict__ gathered, int world, int64_t cols,
                                      double *__restrict__ out) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols)
        return;
    const int64_t P = 1 + 4 * cols;
    double t = 0.0;
    for (int r = 0; r < world; r++)
        t = __dadd_rn(t, gathered[r * P + 1 + 3 * cols + c]);
    out[c] = t;
}
// sum over ALL ranks' rows of (x - mu)^2 from the gathered statistics: every rank's identity around its own pivot
__global__ void col_stats_answer_all_kernel(const double *__restrict__ gathered, int world, int64_t cols,
                                            const double *__restrict__ mu, double *__restrict__ out,
                                            int32_t *__restrict__ flag) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols)
        return;
    const int64_t P = 1 + 4 * cols;
    double tot = 0.0;
    for (int r = 0; r < world; r++) {
        const double *g = gathered + r * P;
        const double n = g[0], K = g[1 + c], S1 = g[1 + cols + c], S2 = g[1 + 2 * cols + c];
        const double d = __dsub_rn(mu[c], K);
        const double v = __fma_rn(__dmul_rn(n, d), d, __fma_rn(__dmul_rn(-2.0, d), S1, S2));
        if (!(S2 <= 1000.0 * v) && S2 != 0.0)
            atomicExch(flag, 1);
        tot = __dadd_rn(tot, v);
    }
    out[c] = tot;
}

size_t col_stats_scratch_bytes(int64_t cols) { return (size_t)sm_count() * 4 * 3 * (size_t)cols * sizeof(double); }

// column sums (out_mode 0) or means (1) of X into `out`, statistics into `stats` (3 * cols doubles)
int col_stats_pass(const double *X, int64_t rows, int64_t cols, int64_t ld, int out_mode, double *out, double *stats,
                   void *scratch, size_t scratch_bytes, cudaStream_t st) {
    int CS_TX = 1;
    while (CS_TX < 32 && CS_TX * 2 < cols)
        CS_TX *= 2;
    const int CS_TY = CS_THREADS / CS_TX; // >= 8
    const int gy = (int)((cols + CS_TX * 2 - 1) / (CS_TX * 2));
    int64_t gx = ((int64_t)sm_count() * 4 + gy - 1) / gy;
    const int64_t max_gx = (rows + CS_TY - 1) / CS_TY;
    if (gx > max_gx)
        gx = max_gx;
    if (gx < 1)
        gx = 1;
    DB2_CHECK(scratch && scratch_bytes >= (size_t)gx * 3 * cols * sizeof(double), DB2_EINVAL,
              "column statistics scratch too small");
    const int vec = aligned16(X) && ld % 2 == 0;
    col_stats_partial_kernel<<<dim3((unsigned)gx, gy), dim3(CS_TX, CS_TY), 0, st>>>(X, rows, cols, ld, vec,
                                                                                 static_cast<double *>(scratch));
    DB2_TRY(after_launch("col_stats_partial_kernel"));
    const int64_t warps = 3 * cols;
    col_stats_final_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(
        static_cast<const double *>(scratch), (int)gx, cols, rows, X, out_mode, out, stats);
    return after_launch("col_stats_final_kernel");
}

int col_stats_answer(const double *stats, int64_t cols, int64_t rows, const double *mu, int kind, double *out,
                     int32_t *flag, cudaStream_t st) {
    col_stats_answer_kernel<<<(unsigned)((cols + 127) / 128), 128, 0, st>>>(stats, cols, rows, mu, kind, out, flag);
    return after_launch("col_stats_answer_kernel");
}

static void count(db2_context *ctx, uint64_t before) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load(std::memory_order_relaxed) - before;
}

static bool stats_match(const db2_context *ctx, const std::shared_ptr<DevBuf> &buf, int64_t off, int64_t ld,
                        int64_t rows, int64_t cols) {
    const ColStats *cs = ctx->colstats.get();
    if (!cs || !buf)
        return false;
    std::shared_ptr<DevBuf> alive = cs->buf.lock();
    return alive && alive.get() == buf.get() && cs->version == buf->version && cs->off == off && cs->ld == ld &&
           cs->rows == rows && cs->cols == cols;
}

// runs the answer kernel and reads its flag: false = the identity is ill-conditioned for this data
static int answer_checked(db2_context *ctx, const DevBuf &stats, const double *mu, int kind, int64_t rows, int64_t cols,
                          double *out, bool *ok) {
    int32_t *flag = ctx->dev_status + 24;
    DB2_CUDA(cudaMemsetAsync(flag, 0, sizeof(int32_t), ctx->stream));
    DB2_TRY(col_stats_answer(static_cast<const double *>(stats.ptr), cols, rows, mu, kind, out, flag, ctx->stream));
    int32_t *h = ctx->host_status + 24;
    DB2_CUDA(cudaMemcpyAsync(h, flag, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    *ok = *h == 0;
    return DB2_OK;
}

static bool stats_candidate(const db2_context *ctx, const db2_matrix *m) {
    return !ctx->eager && m->dtype == DB2_F64 && !m->deferred() && m->rows >= 2 && m->cols >= 1 && m->cols <= 8192 &&
           m->rows * m->cols >= ((int64_t)1 << 22);
}

static int run_stats(db2_context *ctx, db2_matrix *arg, int out_mode, double *out,
                     std::shared_ptr<DevBuf> *stats_out = nullptr) {
    auto cs = std::make_shared<ColStats>();
    cs->stats = make_devbuf(ctx, (size_t)3 * arg->cols * sizeof(double));
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, col_stats_scratch_bytes(arg->cols), &scratch));
    DB2_TRY(col_stats_pass(static_cast<const double *>(arg->dev_ptr()), arg->rows, arg->cols, arg->dev_ld, out_mode, out,
                           static_cast<double *>(cs->stats->ptr), scratch, ctx->scratch_bytes, ctx->stream));
    if (stats_out)
        *stats_out = cs->stats;
    if (!arg->dev->owned) // a caller-owned buffer may be rewritten behind the runtime's back: nothing is remembered
        return DB2_OK;
    cs->buf = arg->dev;
    cs->version = arg->dev->version;
    cs->off = arg->dev_off;
    cs->ld = arg->dev_ld;
    cs->rows = arg->rows;
    cs->cols = arg->cols;
    ctx->colstats = cs;
    return DB2_OK;
}

int colstats_try_agg_col(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled) {
    *handled = false;
    const bool fills = op == DB2_AGG_SUM || op == DB2_AGG_MEAN, answers = op == DB2_AGG_VAR || op == DB2_AGG_STDDEV;
    if ((!fills && !answers) || !stats_candidate(ctx, arg))
        return DB2_OK;
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(arg));
    if (fills) {
        DB2_TRY(prepare_result(ctx, res, DB2_F64, 1, arg->cols));
        DB2_CHECK((*res)->dev_ld >= arg->cols, DB2_EINVAL, "bad result");
        DB2_TRY(run_stats(ctx, arg, op == DB2_AGG_MEAN ? 1 : 0, static_cast<double *>((*res)->dev_ptr())));
        if (op == DB2_AGG_SUM && ctx->colstats && ctx->colstats->buf.lock() == arg->dev) {
            ctx->colstats->sum_buf = (*res)->dev; // an all-reduce of these sums will carry the statistics along
            ctx->colstats->sum_version = (*res)->dev->version;
        }
        count(ctx, before);
        *handled = true;
        return DB2_OK;
    }
    std::shared_ptr<DevBuf> stats;
    if (stats_match(ctx, arg->dev, arg->dev_off, arg->dev_ld, arg->rows, arg->cols)) {
        stats = ctx->colstats->stats;
    } else {
        auto tmp = make_devbuf(ctx, (size_t)arg->cols * sizeof(double));
        DB2_TRY(run_stats(ctx, arg, 1, static_cast<double *>(tmp->ptr), &stats));
    }
    DB2_TRY(prepare_result(ctx, res, DB2_F64, 1, arg->cols));
    bool ok = false;
    DB2_TRY(answer_checked(ctx, *stats, nullptr, op == DB2_AGG_VAR ? 1 : 2, arg->rows, arg->cols,
                           static_cast<double *>((*res)->dev_ptr()), &ok));
    count(ctx, before);
    *handled = ok; // not ok: the two-pass kernels overwrite the result
    return DB2_OK;
}

int colstats_try_sqdev(db2_context *ctx, const Expr &e, db2_matrix **res, bool *handled, const int32_t **run_if) {
    *handled = false;
    *run_if = nullptr;
    if (e.gemm || e.steps.size() != 2 || e.dtype != DB2_F64)
        return DB2_OK;
    const ExprStep &sub = e.steps[0], &sq = e.steps[1];
    if (sub.kind != FK_ROWVEC || sub.op != FO_SUB || sub.reversed || sq.op != FO_SQUARE || sub.operand.ld < 1)
        return DB2_OK;
    if (!stats_match(ctx, e.base.buf, e.base.off, e.base.ld, e.rows, e.cols))
        return DB2_OK;
    const uint64_t before = g_launches.load();
    DB2_TRY(prepare_result(ctx, res, DB2_F64, 1, e.cols));
    bool ok = false;
    const ColStats &cs = *ctx->colstats;
    if (cs.gathered && cs.world == ctx->world && ctx->world > 1) {
        // the statistics of every rank are here: the result is the sum over ALL shards, marked as combined so that
        // the all-reduce the caller issues next is a no-op
        int32_t *flag = ctx->dev_status + 24, *h = ctx->host_status + 24;
        DB2_CUDA(cudaMemsetAsync(flag, 0, sizeof(int32_t), ctx->stream));
        col_stats_answer_all_kernel<<<(unsigned)((e.cols + 127) / 128), 128, 0, ctx->stream>>>(
            static_cast<const double *>(cs.gathered->ptr), cs.world, e.cols,
            static_cast<const double *>(sub.operand.ptr(8)), static_cast<double *>((*res)->dev_ptr()), flag);
        DB2_TRY(after_launch("col_stats_answer_all_kernel"));
        DB2_CUDA(cudaMemcpyAsync(h, flag, sizeof(int32_t), cudaMemcpyDeviceToHost, ctx->stream));
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
        // the flag must be the same on every rank (they all evaluate the same gathered numbers), so either all ranks
        // take this path or none does
        ok = *h == 0;
        (*res)->combined = ok;
    } else {
        // one shard: no host decision is needed.  The answer kernel raises the flag for ill-conditioned data and the
        // caller queues the ordinary pass behind it, to run only if the flag is up
        int32_t *flag = ctx->dev_status + 24;
        DB2_CUDA(cudaMemsetAsync(flag, 0, sizeof(int32_t), ctx->stream));
        DB2_TRY(col_stats_answer(static_cast<const double *>(cs.stats->ptr), e.cols, e.rows,
                                 static_cast<const double *>(sub.operand.ptr(8)), 0,
                                 static_cast<double *>((*res)->dev_ptr()), flag, ctx->stream));
        count(ctx, before);
        *run_if = flag;
        return DB2_OK;
    }
    count(ctx, before);
    *handled = ok;
    return DB2_OK;
}

int colstats_try_allreduce(db2_context *ctx, db2_matrix *m, bool *handled) {
    *handled = false;
    ColStats *cs = ctx->colstats.get();
    if (!cs || !m->dev || cs->sum_buf.lock() != m->dev || cs->sum_version != m->dev->version || m->rows != 1 ||
        m->cols != cs->cols || !cs->buf.lock())
        return DB2_OK;
    const int64_t cols = cs->cols, P = 1 + 4 * cols;
    const uint64_t before = g_launches.load();
    auto pkt = make_devbuf(ctx, (size_t)P * sizeof(double));
    auto gathered = make_devbuf(ctx, (size_t)P * ctx->world * sizeof(double));
    col_stats_pack_kernel<<<(unsigned)((3 * cols + 127) / 128), 128, 0, ctx->stream>>>(
        static_cast<const double *>(cs->stats->ptr), static_cast<const double *>(m->dev_ptr()), cols, cs->rows,
        static_cast<double *>(pkt->ptr));
    DB2_TRY(after_launch("col_stats_pack_kernel"));
    DB2_TRY(comm_allgather_f64(ctx, static_cast<const double *>(pkt->ptr), static_cast<double *>(gathered->ptr),
                               (size_t)P));
    col_stats_fold_kernel<<<(unsigned)((cols + 127) / 128), 128, 0, ctx->stream>>>(
        static_cast<const double *>(gathered->ptr), ctx->world, cols, static_cast<double *>(m->dev_ptr()));
    DB2_TRY(after_launch("col_stats_fold_kernel"));
    m->host_valid = false;
    cs->gathered = gathered;
    cs->world = ctx->world;
    cs->sum_buf.reset(); // the buffer now holds the global sums
    count(ctx, before);
    *handled = true;
    return DB2_OK;
}

} // namespace db2
