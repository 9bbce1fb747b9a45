// The kernel-call sequences that the benchmark workloads lower to, issued from native code.
//
// DAPHNE's JIT-compiled `main` calls one kernel per operator through the C ABI with next to no host time between the
// calls.  These functions are that caller for the five workloads: the same operator calls, in the same order, as the
// DaphneDSL scripts lower to (PhyOperatorSelection: t(X) @ X -> syrk, t(X) @ y -> gemv; one kernel call per op), made
// through the public db2_* operator interface -- nothing here reaches below it.  With a communicator on the context
// they run row-sharded: every rank calls them on its row block and the ADD partials are combined on the device.
#include "runtime.h"

#include <functional>
#include <vector>

using namespace db2;

namespace {

struct H { // owning handle
    db2_matrix *m = nullptr;
    H() = default;
    H(const H &) = delete;
    ~H() { reset(); }
    void reset(db2_matrix *n = nullptr) {
        if (m)
            db2_matrix_decref(m);
        m = n;
    }
    db2_matrix *release() {
        db2_matrix *r = m;
        m = nullptr;
        return r;
    }
    db2_matrix **operator&() { return &m; }
    operator db2_matrix *() const { return m; }
};
struct HC {
    db2_csr *m = nullptr;
    ~HC() {
        if (m)
            db2_csr_decref(m);
    }
};

int combine(db2_context *ctx, db2_matrix *m) { return ctx->world > 1 ? db2_allreduce(ctx, m, DB2_COMBINE_ADD) : DB2_OK; }

// two ADD partials of one step, combined by one NCCL launch
int combine2(db2_context *ctx, db2_matrix *a, db2_matrix *b) {
    if (ctx->world == 1)
        return DB2_OK;
    DB2_TRY(db2_comm_group_begin(ctx));
    int rc = db2_allreduce(ctx, a, DB2_COMBINE_ADD);
    if (rc == DB2_OK)
        rc = db2_allreduce(ctx, b, DB2_COMBINE_ADD);
    const int rc_end = db2_comm_group_end(ctx);
    return rc != DB2_OK ? rc : rc_end;
}

int scalar_op(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, double s) {
    return db2_ewBinaryObjSca(ctx, op, res, lhs, &s);
}

} // namespace

extern "C" {

// Connected components by label propagation (test/api/cli/algorithms/components.daphne:14-26):
//   c = seq(1, n, 1); while (diff > 0 && iter <= maxi) { u = max(aggMax(G * t(c), 0), c); diff = sum(u != c); c = u; }
// G holds the rows [row_lo, row_lo + G.rows) of the n x n adjacency matrix.  Sharded: the change count is combined on
// the device and the label blocks are all-gathered behind it on the same stream; one value is read per iteration.
//
// The loop condition needs the count of trip k on the host.  Trip k + 1 is queued BEFORE that count is awaited, so
// the device works on it while the value travels and the host prepares the calls.  Should trip k turn out to have
// changed nothing, the script would have stopped there: the labels after trip k are returned and trip k + 1 (which
// reproduces them: c is a fixpoint) is dropped.  Labels and the iteration count are those of the script's loop.
int db2w_connected_components(db2_context *ctx, db2_csr *G, int64_t row_lo, int64_t maxi, db2_matrix **labels,
                              int64_t *iterations) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && G && labels && iterations, DB2_EINVAL, "null argument");
    int64_t rows = 0, n = 0;
    DB2_TRY(db2_csr_info(G, &rows, &n, nullptr));
    const bool sharded = ctx->world > 1;
    H c_full, c_loc; // the labels after trip it - 1
    const double one = 1.0, last = (double)n;
    DB2_TRY(db2_seq(ctx, &c_full, DB2_F64, &one, &last, &one));
    DB2_TRY(db2_matrix_slice_rows(c_full, row_lo, row_lo + rows, &c_loc));
    int64_t it = 1;
    for (;;) {
        const bool queue = it <= maxi;
        H n_full, n_loc; // the labels after trip it
        if (queue) {
            H tc, mx, u, ne;
            HC prod;
            DB2_TRY(db2_transpose(ctx, &tc, c_full));
            DB2_TRY(db2_ewMulCsrDense(ctx, &prod.m, G, tc));
            DB2_TRY(db2_aggRowCsr(ctx, DB2_AGG_MAX, &mx, prod.m));
            DB2_TRY(db2_ewBinaryMat(ctx, DB2_MAX, &u, mx, c_loc));
            DB2_TRY(db2_ewBinaryMat(ctx, DB2_NEQ, &ne, u, c_loc));
            if (sharded) {
                H cnt;
                DB2_TRY(db2_aggCol(ctx, DB2_AGG_SUM, &cnt, ne));
                DB2_TRY(db2_comm_group_begin(ctx)); // the count and the labels travel in one NCCL launch
                int rc = db2_allreduce(ctx, cnt, DB2_COMBINE_ADD);
                if (rc == DB2_OK)
                    rc = db2_allgatherv_rows(ctx, u, n, &n_full);
                const int rc_end = db2_comm_group_end(ctx);
                DB2_TRY(rc != DB2_OK ? rc : rc_end);
                DB2_TRY(db2_scalarStart(ctx, cnt, (int)(it & 1)));
                DB2_TRY(db2_matrix_slice_rows(n_full, row_lo, row_lo + rows, &n_loc));
            } else {
                DB2_TRY(db2_aggAllStart(ctx, DB2_AGG_SUM, ne, (int)(it & 1)));
                db2_matrix_incref(u);
                n_loc.reset(u);
                n_full.reset(u.release());
            }
        }
        if (it > 1) {
            double diff = 0.0;
            DB2_TRY(db2_scalarWait(ctx, (int)((it - 1) & 1), &diff));
            if (!(diff > 0.0) || !queue)
                break; // trip it - 1 was the script's last
        } else if (!queue) {
            break;
        }
        c_full.reset(n_full.release());
        c_loc.reset(n_loc.release());
        it++;
    }
    *iterations = it - 1;
    *labels = c_loc.release();
    return DB2_OK;
    DB2_API_END
}

// Column standardisation and aggregation, the memory-bound pipeline of the benchmark:
//   mu = mean(X, 1); sd = sqrt(var(X, 1)); Z = (X - mu) / sd;
//   r = sum(Z ^ 2, 0); s = sum(r); m = aggMax(Z, 0); i = idxMax(Z, 0);
// with mean / var issued as their ADD-combinable forms (column sums over the global row count n_total), so that row
// shards on several GPUs give the global statistics.  s is returned as a 1 x 1 matrix on the device (combined over
// the ranks): nothing in here waits for the host.  ev_rows_begin / ev_rows_end (optional, db2_event_create) are
// recorded around the pass that produces r, m and i.
int db2w_standardise(db2_context *ctx, db2_matrix *X, int64_t n_total, db2_matrix **mu_out, db2_matrix **sd_out,
                     db2_matrix **r_out, db2_matrix **max_out, db2_matrix **idx_out, db2_matrix **s_out,
                     void *ev_rows_begin, void *ev_rows_end) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && X && mu_out && sd_out && r_out && max_out && idx_out && s_out, DB2_EINVAL, "null argument");
    const double n = (double)(n_total > 0 ? n_total : X->rows), two = 2.0;
    H s1, mu, d, d2, v, var, sd, xc, Z, z2, r, m, idx, s;
    DB2_TRY(db2_aggCol(ctx, DB2_AGG_SUM, &s1, X));
    DB2_TRY(combine(ctx, s1));
    DB2_TRY(db2_ewBinaryObjSca(ctx, DB2_DIV, &mu, s1, &n));
    DB2_TRY(db2_ewBinaryMat(ctx, DB2_SUB, &d, X, mu));
    DB2_TRY(db2_ewBinaryObjSca(ctx, DB2_POW, &d2, d, &two));
    d.reset();
    DB2_TRY(db2_aggCol(ctx, DB2_AGG_SUM, &v, d2));
    d2.reset();
    DB2_TRY(combine(ctx, v));
    DB2_TRY(db2_ewBinaryObjSca(ctx, DB2_DIV, &var, v, &n));
    DB2_TRY(db2_ewUnaryMat(ctx, DB2_U_SQRT, &sd, var));
    DB2_TRY(db2_ewBinaryMat(ctx, DB2_SUB, &xc, X, mu));
    DB2_TRY(db2_ewBinaryMat(ctx, DB2_DIV, &Z, xc, sd));
    xc.reset();
    DB2_TRY(db2_ewBinaryObjSca(ctx, DB2_POW, &z2, Z, &two));
    DB2_TRY(db2_aggRow(ctx, DB2_AGG_SUM, &r, z2));
    z2.reset();
    DB2_TRY(db2_aggRow(ctx, DB2_AGG_MAX, &m, Z));
    DB2_TRY(db2_aggRow(ctx, DB2_AGG_IDXMAX, &idx, Z));
    Z.reset();
    if (ev_rows_begin)
        DB2_TRY(db2_event_record(ev_rows_begin, ctx->stream));
    void *unused = nullptr;
    DB2_TRY(db2_matrix_device_ptr(r, &unused, nullptr)); // the three row aggregations come out of one pass over X
    if (ev_rows_end)
        DB2_TRY(db2_event_record(ev_rows_end, ctx->stream));
    DB2_TRY(db2_aggCol(ctx, DB2_AGG_SUM, &s, r));
    if (ctx->world > 1) // nobody on the device needs s: its combine runs beside the stream
        DB2_TRY(db2_allreduce_async(ctx, s, DB2_COMBINE_ADD));
    *mu_out = mu.release();
    *sd_out = sd.release();
    *r_out = r.release();
    *max_out = m.release();
    *idx_out = idx.release();
    *s_out = s.release();
    return DB2_OK;
    DB2_API_END
}

// K-means assignment + update (test/api/cli/algorithms/kmeans.daphne:14-21):
//   xs = sum(X ^ 2, 0);
//   for i: D = (X @ t(C)) * -2.0 + xs + t(sum(C ^ 2, 0)); a = idxMin(D, 0);
//          P = ctable(seq(0, n - 1), a, 1.0, n, k); C = (t(P) @ X) / t(sum(P, 1));
int db2w_kmeans(db2_context *ctx, db2_matrix *X, db2_matrix *C0, int iterations, db2_matrix **C_out,
                db2_matrix **assign_out) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && X && C0 && C_out && assign_out, DB2_EINVAL, "null argument");
    const int64_t n = X->rows, k = C0->rows;
    H x2, xs, rows;
    DB2_TRY(scalar_op(ctx, DB2_POW, &x2, X, 2.0));
    DB2_TRY(db2_aggRow(ctx, DB2_AGG_SUM, &xs, x2));
    x2.reset();
    const int64_t zero = 0, lastrow = n - 1, inc = 1;
    DB2_TRY(db2_seq(ctx, &rows, DB2_I64, &zero, &lastrow, &inc));
    H Cm, assign;
    db2_matrix_incref(C0);
    Cm.reset(C0);
    for (int i = 0; i < iterations; i++) {
        H c2, cs, cst, xc, t1, t2, D, idx, P, sums, counts, ct, Cn;
        DB2_TRY(scalar_op(ctx, DB2_POW, &c2, Cm, 2.0));
        DB2_TRY(db2_aggRow(ctx, DB2_AGG_SUM, &cs, c2));
        DB2_TRY(db2_transpose(ctx, &cst, cs));
        DB2_TRY(db2_matMul(ctx, &xc, X, Cm, 0, 1));
        DB2_TRY(scalar_op(ctx, DB2_MUL, &t1, xc, -2.0));
        DB2_TRY(db2_ewBinaryMat(ctx, DB2_ADD, &t2, t1, xs));
        DB2_TRY(db2_ewBinaryMat(ctx, DB2_ADD, &D, t2, cst));
        DB2_TRY(db2_aggRow(ctx, DB2_AGG_IDXMIN, &idx, D));
        assign.reset();
        DB2_TRY(db2_castObj(ctx, &assign, idx, DB2_I64));
        D.reset();
        t2.reset();
        t1.reset();
        xc.reset();
        DB2_TRY(db2_ctable(ctx, &P, rows, assign, 1.0, n, k));
        DB2_TRY(db2_matMul(ctx, &sums, P, X, 1, 0));
        DB2_TRY(db2_aggCol(ctx, DB2_AGG_SUM, &counts, P));
        DB2_TRY(combine2(ctx, sums, counts));
        P.reset();
        DB2_TRY(db2_transpose(ctx, &ct, counts));
        DB2_TRY(db2_ewBinaryMat(ctx, DB2_DIV, &Cn, sums, ct));
        Cm.reset(Cn.release());
    }
    *C_out = Cm.release();
    *assign_out = assign.release();
    return DB2_OK;
    DB2_API_END
}

// Linear regression by the normal equations (lmDS, scripts/algorithms/lmDS_.daph:98-112):
//   A = t(X) @ X + diagMatrix(fill(lambda, ncol(X), 1)); b = t(X) @ y; beta = solve(A, b);
int db2w_normal_equations(db2_context *ctx, db2_matrix *X, db2_matrix *y, double lambda, db2_matrix **A_out,
                          db2_matrix **b_out, db2_matrix **beta_out) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && X && y && A_out && b_out && beta_out, DB2_EINVAL, "null argument");
    H xtx, xty, lam, diag, A, beta;
    DB2_TRY(db2_syrk(ctx, &xtx, X, 1));
    DB2_TRY(db2_gemv(ctx, &xty, X, y));
    DB2_TRY(combine2(ctx, xtx, xty));
    DB2_TRY(db2_fill(ctx, &lam, DB2_F64, &lambda, X->cols, 1));
    DB2_TRY(db2_diagMatrix(ctx, &diag, lam));
    DB2_TRY(db2_ewBinaryMat(ctx, DB2_ADD, &A, xtx, diag));
    DB2_TRY(db2_solve(ctx, &beta, A, xty));
    *A_out = A.release();
    *b_out = xty.release();
    *beta_out = beta.release();
    return DB2_OK;
    DB2_API_END
}

} // extern "C"

// ---- column standardisation over a device group (one process, several GPUs) ----
namespace {

struct HD { // owning handle of a distributed matrix
    db2_dist *d = nullptr;
    ~HD() {
        if (d)
            db2_dist_decref(d);
    }
    db2_dist *release() {
        db2_dist *r = d;
        d = nullptr;
        return r;
    }
};

// the compiled bodies (what the lowering outlines as _vect_cudaN): they release their inputs and hand over results
void body_col_sums(db2_matrix ***outs, db2_matrix **ins, db2_context *ctx) {
    db2_aggCol(ctx, DB2_AGG_SUM, outs[0], ins[0]);
    db2_matrix_decref(ins[0]);
}
void body_sq_dev(db2_matrix ***outs, db2_matrix **ins, db2_context *ctx) {
    H d, d2;
    const double two = 2.0;
    db2_ewBinaryMat(ctx, DB2_SUB, &d, ins[0], ins[1]);
    db2_ewBinaryObjSca(ctx, DB2_POW, &d2, d, &two);
    db2_aggCol(ctx, DB2_AGG_SUM, outs[0], d2);
    db2_matrix_decref(ins[0]);
    db2_matrix_decref(ins[1]);
}
void body_rows(db2_matrix ***outs, db2_matrix **ins, db2_context *ctx) {
    H xc, Z, z2;
    const double two = 2.0;
    db2_ewBinaryMat(ctx, DB2_SUB, &xc, ins[0], ins[1]);
    db2_ewBinaryMat(ctx, DB2_DIV, &Z, xc, ins[2]);
    db2_ewBinaryObjSca(ctx, DB2_POW, &z2, Z, &two);
    db2_aggRow(ctx, DB2_AGG_SUM, outs[0], z2);
    db2_aggRow(ctx, DB2_AGG_MAX, outs[1], Z);
    db2_aggRow(ctx, DB2_AGG_IDXMAX, outs[2], Z);
    db2_aggCol(ctx, DB2_AGG_SUM, outs[3], *outs[0]);
    for (int i = 0; i < 3; i++)
        db2_matrix_decref(ins[i]);
}

// out = f(in) on every device of the group (small replicated follow-up arithmetic between two pipelines)
struct EachDevice {
    std::function<int(db2_context *, db2_matrix *, db2_matrix **)> f;
    db2_dist *in;
    std::vector<db2_matrix *> *res;
};
int each_device_call(int d, db2_context *c, void *user) {
    EachDevice *e = static_cast<EachDevice *>(user);
    db2_matrix *shard = nullptr;
    DB2_TRY(db2_dist_shard(e->in, d, &shard, nullptr));
    return e->f(c, shard, &(*e->res)[d]);
}
template <typename F> int on_every_device(db2_group *g, db2_dist *in, db2_dist **out, F &&f) {
    int n = 0;
    DB2_TRY(db2_group_size(g, &n));
    std::vector<db2_matrix *> res(n, nullptr);
    EachDevice each{f, in, &res};
    int rc = db2_group_run(g, each_device_call, &each); // all devices at once, each on its worker thread
    if (rc == DB2_OK)
        rc = db2_dist_from_shards(g, res.data(), -1, out);
    for (db2_matrix *m : res)
        if (m) {
            bind_device(m->ctx);
            db2_matrix_decref(m);
        }
    return rc;
}

} // namespace

extern "C" {

int db2w_standardise_group(db2_group *g, db2_dist *X, db2_dist **mu_out, db2_dist **sd_out, db2_dist **r_out,
                           db2_dist **max_out, db2_dist **idx_out, db2_dist **s_out) {
    DB2_API_BEGIN
    DB2_CHECK(g && X && mu_out && sd_out && r_out && max_out && idx_out && s_out, DB2_EINVAL, "null argument");
    int64_t rows = 0;
    DB2_TRY(db2_dist_info(X, nullptr, &rows, nullptr, nullptr));
    const double n = (double)rows;
    const int64_t rows_split = DB2_SPLIT_ROWS, none = DB2_SPLIT_NONE;
    HD sums, mu, v, sd;
    {
        db2_dist *ins[1] = {X};
        const int64_t splits[1] = {rows_split}, combines[1] = {DB2_COMBINE_ADD};
        DB2_TRY(db2_vectorizedPipelineGroup(g, &sums.d, 1, nullptr, ins, 1, nullptr, nullptr, splits, combines,
                                            body_col_sums, 0));
    }
    DB2_TRY(on_every_device(g, sums.d, &mu.d, [&](db2_context *c, db2_matrix *m, db2_matrix **o) {
        return db2_ewBinaryObjSca(c, DB2_DIV, o, m, &n);
    }));
    {
        db2_dist *ins[2] = {X, mu.d};
        const int64_t splits[2] = {rows_split, none}, combines[1] = {DB2_COMBINE_ADD};
        DB2_TRY(db2_vectorizedPipelineGroup(g, &v.d, 1, nullptr, ins, 2, nullptr, nullptr, splits, combines, body_sq_dev,
                                            0));
    }
    DB2_TRY(on_every_device(g, v.d, &sd.d, [&](db2_context *c, db2_matrix *m, db2_matrix **o) {
        H var;
        DB2_TRY(db2_ewBinaryObjSca(c, DB2_DIV, &var, m, &n));
        return db2_ewUnaryMat(c, DB2_U_SQRT, o, var);
    }));
    db2_dist *outs[4] = {nullptr, nullptr, nullptr, nullptr};
    {
        db2_dist *ins[3] = {X, mu.d, sd.d};
        const int64_t splits[3] = {rows_split, none, none};
        const int64_t combines[4] = {DB2_COMBINE_ROWS, DB2_COMBINE_ROWS, DB2_COMBINE_ROWS, DB2_COMBINE_ADD};
        DB2_TRY(db2_vectorizedPipelineGroup(g, outs, 4, nullptr, ins, 3, nullptr, nullptr, splits, combines, body_rows,
                                            0));
    }
    *mu_out = mu.release();
    *sd_out = sd.release();
    *r_out = outs[0];
    *max_out = outs[1];
    *idx_out = outs[2];
    *s_out = outs[3];
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
