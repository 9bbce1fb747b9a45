// Deferred evaluation: cheap elementwise operator calls on large f64 matrices are recorded as a chain on their base
// operand; row aggregations of such chains (or of plain matrices) are parked as "pending" results; the first time a
// pending or deferred value is actually needed, one fused pass (fused.cu) produces it together with every pending
// sibling whose chain is a prefix-compatible view of the same base operand.
//
// Why this is safe: DAPHNE's data objects are immutable values (the compiler's SSA form; results are fresh objects),
// so a chain may keep reading its operands until it is evaluated; every operand's buffer is kept alive by the chain.
// Callers that wrap their own device buffers must not overwrite them while results derived from them are alive.
// A context and its matrices are driven by one host thread at a time (the reference runs one WorkerGPU thread per
// CUDA context, src/runtime/local/vectorized/WorkerGPU.h:38-52).
#include "fused.cuh"
#include "runtime.h"

#include <algorithm>
#include <cmath>
#include <string>

namespace db2 {

static constexpr int64_t LAZY_MIN_ELEMS = 1 << 16; // below this an immediate kernel is cheaper than bookkeeping

static int fused_binary_op(int op) {
    switch (op) {
    case DB2_ADD: return FO_ADD;
    case DB2_SUB: return FO_SUB;
    case DB2_MUL: return FO_MUL;
    case DB2_DIV: return FO_DIV;
    case DB2_EQ: return FO_EQ;
    case DB2_NEQ: return FO_NEQ;
    case DB2_LT: return FO_LT;
    case DB2_LE: return FO_LE;
    case DB2_GT: return FO_GT;
    case DB2_GE: return FO_GE;
    case DB2_MIN: return FO_MIN;
    case DB2_MAX: return FO_MAX;
    case DB2_AND: return FO_AND;
    case DB2_OR: return FO_OR;
    default: return -1;
    }
}
static int fused_unary_op(int op) {
    switch (op) {
    case DB2_U_MINUS: return FO_NEG;
    case DB2_U_ABS: return FO_ABS;
    case DB2_U_SIGN: return FO_SIGN;
    case DB2_U_FLOOR: return FO_FLOOR;
    case DB2_U_CEIL: return FO_CEIL;
    case DB2_U_ROUND: return FO_ROUND;
    case DB2_U_ISNAN: return FO_ISNAN;
    default: return -1;
    }
}

static bool lazy_candidate(const db2_context *ctx, const db2_matrix *m) {
    return !ctx->eager && m->dtype == DB2_F64 && m->rows * m->cols >= LAZY_MIN_ELEMS && m->cols < (1 << 30);
}

static int operand_of(db2_matrix *m, Operand *out) {
    DB2_TRY(ensure_device(m)); // materialises deferred operands
    out->buf = m->dev;
    out->off = m->dev_off;
    out->ld = m->dev_ld;
    out->rows = m->rows;
    out->cols = m->cols;
    return DB2_OK;
}

// the chain that `m` stands for: its own when deferred, else a fresh chain on the matrix itself
static int chain_of(db2_matrix *m, std::shared_ptr<Expr> *out) {
    auto e = std::make_shared<Expr>();
    if (m->lazy) {
        *e = *m->lazy;
    } else {
        e->dtype = m->dtype;
        e->rows = m->rows;
        e->cols = m->cols;
        DB2_TRY(operand_of(m, &e->base));
    }
    *out = e;
    return DB2_OK;
}

static void set_lazy(db2_matrix *r, std::shared_ptr<Expr> e) {
    r->lazy = std::move(e);
    r->ctx->lazies.push_back(r);
}
static void unlazy(db2_matrix *m) {
    auto &v = m->ctx->lazies;
    v.erase(std::remove(v.begin(), v.end(), m), v.end());
}

static db2_matrix *new_deferred(db2_context *ctx, int dtype, int64_t rows, int64_t cols) {
    db2_matrix *m = new db2_matrix();
    m->ctx = ctx;
    m->dtype = dtype;
    m->rows = rows;
    m->cols = cols;
    return m;
}

int lazy_try_binary(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, bool *handled) {
    *handled = false;
    const int fop = fused_binary_op(op);
    if (*res != nullptr || fop < 0 || !lazy_candidate(ctx, lhs) || rhs->dtype != DB2_F64)
        return DB2_OK;
    if (lhs->pend_src) // a pending aggregate is a column vector: it is produced and the operator runs at once
        return DB2_OK;
    // (a pending rhs is produced by operand_of below and becomes an ordinary operand of the chain)
    int kind;
    if (lhs->rows == rhs->rows && lhs->cols == rhs->cols)
        kind = FK_MATRIX;
    else if (lhs->cols == rhs->cols && rhs->rows == 1 && lhs->rows > 1)
        kind = FK_ROWVEC;
    else if (lhs->rows == rhs->rows && rhs->cols == 1 && lhs->cols > 1)
        kind = FK_COLVEC;
    else
        return DB2_OK; // unusual broadcast forms run immediately
    std::shared_ptr<Expr> e;
    ExprStep st;
    st.kind = kind;
    st.op = fop;
    if (kind == FK_MATRIX && rhs->lazy && !lhs->lazy) {
        // the deferred side is the right operand: continue ITS chain with the operands swapped
        DB2_TRY(chain_of(rhs, &e));
        st.reversed = true;
        DB2_TRY(operand_of(lhs, &st.operand));
    } else {
        DB2_TRY(chain_of(lhs, &e));
        DB2_TRY(operand_of(rhs, &st.operand)); // a deferred rhs is produced first
    }
    if ((int)e->steps.size() >= FUSED_MAX_STEPS)
        return DB2_OK; // chain full: run this operator immediately (its inputs are materialised on demand)
    e->steps.push_back(st);
    db2_matrix *r = new_deferred(ctx, DB2_F64, lhs->rows, lhs->cols);
    set_lazy(r, e);
    *res = r;
    *handled = true;
    return DB2_OK;
}

int lazy_try_scalar(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, const void *scalar, bool *handled) {
    *handled = false;
    if (*res != nullptr || !lazy_candidate(ctx, lhs) || lhs->pend_src)
        return DB2_OK;
    const double s = *static_cast<const double *>(scalar);
    int fop = fused_binary_op(op);
    if (op == DB2_POW && s == 2.0)
        fop = FO_SQUARE;
    if (fop < 0)
        return DB2_OK;
    std::shared_ptr<Expr> e;
    DB2_TRY(chain_of(lhs, &e));
    if ((int)e->steps.size() >= FUSED_MAX_STEPS)
        return DB2_OK;
    ExprStep st;
    st.kind = FK_SCALAR;
    st.op = fop;
    st.imm = s;
    e->steps.push_back(st);
    db2_matrix *r = new_deferred(ctx, DB2_F64, lhs->rows, lhs->cols);
    set_lazy(r, e);
    *res = r;
    *handled = true;
    return DB2_OK;
}

int lazy_try_unary(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled) {
    *handled = false;
    const int fop = fused_unary_op(op);
    if (*res != nullptr || fop < 0 || !lazy_candidate(ctx, arg) || arg->pend_src)
        return DB2_OK;
    std::shared_ptr<Expr> e;
    DB2_TRY(chain_of(arg, &e));
    if ((int)e->steps.size() >= FUSED_MAX_STEPS)
        return DB2_OK;
    ExprStep st;
    st.kind = FK_UNARY;
    st.op = fop;
    e->steps.push_back(st);
    db2_matrix *r = new_deferred(ctx, DB2_F64, arg->rows, arg->cols);
    set_lazy(r, e);
    *res = r;
    *handled = true;
    return DB2_OK;
}

static bool row_agg_fusable(int op) {
    return op == DB2_AGG_SUM || op == DB2_AGG_PROD || op == DB2_AGG_MIN || op == DB2_AGG_MAX ||
           op == DB2_AGG_IDXMIN || op == DB2_AGG_IDXMAX || op == DB2_AGG_MEAN;
}

int lazy_try_agg_row(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled) {
    *handled = false;
    if (*res != nullptr || !row_agg_fusable(op) || !lazy_candidate(ctx, arg) || arg->pend_src || arg->cols < 2)
        return DB2_OK;
    std::shared_ptr<Expr> e;
    if (arg->lazy)
        e = std::const_pointer_cast<Expr>(arg->lazy); // shared, never modified
    else
        DB2_TRY(chain_of(arg, &e));
    const bool idx = op == DB2_AGG_IDXMIN || op == DB2_AGG_IDXMAX;
    db2_matrix *r = new_deferred(ctx, idx ? DB2_U64 : DB2_F64, arg->rows, 1);
    r->pend_src = e;
    r->pend_op = op;
    ctx->pending.push_back(r);
    *res = r;
    *handled = true;
    // bound the backlog: a full group is produced right away
    int same_base = 0;
    for (db2_matrix *p : ctx->pending)
        if (p->pend_src->same_base(*e))
            same_base++;
    if (same_base >= FUSED_MAX_AGGS)
        return lazy_force(r);
    return DB2_OK;
}

// fills the device-side program from a chain; returns false if the chain cannot be expressed (never for chains
// built above)
static void build_program(const Expr &e, size_t nsteps, FusedProgram *P) {
    memset(P, 0, sizeof(*P));
    const bool no_base = e.gemm || e.csr;
    P->base = no_base ? nullptr : e.base.ptr(8);
    P->base_ld = no_base ? e.cols : e.base.ld;
    P->rows = e.rows;
    P->cols = e.cols;
    P->nsteps = (int)nsteps;
    int smem = 0;
    const int smem_budget = (56 * 1024) / 8; // doubles, on top of the 33 KB tile
    for (size_t i = 0; i < nsteps; i++) {
        const ExprStep &s = e.steps[i];
        FusedStep &d = P->steps[i];
        d.kind = s.kind;
        d.op = s.op;
        d.reversed = s.reversed ? 1 : 0;
        d.smem_off = -1;
        d.imm = s.imm;
        if (s.kind == FK_MATRIX || s.kind == FK_ROWVEC || s.kind == FK_COLVEC) {
            d.ptr = s.operand.ptr(8);
            d.ld = s.operand.ld;
        }
        if (s.kind == FK_ROWVEC) {
            // the operand, then (for a divisor) its reciprocal helpers, each padded to an even number of values so
            // that pairs stay 16-byte aligned for an odd number of columns
            const int need = (int)((e.cols + 1) & ~(int64_t)1) * ((s.op == FO_DIV && !s.reversed) ? 2 : 1);
            if (smem + need <= smem_budget) {
                d.smem_off = smem;
                smem += need;
            }
        }
    }
    P->smem_elems = smem;
}

static bool is_prefix(const Expr &a, const Expr &b) { // a's chain is a prefix of b's (same base)
    if (!a.same_base(b) || a.rows != b.rows || a.cols != b.cols || a.steps.size() > b.steps.size())
        return false;
    for (size_t i = 0; i < a.steps.size(); i++)
        if (!a.steps[i].same(b.steps[i]))
            return false;
    return true;
}

static void unpend(db2_context *ctx, db2_matrix *m) {
    auto &v = ctx->pending;
    v.erase(std::remove(v.begin(), v.end(), m), v.end());
}

static const char *fused_op_name(int op) {
    static const char *n[] = {"ADD", "SUB", "MUL", "DIV", "SQ", "EQ", "NEQ", "LT", "LE", "GT", "GE", "MIN", "MAX", "AND",
                              "OR", "NEG", "ABS", "SIGN", "FLOOR", "CEIL", "ROUND", "ISNAN"};
    return (op >= 0 && op < FO_COUNT) ? n[op] : "?";
}

// Spells a program: "SUB.R|DIV.R|SQ.S#MAX@2,SUM@3+EW" (operand kinds M/R/C/S/U, a trailing r = reversed operands).
static std::string signature_of(const FusedProgram &P) {
    std::string sig;
    for (int i = 0; i < P.nsteps; i++) {
        if (i)
            sig += "|";
        sig += fused_op_name(P.steps[i].op);
        sig += ".";
        sig += "MRCSU"[P.steps[i].kind];
        if (P.steps[i].reversed)
            sig += "r";
    }
    sig += "#";
    static const char *tk[] = {"SUM", "PROD", "MIN", "MAX", "MEAN"};
    for (int i = 0; i < P.ntaps; i++) {
        if (i)
            sig += ",";
        sig += tk[P.taps[i].kind];
        sig += "@" + std::to_string(P.taps[i].after_step);
    }
    if (P.ew_out)
        sig += "+EW";
    return sig;
}

static int tap_kind_of(int agg_op) {
    switch (agg_op) {
    case DB2_AGG_SUM: return FT_SUM;
    case DB2_AGG_PROD: return FT_PROD;
    case DB2_AGG_MIN:
    case DB2_AGG_IDXMIN: return FT_MIN;
    case DB2_AGG_MAX:
    case DB2_AGG_IDXMAX: return FT_MAX;
    default: return FT_MEAN;
    }
}

// One fused pass over `longest`: materialises `ew_target` (may be null) and every pending aggregation in `group`
// (members that do not fit the tap slots stay pending).  MIN/IDXMIN and MAX/IDXMAX of the same chain position share
// one tracker.
static int run_row_pass(db2_context *ctx, const Expr &longest, db2_matrix *ew_target,
                        const std::vector<db2_matrix *> &group);

static void fill_skinny(const Expr &e, SkinnyArgs *a) {
    const GemmSrc &g = *e.gemm;
    a->A = static_cast<const double *>(g.A.ptr(8));
    a->lda = g.A.ld;
    a->n = e.rows;
    a->B = static_cast<const double *>(g.B.ptr(8));
    a->ldb = g.B.ld;
    a->K = (int)g.K;
    a->N = (int)e.cols;
    a->tb = g.tb ? 1 : 0;
}

// can chain and aggregations be applied to the accumulators of the product?
static bool gemm_pass_fusable(const Expr &e, const std::vector<db2_matrix *> &group) {
    int rowvecs = 0, colvecs = 0;
    for (const ExprStep &s : e.steps) {
        if (s.kind == FK_MATRIX || !skinny_op_supported(s.op))
            return false;
        rowvecs += s.kind == FK_ROWVEC;
        colvecs += s.kind == FK_COLVEC;
    }
    if (rowvecs > skinny_vec_slots() || colvecs > skinny_vec_slots())
        return false;
    std::vector<int> kinds;
    for (const db2_matrix *g : group) {
        const int op = g->pend_op;
        if (g->pend_src->steps.size() != e.steps.size() ||
            !(op == DB2_AGG_MIN || op == DB2_AGG_MAX || op == DB2_AGG_IDXMIN || op == DB2_AGG_IDXMAX))
            return false;
    }
    return true;
}

// the live deferred matrix (other than `self`) whose chain is the longest proper, non-empty prefix of e's
static db2_matrix *prefix_sibling(db2_context *ctx, const db2_matrix *self, const Expr &e) {
    db2_matrix *sibling = nullptr;
    for (db2_matrix *m : ctx->lazies)
        if (m != self && m->lazy && !m->lazy->steps.empty() && m->lazy->steps.size() < e.steps.size() &&
            is_prefix(*m->lazy, e) && (!sibling || m->lazy->steps.size() > sibling->lazy->steps.size()))
            sibling = m;
    return sibling;
}

// One pass over a CSR matrix that produces its row aggregation with the chain `e` applied: the final values into
// `target` (may be null), the values of a live prefix of the chain into that matrix, the sum of the final values into
// *sum_dev (device, may be null).
static int run_csr_pass(db2_context *ctx, const Expr &e, db2_matrix *target, double *sum_dev) {
    FusedProgram P;
    build_program(e, e.steps.size(), &P);
    for (int i = 0; i < P.nsteps; i++) // operands are indexed by row: matrices must be rows x 1, row vectors 1 x 1
        DB2_CHECK(P.steps[i].kind != FK_ROWVEC || e.steps[i].operand.cols == 1, DB2_EUNSUPPORTED,
                  "a chain on a CSR row aggregation with a wide row-vector operand");
    db2_matrix *sibling = prefix_sibling(ctx, target, e);
    double *mid = nullptr;
    int mid_after = 0;
    if (sibling) {
        sibling->dev = make_devbuf(ctx, (size_t)sibling->rows * 8);
        sibling->dev_off = 0;
        sibling->dev_ld = 1;
        mid = static_cast<double *>(sibling->dev->ptr);
        mid_after = (int)sibling->lazy->steps.size();
    }
    if (target) {
        target->dev = make_devbuf(ctx, (size_t)e.rows * 8);
        target->dev_off = 0;
        target->dev_ld = 1;
        P.ew_out = target->dev->ptr;
        P.ew_out_ld = 1;
    }
    void *scratch = nullptr;
    const size_t head = 64; // (callers keep a result in front of the partial sums)
    if (sum_dev)
        DB2_TRY(ctx_scratch(ctx, csr_agg_scratch_bytes() + head, &scratch));
    DB2_TRY(csr_agg_pass(ctx, *e.csr, P, mid, mid_after, sum_dev,
                         scratch ? static_cast<char *>(scratch) + head : nullptr,
                         scratch ? ctx->scratch_bytes - head : 0));
    for (db2_matrix *m : {sibling, target})
        if (m) {
            m->dev_valid = true;
            unlazy(m);
            m->lazy.reset();
        }
    return DB2_OK;
}

static int run_row_pass(db2_context *ctx, const Expr &longest, db2_matrix *ew_target,
                        const std::vector<db2_matrix *> &group) {
    if (longest.csr) {
        DB2_CHECK(group.empty(), DB2_EUNSUPPORTED, "row aggregations of a rows x 1 chain are not deferred");
        return run_csr_pass(ctx, longest, ew_target, nullptr);
    }
    if (longest.gemm && !gemm_pass_fusable(longest, group)) {
        // the product is written out and the ordinary pass runs on it
        Expr plain = longest;
        plain.gemm.reset();
        plain.base.buf = make_devbuf(ctx, (size_t)longest.rows * longest.cols * 8);
        plain.base.off = 0;
        plain.base.ld = longest.cols;
        plain.base.rows = longest.rows;
        plain.base.cols = longest.cols;
        SkinnyArgs a;
        memset(&a, 0, sizeof(a));
        fill_skinny(longest, &a);
        a.prog.rows = longest.rows;
        a.prog.cols = longest.cols;
        a.prog.ew_out = plain.base.buf->ptr;
        a.prog.ew_out_ld = longest.cols;
        DB2_TRY(skinny_gemm(a, ctx->stream));
        if (plain.steps.empty() && group.empty() && ew_target) { // the product itself was wanted
            ew_target->dev = plain.base.buf;
            ew_target->dev_off = 0;
            ew_target->dev_ld = longest.cols;
            ew_target->dev_valid = true;
            unlazy(ew_target);
            ew_target->lazy.reset();
            return DB2_OK;
        }
        return run_row_pass(ctx, plain, ew_target, group);
    }
    FusedProgram P;
    build_program(longest, longest.steps.size(), &P);
    if (ew_target) {
        ew_target->dev = make_devbuf(ctx, (size_t)longest.rows * longest.cols * 8);
        ew_target->dev_off = 0;
        ew_target->dev_ld = longest.cols;
        P.ew_out = ew_target->dev->ptr;
        P.ew_out_ld = longest.cols;
    }
    // canonical order: by chain position, then tracker kind
    std::vector<db2_matrix *> sorted(group);
    std::stable_sort(sorted.begin(), sorted.end(), [](const db2_matrix *a, const db2_matrix *b) {
        const size_t pa = a->pend_src->steps.size(), pb = b->pend_src->steps.size();
        if (pa != pb)
            return pa < pb;
        return tap_kind_of(a->pend_op) < tap_kind_of(b->pend_op);
    });
    std::vector<db2_matrix *> served;
    for (db2_matrix *g : sorted) {
        const int after = (int)g->pend_src->steps.size(), kind = tap_kind_of(g->pend_op);
        const bool idx = g->pend_op == DB2_AGG_IDXMIN || g->pend_op == DB2_AGG_IDXMAX;
        int slot = -1;
        for (int t = 0; t < P.ntaps; t++)
            if (P.taps[t].after_step == after && P.taps[t].kind == kind && (idx ? !P.taps[t].out_idx : !P.taps[t].out))
                slot = t;
        if (slot < 0) {
            if (P.ntaps >= FUSED_MAX_AGGS)
                continue; // stays pending
            slot = P.ntaps++;
            P.taps[slot].after_step = after;
            P.taps[slot].kind = kind;
        }
        g->dev = make_devbuf(ctx, (size_t)g->rows * 8);
        g->dev_off = 0;
        g->dev_ld = 1;
        (idx ? P.taps[slot].out_idx : P.taps[slot].out) = g->dev->ptr;
        served.push_back(g);
    }
    int rc = DB2_OK;
    const std::string sig = signature_of(P);
    if (longest.gemm) {
        SkinnyArgs a;
        memset(&a, 0, sizeof(a));
        fill_skinny(longest, &a);
        a.prog = P;
        rc = skinny_gemm(a, ctx->stream);
    } else if (fused_flat_eligible(P))
        rc = fused_flat_pass_f64(P, nullptr, 0, nullptr, nullptr, 0, ctx->stream);
    else if (!fused_row_pass_ct(P, sig.c_str(), ctx->stream, &rc))
        rc = fused_row_pass_f64(P, ctx->stream);
    DB2_TRY(rc);
    if (ew_target) {
        ew_target->dev_valid = true;
        unlazy(ew_target);
        ew_target->lazy.reset();
    }
    for (db2_matrix *g : served) {
        g->dev_valid = true;
        g->pend_src.reset();
        g->pend_op = -1;
        unpend(ctx, g);
    }
    return DB2_OK;
}

int lazy_force(db2_matrix *m) {
    db2_context *ctx = m->ctx;
    bind_device(ctx);
    if (m->onehot)
        return onehot_force(m);
    if (m->syrk_of)
        return syrk_force(m);
    const uint64_t before = g_launches.load();
    int rc = DB2_OK;
    if (m->lazy) {
        // materialisation; pending aggregations of prefixes of this chain ride along
        std::shared_ptr<const Expr> e = m->lazy;
        std::vector<db2_matrix *> group;
        for (db2_matrix *p : ctx->pending)
            if ((int)group.size() < FUSED_MAX_AGGS && is_prefix(*p->pend_src, *e))
                group.push_back(p);
        rc = run_row_pass(ctx, *e, m, group);
    } else if (m->pend_src) {
        std::shared_ptr<const Expr> longest = m->pend_src;
        std::vector<db2_matrix *> group{m};
        for (db2_matrix *p : ctx->pending) {
            if (p == m || (int)group.size() >= FUSED_MAX_AGGS)
                continue;
            if (is_prefix(*p->pend_src, *longest)) {
                group.push_back(p);
            } else if (is_prefix(*longest, *p->pend_src)) {
                longest = p->pend_src;
                group.push_back(p);
            }
        }
        rc = run_row_pass(ctx, *longest, nullptr, group);
        if (rc == DB2_OK && m->pend_src) // more distinct trackers than one pass holds: serve m on its own
            rc = run_row_pass(ctx, *std::shared_ptr<const Expr>(m->pend_src), nullptr, {m});
    }
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.launches += g_launches.load() - before;
    }
    return rc;
}

int lazy_flush_all(db2_context *ctx) {
    while (!ctx->pending.empty())
        DB2_TRY(lazy_force(ctx->pending.front()));
    return DB2_OK;
}

void lazy_forget(db2_matrix *m) {
    if (m->syrk_of && m->ctx && m->ctx->syrk_waiting == m)
        m->ctx->syrk_waiting = nullptr;
    if (m->pend_src && m->ctx)
        unpend(m->ctx, m);
    if (m->lazy && m->ctx)
        unlazy(m);
}

int lazy_try_agg_col(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled) {
    *handled = false;
    if (!arg->lazy || ctx->eager)
        return DB2_OK; // plain matrices use the dedicated column kernels
    const bool ok = op == DB2_AGG_SUM || op == DB2_AGG_PROD || op == DB2_AGG_MIN || op == DB2_AGG_MAX ||
                    op == DB2_AGG_IDXMIN || op == DB2_AGG_IDXMAX || op == DB2_AGG_MEAN;
    if (!ok)
        return DB2_OK; // VAR/STDDEV: the argument is materialised and the two-pass kernels run
    std::shared_ptr<const Expr> e = arg->lazy;
    if (e->gemm)
        return DB2_OK; // the deferred product is produced first (ensure_device), then the column kernels run
    if (e->csr) {
        // sum of a chain on a CSR row aggregation: the pass leaves it on the device (1 x 1), e.g. the number of
        // labels that changed, which a multi-GPU run combines before anybody reads it
        if (op != DB2_AGG_SUM || *res != nullptr)
            return DB2_OK;
        DB2_TRY(prepare_result(ctx, res, DB2_F64, 1, 1));
        DB2_TRY(run_csr_pass(ctx, *e, nullptr, static_cast<double *>((*res)->dev_ptr())));
        *handled = true;
        return DB2_OK;
    }
    const int32_t *run_if = nullptr;
    if (op == DB2_AGG_SUM) { // sum((X - mu)^2) right after the column sums of X: answered from the statistics
        DB2_TRY(colstats_try_sqdev(ctx, *e, res, handled, &run_if));
        if (*handled)
            return DB2_OK;
    }
    const bool idx = op == DB2_AGG_IDXMIN || op == DB2_AGG_IDXMAX;
    DB2_TRY(prepare_result(ctx, res, idx ? DB2_U64 : DB2_F64, 1, arg->cols));
    FusedProgram P;
    build_program(*e, e->steps.size(), &P);
    P.run_if = run_if;
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, fused_col_scratch_bytes(arg->cols), &scratch));
    int rc = DB2_OK;
    const std::string sig = signature_of(P);
    if (!fused_col_pass_ct(P, sig.c_str(), op, (*res)->dev_ptr(), scratch, ctx->scratch_bytes, ctx->stream, &rc))
        rc = fused_col_pass_f64(P, op, (*res)->dev_ptr(), scratch, ctx->scratch_bytes, ctx->stream);
    DB2_TRY(rc);
    *handled = true;
    return DB2_OK;
}

int lazy_try_agg_row_csr(db2_context *ctx, int op, db2_matrix **res, db2_csr *arg, bool *handled) {
    *handled = false;
    int64_t rows = 0;
    DB2_TRY(db2_csr_info(arg, &rows, nullptr, nullptr));
    if (*res != nullptr || ctx->eager || rows < LAZY_MIN_ELEMS)
        return DB2_OK;
    auto e = std::make_shared<Expr>();
    e->rows = rows;
    e->cols = 1;
    e->csr = std::make_shared<CsrSrc>(arg, op);
    db2_matrix *r = new_deferred(ctx, DB2_F64, rows, 1);
    set_lazy(r, e);
    *res = r;
    *handled = true;
    return DB2_OK;
}

int lazy_try_matmul(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, int transa, int transb,
                    bool *handled) {
    *handled = false;
    if (*res != nullptr || ctx->eager || transa || lhs->dtype != DB2_F64 || rhs->dtype != DB2_F64)
        return DB2_OK;
    const int64_t m = lhs->rows, k = lhs->cols, n = transb ? rhs->rows : rhs->cols;
    if ((transb ? rhs->cols : rhs->rows) != k || m * n < LAZY_MIN_ELEMS || n > 64 || k > 128)
        return DB2_OK;
    auto g = std::make_shared<GemmSrc>();
    DB2_TRY(operand_of(lhs, &g->A));
    DB2_TRY(operand_of(rhs, &g->B));
    if (!skinny_shape_ok(m, k, n, g->A.ptr(8), g->A.ld))
        return DB2_OK;
    g->tb = transb != 0;
    g->K = k;
    auto e = std::make_shared<Expr>();
    e->rows = m;
    e->cols = n;
    e->gemm = g;
    db2_matrix *r = new_deferred(ctx, DB2_F64, m, n);
    set_lazy(r, e);
    *res = r;
    *handled = true;
    return DB2_OK;
}

// sum(chain) in one flat pass; a live deferred matrix whose chain is a proper prefix (e.g. u of sum(u != c)) is
// materialised by the same pass
int lazy_try_agg_all_start(db2_context *ctx, int op, double *pinned, db2_matrix *arg, bool *handled) {
    *handled = false;
    if (!arg->lazy || ctx->eager || op != DB2_AGG_SUM || arg->dtype != DB2_F64)
        return DB2_OK;
    std::shared_ptr<const Expr> e = arg->lazy;
    if (!e->csr)
        return DB2_OK;
    const uint64_t before = g_launches.load();
    DB2_TRY(run_csr_pass(ctx, *e, nullptr, pinned));
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load() - before;
    ctx->stats.d2h_bytes += sizeof(double);
    *handled = true;
    return DB2_OK;
}

int lazy_try_agg_all(db2_context *ctx, int op, double *res_host, db2_matrix *arg, bool *handled) {
    *handled = false;
    if (!arg->lazy || ctx->eager || op != DB2_AGG_SUM || arg->dtype != DB2_F64)
        return DB2_OK;
    std::shared_ptr<const Expr> e = arg->lazy;
    if (e->gemm)
        return DB2_OK;
    if (e->csr) { // one pass over the CSR arrays: aggregate, chain, live prefix of the chain, sum
        const uint64_t before = g_launches.load();
        // the last block of the pass writes the sum straight into pinned host memory (device-accessible under unified
        // addressing): the host only waits for the stream, no copy is queued behind the kernel
        double *pinned = reinterpret_cast<double *>(ctx->host_status + 48);
        DB2_TRY(run_csr_pass(ctx, *e, nullptr, pinned));
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
        *res_host = *pinned;
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.launches += g_launches.load() - before;
        ctx->stats.d2h_bytes += sizeof(double);
        *handled = true;
        return DB2_OK;
    }
    FusedProgram P;
    build_program(*e, e->steps.size(), &P);
    if (!fused_flat_eligible(P))
        return DB2_OK;
    db2_matrix *sibling = prefix_sibling(ctx, arg, *e);
    const uint64_t before = g_launches.load();
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, fused_flat_scratch_bytes() + 64, &scratch));
    void *mid = nullptr;
    int mid_after = 0;
    if (sibling) {
        sibling->dev = make_devbuf(ctx, (size_t)sibling->rows * sibling->cols * 8);
        sibling->dev_off = 0;
        sibling->dev_ld = sibling->cols;
        mid = sibling->dev->ptr;
        mid_after = (int)sibling->lazy->steps.size();
    }
    // the sum sits in the first 8 bytes of the scratch area, the partials behind it
    DB2_TRY(fused_flat_pass_f64(P, mid, mid_after, static_cast<double *>(scratch), static_cast<char *>(scratch) + 64,
                                ctx->scratch_bytes - 64, ctx->stream));
    if (sibling) {
        sibling->dev_valid = true;
        unlazy(sibling);
        sibling->lazy.reset();
    }
    DB2_CUDA(cudaMemcpyAsync(res_host, scratch, sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.launches += g_launches.load() - before;
        ctx->stats.d2h_bytes += sizeof(double);
    }
    *handled = true;
    return DB2_OK;
}

} // namespace db2
