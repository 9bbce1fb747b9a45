// Internal C++ view of the runtime objects behind the opaque handles of the C-ABI.
#pragma once

#include "common.cuh"

#include <map>
#include <memory>
#include <unordered_map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace db2 {
struct Expr;
struct OneHot;
struct ColStats;
struct Operand;
struct DevBuf;
} // namespace db2

struct db2_matrix;
struct db2_csr;

struct db2_context {
    int device = 0;
    // deferred evaluation (lazy.cu): row aggregations waiting to be served by one fused pass
    std::vector<db2_matrix *> pending;
    std::vector<db2_matrix *> lazies; // live matrices that stand for an unevaluated elementwise chain
    bool eager = false; // DB2_EAGER=1: run every operator call immediately (no fusion)
    cudaStream_t stream = nullptr;
    cudaStream_t side_stream = nullptr; // collectives and result copies that run beside the compute stream
    // device buffers that a copy on the side stream still reads (db2_matrix_to_host_async): kept from the allocator,
    // which hands freed blocks straight back to the compute stream, until db2_context_side_sync
    std::vector<std::shared_ptr<db2::DevBuf>> side_keep;
    // caching device allocator: freed blocks are kept by size and handed out again without calling the driver; all
    // work of a context is ordered on its one stream, so a freed block may be reused immediately
    std::multimap<size_t, void *> free_blocks;
    std::unordered_map<void *, size_t> block_size;
    size_t cached_bytes = 0;
    size_t mem_free_seen = 0; // free device memory at the last query (pipeline.cu sizes its batches from it)
    size_t mem_budget = 0; // > 0: pooled allocations may hold at most this many bytes (db2_context_set_mem_budget)
    // reusable scratch for two-stage reductions (grown on demand, stream-ordered reuse)
    void *scratch = nullptr;
    size_t scratch_bytes = 0;
    // device status word for domain errors + pinned host mirror
    int32_t *dev_status = nullptr;
    int32_t *host_status = nullptr;
    // db2_aggAllStart / db2_scalarStart: one event per outstanding scalar (the values sit in host_status)
    cudaEvent_t scalar_ev[2] = {nullptr, nullptr};
    // cross-GPU combine (comm.cu): this context's rank among `world` row shards and its NCCL communicator
    int rank = 0, world = 1;
    void *comm = nullptr;
    bool comm_is_fake = false;   // installed by the test hook db2_comm_test_attach: never passed to NCCL's destroy
    // member of a single-process device group (group.cu): the communicator that ncclCommInitAll made for this device
    void *group_comm = nullptr;
    int dup = 0; // number of contexts of the same group, listed before this one, that share its physical device
    // column statistics of the matrix that was last aggregated by columns (colstats.cu)
    std::shared_ptr<db2::ColStats> colstats;
    // the t(X) X that was asked for last and has not been computed yet (db2_matrix::syrk_of)
    db2_matrix *syrk_waiting = nullptr;
    std::mutex mu;
    db2_stats stats{};
    // the handle returned by db2_context_create holds one reference, every pooled buffer another: a context is torn
    // down when the last of them goes, so matrices may outlive db2_context_destroy
    std::atomic<int> refs{1};
};

namespace db2 {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string &m) : std::runtime_error(m), code(c) {}
};

// RAII device buffer from the context's pool (or borrowed from the caller)
struct DevBuf {
    db2_context *ctx;
    void *ptr;
    size_t bytes;
    bool owned;
    uint64_t version = 0; // bumped whenever a kernel writes into an existing buffer (results placed through views)
    // set while work on ANOTHER stream than the context's still writes the buffer (db2_allreduce_async): whoever
    // touches the buffer next makes the context's stream wait for it first (wait_ready)
    cudaEvent_t ready = nullptr;
    ~DevBuf();
};

// (pivot, S1, S2) per column of one device-resident matrix, valid while that buffer lives and is not rewritten
struct ColStats {
    std::weak_ptr<DevBuf> buf;
    uint64_t version = 0;
    int64_t off = 0, ld = 0, rows = 0, cols = 0;
    std::shared_ptr<DevBuf> stats; // 3 * cols doubles
    // row-sharded runs: the buffer the column sums of this shard went to, and -- once that result has been combined
    // over the ranks -- every rank's (rows, pivot, S1, S2, sums), so that the squared deviations from the GLOBAL mean
    // are answered for all shards at once, without a second exchange
    std::weak_ptr<DevBuf> sum_buf;
    uint64_t sum_version = 0;
    std::shared_ptr<DevBuf> gathered; // world x (1 + 4 * cols) doubles
    int world = 1;
};

struct HostBuf {
    void *ptr;
    size_t bytes;
    bool owned; // owned buffers are pinned (cudaMallocHost)
    ~HostBuf();
};

int ctx_alloc(db2_context *ctx, size_t bytes, void **out);
int ctx_free(db2_context *ctx, void *ptr, size_t bytes);
int ctx_scratch(db2_context *ctx, size_t bytes, void **out);
void ctx_release(db2_context *ctx);
std::shared_ptr<DevBuf> make_devbuf(db2_context *ctx, size_t bytes); // throws Error

inline void wait_ready(db2_context *ctx, DevBuf *b) {
    if (b && b->ready) {
        cudaStreamWaitEvent(ctx->stream, b->ready, 0);
        cudaEventDestroy(b->ready);
        b->ready = nullptr;
    }
}

inline void bind_device(const db2_context *ctx) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess || cur != ctx->device)
        cudaSetDevice(ctx->device);
}

} // namespace db2

struct db2_matrix {
    std::atomic<int> refs{1};
    db2_context *ctx = nullptr;
    int dtype = DB2_F64;
    int64_t rows = 0, cols = 0;
    // device placement
    std::shared_ptr<db2::DevBuf> dev;
    int64_t dev_off = 0; // element offset of (0,0) inside dev
    int64_t dev_ld = 0;
    bool dev_valid = false;
    // host placement
    std::shared_ptr<db2::HostBuf> host;
    int64_t host_off = 0;
    int64_t host_ld = 0;
    bool host_valid = false;
    // deferred elementwise chain: the values are expr(base operand) and no placement is valid yet
    std::shared_ptr<const db2::Expr> lazy;
    // pending row aggregation `pend_op` of `pend_src`, produced together with its siblings when first needed
    std::shared_ptr<const db2::Expr> pend_src;
    int pend_op = -1;

    // one-hot rows (r, idx[r]) = weight that have not been written out (onehot.cu)
    std::shared_ptr<const db2::OneHot> onehot;
    // t(X) X that has not been computed yet (ops_la.cu): a gemv on the same X that arrives first is computed in the
    // same pass over X; any other use computes the product alone
    std::shared_ptr<const db2::Operand> syrk_of;
    // the matrix is the int64 sequence seq_start, seq_start + seq_inc, ... (set by db2_seq; values are on the device too)
    bool is_seq = false;
    int64_t seq_start = 0, seq_inc = 0;

    bool is_view = false; // shares its buffers with a parent (row slice): results written through it stay in place
    // the values already are the combination over the row shards of all ranks (computed from exchanged statistics): the
    // next all-reduce of this matrix has nothing left to do
    bool combined = false;

    bool deferred() const { return (bool)lazy || (bool)pend_src || (bool)onehot || (bool)syrk_of; }
    size_t esize() const { return db2::dtype_size(dtype); }
    void *dev_ptr() const { return static_cast<char *>(dev->ptr) + dev_off * (int64_t)esize(); }
    void *host_ptr() const { return static_cast<char *>(host->ptr) + host_off * (int64_t)esize(); }
};

namespace db2 {

// ---- deferred evaluation (lazy.cu) ----
struct Operand { // a materialised device operand; holds its buffer alive
    std::shared_ptr<DevBuf> buf;
    int64_t off = 0, ld = 0, rows = 0, cols = 0;
    const void *ptr(size_t es) const { return static_cast<const char *>(buf->ptr) + off * (int64_t)es; }
    bool same(const Operand &o) const {
        return buf.get() == o.buf.get() && off == o.off && ld == o.ld && rows == o.rows && cols == o.cols;
    }
};
struct ExprStep {
    int kind = 0, op = 0; // FusedOperandKind, FusedOp
    bool reversed = false;
    Operand operand;
    double imm = 0.0;
    bool same(const ExprStep &o) const {
        if (kind != o.kind || op != o.op || reversed != o.reversed)
            return false;
        if (kind == 3)
            return memcmp(&imm, &o.imm, sizeof(double)) == 0;
        if (kind == 4)
            return true;
        return operand.same(o.operand);
    }
};
struct GemmSrc { // the base values are the product A @ op(B) (tall-skinny, skinny.cu), not yet computed
    Operand A, B;
    bool tb = false;
    int64_t K = 0;
};
struct CsrSrc { // the base values are the row aggregation `op` of a CSR matrix (csr.cu), not yet computed
    db2_csr *m; // holds a reference; may itself be a deferred sparse (.) dense product
    int op;
    CsrSrc(db2_csr *m, int op);
    ~CsrSrc();
    CsrSrc(const CsrSrc &) = delete;
};
struct Expr {
    int dtype = DB2_F64;
    int64_t rows = 0, cols = 0;
    Operand base;                        // materialised base operand, unless ...
    std::shared_ptr<const GemmSrc> gemm; // ... the chain starts from a deferred product
    std::shared_ptr<const CsrSrc> csr;   // ... or from a deferred row aggregation of a CSR matrix (rows x 1)
    std::vector<ExprStep> steps;
    bool same_base(const Expr &o) const {
        if (csr || o.csr)
            return csr && o.csr && csr->m == o.csr->m && csr->op == o.csr->op;
        if (gemm || o.gemm)
            return gemm && o.gemm && gemm->A.same(o.gemm->A) && gemm->B.same(o.gemm->B) && gemm->tb == o.gemm->tb;
        return base.same(o.base);
    }
};
struct OneHot { // rows x cols matrix with one stored entry per row: (r, idx[r]) = weight
    Operand idx; // int64 column vector
    double weight = 1.0;
};
// column aggregation through the one-pass statistics (colstats.cu): SUM / MEAN fill them, VAR / STDDEV and the
// deferred  sum((X - mu)^2)  are answered from them
int colstats_try_agg_col(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled);
// handled: the result is complete.  Otherwise, with *run_if set: the result was written from the statistics and the
// device word *run_if says whether the data turned out ill-conditioned for that (non-zero) -- the caller queues the
// ordinary pass with that word as its condition, and nobody waits for the host to look at it.
int colstats_try_sqdev(db2_context *ctx, const Expr &e, db2_matrix **res, bool *handled, const int32_t **run_if);
// all-reduce (ADD) of the column sums that filled the statistics: one all-gather that also carries every rank's
// statistics (colstats.cu); comm_allgather_f64 is the raw collective (comm.cu)
int colstats_try_allreduce(db2_context *ctx, db2_matrix *m, bool *handled);
int comm_allgather_f64(db2_context *ctx, const double *send, double *recv, size_t count);
int onehot_force(db2_matrix *m); // writes the dense rows
int onehot_try_matmul(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, int transa, int transb,
                      bool *handled);
int onehot_try_agg_col(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled);
// Each returns DB2_OK and sets *handled when the call was recorded instead of executed.
int lazy_try_binary(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, bool *handled);
int lazy_try_scalar(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, const void *scalar, bool *handled);
int lazy_try_unary(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled);
int lazy_try_agg_row(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled);
// row aggregation of a CSR matrix (or of a deferred sparse (.) dense product): deferred, so that a following chain on
// the rows x 1 result (max(., c), . != c), its sum and its intermediate results come out of the same pass
int lazy_try_agg_row_csr(db2_context *ctx, int op, db2_matrix **res, db2_csr *arg, bool *handled);
int lazy_try_agg_col(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg, bool *handled);
// A @ op(B) for a tall lhs and at most 64 result columns: deferred, so that a following chain and row extremum are
// applied to the accumulators
int lazy_try_matmul(db2_context *ctx, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs, int transa, int transb,
                    bool *handled);
// full aggregation of a deferred chain without materialising it (SUM of flat-evaluable chains); *res_host gets the value
int syrk_force(db2_matrix *m); // ops_la.cu: computes a deferred t(X) X on its own
int lazy_try_agg_all(db2_context *ctx, int op, double *res_host, db2_matrix *arg, bool *handled);
// the same without the wait: the sum is written to `pinned` (pinned host memory) by the pass that this call queues
int lazy_try_agg_all_start(db2_context *ctx, int op, double *pinned, db2_matrix *arg, bool *handled);
int lazy_force(db2_matrix *m);          // materialises a deferred matrix (and the pending siblings it can serve)
int lazy_flush_all(db2_context *ctx);   // produces every pending aggregation
void lazy_forget(db2_matrix *m);        // a deferred matrix is being destroyed

// device groups (comm.cu): NCCL communicators for the contexts of one process, grouped all-reduce
int nccl_init_group(const std::vector<db2_context *> &ctxs);
void nccl_destroy_group(const std::vector<db2_context *> &ctxs);
int nccl_allreduce_group(const std::vector<db2_context *> &ctxs, const std::vector<db2_matrix *> &ms, int combine);

// makes the device placement current (allocation + async H2D when only the host copy is valid)
int ensure_device(db2_matrix *m);
// result allocation following the reference's "*res == nullptr means allocate" convention; checks shape/type otherwise
int prepare_result(db2_context *ctx, db2_matrix **res, int dtype, int64_t rows, int64_t cols);
} // namespace db2

#define DB2_API_BEGIN try {
#define DB2_API_END                                                                                                    \
    }                                                                                                                  \
    catch (const ::db2::Error &e) { return ::db2::set_error(e.code, "%s", e.what()); }                                 \
    catch (const std::bad_alloc &) { return ::db2::set_error(DB2_ENOMEM, "out of host memory"); }                      \
    catch (const std::exception &e) { return ::db2::set_error(DB2_EINVAL, "%s", e.what()); }
