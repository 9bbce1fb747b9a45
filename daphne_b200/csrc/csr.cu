// CSR matrices on the device: residency, sparse (.) dense elementwise multiply, row aggregation, sparse x dense.
//
// The reference keeps CSRMatrix on the host only (three arrays with 64-bit size_t indices,
// src/runtime/local/datastructures/CSRMatrix.h:70-72) and materialises G * t(c) as a new CSR matrix in every
// iteration of connected components (EwBinaryMat.h:254-317) before aggregating it (AggRow.h:178-238).  Here a CSR
// matrix gets a device placement with 32-bit column indices (half the index traffic; 64-bit is kept when the column
// count needs it), the elementwise multiply with a dense operand is DEFERRED (the result remembers its two inputs),
// and the row aggregation of such a deferred product is ONE pass: per stored entry one value, one index and one
// gathered operand (L2-resident for a 1 x n row vector), no intermediate matrix.  The product is only materialised
// (count, scan, fill) when its arrays are actually requested.
#include "fused_step.cuh"
#include "runtime.h"


struct db2_csr {
    std::atomic<int> refs{1};
    db2_context *ctx = nullptr;
    int64_t rows = 0, cols = 0, nnz = 0; // nnz of the underlying arrays (a row view shares them)
    int64_t row0 = 0;                    // first row of this view inside the shared row-offset array
    // host placement (borrowed, reference layout)
    const double *h_val = nullptr;
    const uint64_t *h_col = nullptr, *h_off = nullptr;
    // device placement
    std::shared_ptr<db2::DevBuf> d_val, d_col, d_off;
    bool idx32 = true;
    bool unit_vals = false; // every stored value is exactly 1.0: kernels need not read the value array
    bool dev_valid = false;
    // deferred product lhs (.) rhs
    db2_csr *lazy_lhs = nullptr;
    db2_matrix *lazy_rhs = nullptr;

    const uint64_t *off_ptr() const { return static_cast<const uint64_t *>(d_off->ptr) + row0; }
};

namespace db2 {

enum { SK_NONE = 0, SK_ROWVEC = 1, SK_COLVEC = 2, SK_MATRIX = 3 };

template <typename IT> __global__ void narrow_idx_kernel(const uint64_t *in, IT *out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = (IT)in[i];
}
template <typename IT> __global__ void widen_idx_kernel(const IT *in, uint64_t *out, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = (uint64_t)in[i];
}

__device__ __forceinline__ double scale_at(int skind, const double *sc, int64_t sc_ld, int64_t r, int64_t c) {
    if (skind == SK_ROWVEC)
        return __ldg(sc + c);
    if (skind == SK_COLVEC)
        return __ldg(sc + r * sc_ld);
    return __ldg(sc + r * sc_ld + c);
}

// Epilogue of the row aggregation: a deferred elementwise chain on the rows x 1 result (lazy.cu), evaluated while the
// row's aggregate is still in a register.  Connected components issues  u = max(aggMax(G * t(c), 0), c);
// diff = sum(u != c)  as four operator calls; with the epilogue they are ONE pass that writes u and leaves the sum on
// the device.
struct CsrEpi {
    int32_t active, nsteps, mid_after, pad;
    double *mid_out; // values after mid_after steps (may be null)
    double *ew_out;  // final values (may be null)
    double *partials, *sum_out; // per-block sums of the final values; the last block folds them in block order
    unsigned int *ticket;
    // the operand of the first step that reads a vector is fetched together with the row's offsets (its latency then
    // overlaps the gathers); steps that read the same vector again reuse the value
    const double *pre_ptr;
    int64_t pre_ld;
    FusedStep steps[FUSED_MAX_STEPS];
};

// Row aggregation of val[i] * scale(r, col[i]); entries whose scale is exactly zero do not exist in the product
// (EwBinaryMat.h:295-302) and therefore count as implicit zeros.  G lanes per row; every lane group works on U rows
// at a time so that the dependent loads of a row (offsets -> column index -> gathered operand) of U rows overlap.
// UNIT: every stored value is exactly 1.0 (adjacency matrices), the value array is not read.
template <int G, typename IT, bool UNIT, int op>
__global__ void __launch_bounds__(256)
    csr_agg_row_kernel(const double *__restrict__ val, const IT *__restrict__ col,
                       const uint64_t *__restrict__ off, int64_t rows, int64_t cols, int skind,
                       const double *__restrict__ sc, int64_t sc_ld, double *__restrict__ out,
                       const __grid_constant__ CsrEpi E) {
    constexpr int RPC = 256 / G, U = 4;
    double local_sum = 0.0;
    // a row's aggregate leaves the kernel here: stored as it is, or sent through the chain of the epilogue
    auto emit = [&](int64_t r, double a, double pre, bool have_pre) {
        if (!E.active) {
            out[r] = a;
            return;
        }
        double v[1] = {a}, o[1], y[1];
        if (E.mid_out && E.mid_after == 0)
            E.mid_out[r] = a;
        for (int s = 0; s < E.nsteps; s++) {
            const FusedStep &st = E.steps[s];
            if (st.kind == FK_MATRIX || st.kind == FK_COLVEC)
                o[0] = (have_pre && st.ptr == E.pre_ptr && st.ld == E.pre_ld)
                           ? pre
                           : __ldg(static_cast<const double *>(st.ptr) + r * st.ld);
            else if (st.kind == FK_ROWVEC)
                o[0] = __ldg(static_cast<const double *>(st.ptr));
            else
                o[0] = st.imm;
            y[0] = (st.op == FO_DIV && !st.reversed) ? div_helper(o[0]) : 0.0;
            apply_step<1>(st.op, st.reversed != 0, v, o, y);
            if (E.mid_out && E.mid_after == s + 1)
                E.mid_out[r] = v[0];
        }
        if (E.ew_out)
            E.ew_out[r] = v[0];
        local_sum = __dadd_rn(local_sum, v[0]);
    };
    // A row much longer than the others would keep its G lanes busy for length / G dependent steps while the rest of
    // the warp waits (a hub of a power-law graph).  Such rows are only noted here and taken by the whole block at the
    // end of the kernel; when the list is full they are processed in place after all.
    constexpr int LONG_ROW = 64 * G, MAX_LONG = 64;
    __shared__ int64_t long_rows[MAX_LONG];
    __shared__ int n_long;
    __shared__ double red_v[8];
    __shared__ int red_k[8];
    if (threadIdx.x == 0)
        n_long = 0;
    __syncthreads();
    const int lane = threadIdx.x % G, grp = threadIdx.x / G;
    const int64_t stride = (int64_t)gridDim.x * RPC;
    const int64_t rows_padded = (rows + RPC - 1) / RPC * RPC;
    const double init = (op == DB2_AGG_MAX) ? -INFINITY : (op == DB2_AGG_MIN) ? INFINITY : (op == DB2_AGG_PROD) ? 1.0 : 0.0;
    auto combine = [&](double a, double x) {
        if (op == DB2_AGG_SUM)
            return __dadd_rn(a, x);
        if (op == DB2_AGG_PROD)
            return __dmul_rn(a, x);
        if (op == DB2_AGG_MAX)
            return (a < x) ? x : a;
        return (x < a) ? x : a;
    };
    for (int64_t r0 = (int64_t)blockIdx.x * RPC + grp; r0 < rows_padded; r0 += stride * U) {
        uint64_t b[U], e[U];
        double acc[U], pre[U];
        int kept[U]; // entries of the row that exist in the product (only compared with the column count)
        bool deferred[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int64_t r = r0 + u * stride;
            const bool live = r < rows;
            b[u] = live ? off[r] : 0;
            e[u] = live ? off[r + 1] : 0;
            pre[u] = (live && lane == 0 && E.pre_ptr) ? __ldg(E.pre_ptr + r * E.pre_ld) : 0.0;
            acc[u] = init;
            kept[u] = 0;
            deferred[u] = false;
        }
        // every warp is converged here (all threads of the block make the same number of turns): the groups that want
        // a slot for a long row are counted with ballots and the warp takes its slots with one atomic
        {
            const int wl = threadIdx.x % 32, leader = wl / G * G;
            bool want[U], any = false;
#pragma unroll
            for (int u = 0; u < U; u++) {
                want[u] = e[u] - b[u] > (uint64_t)LONG_ROW; // the same in all G lanes of a group
                any |= want[u];
            }
            if (__any_sync(0xffffffffu, any)) { // warp-uniform, rare
                unsigned leaders[U];
                int total = 0;
#pragma unroll
                for (int u = 0; u < U; u++) {
                    leaders[u] = __ballot_sync(0xffffffffu, want[u] && lane == 0);
                    total += __popc(leaders[u]);
                }
                int base = 0;
                if (wl == 0)
                    base = atomicAdd(&n_long, total);
                base = __shfl_sync(0xffffffffu, base, 0);
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int slot = base + __popc(leaders[u] & ((1u << leader) - 1u));
                    base += __popc(leaders[u]);
                    if (want[u] && slot < MAX_LONG) {
                        if (lane == 0)
                            long_rows[slot] = r0 + u * stride;
                        deferred[u] = true;
                        e[u] = b[u]; // nothing to do here
                    }
                }
            }
        }
        // first entry of every lane: the loads of the U rows are issued back to back
        int64_t cc[U];
        double xx[U], ss[U];
        bool have[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint64_t i = b[u] + lane;
            have[u] = i < e[u];
            cc[u] = have[u] ? (int64_t)col[i] : 0;
            xx[u] = (UNIT || !have[u]) ? 1.0 : val[i];
        }
#pragma unroll
        for (int u = 0; u < U; u++)
            ss[u] = (have[u] && skind != SK_NONE) ? scale_at(skind, sc, sc_ld, r0 + u * stride, cc[u]) : 1.0;
#pragma unroll
        for (int u = 0; u < U; u++)
            if (have[u] && !(skind != SK_NONE && ss[u] == 0.0)) {
                kept[u]++;
                acc[u] = combine(acc[u], skind != SK_NONE ? __dmul_rn(xx[u], ss[u]) : xx[u]);
            }
        // rows with more than G entries (a lock-step loop over the U rows was measured: more loads in flight per
        // thread, but 78 registers instead of 64 and no gain -- the pass is bound by the tag lookups of the gathers
        // in L1, one per distinct 128-byte line, not by their latency)
#pragma unroll
        for (int u = 0; u < U; u++)
            for (uint64_t i = b[u] + lane + G; i < e[u]; i += G) {
                const int64_t c = (int64_t)col[i];
                double x = UNIT ? 1.0 : val[i];
                if (skind != SK_NONE) {
                    const double s = scale_at(skind, sc, sc_ld, r0 + u * stride, c);
                    if (s == 0.0)
                        continue;
                    x = __dmul_rn(x, s);
                }
                kept[u]++;
                acc[u] = combine(acc[u], x);
            }
#pragma unroll
        for (int u = 0; u < U; u++) {
#pragma unroll
            for (int m = G / 2; m >= 1; m >>= 1) {
                acc[u] = combine(acc[u], shfl_xor(acc[u], m));
                kept[u] += __shfl_xor_sync(0xffffffffu, kept[u], m);
            }
            const int64_t r = r0 + u * stride;
            if (r < rows && lane == 0 && !deferred[u]) {
                double a = acc[u];
                if (op != DB2_AGG_SUM && kept[u] < cols) { // one implicit zero takes part (AggRow.h:167-176)
                    if (op == DB2_AGG_MAX)
                        a = (a < 0.0) ? 0.0 : a;
                    else if (op == DB2_AGG_MIN)
                        a = (0.0 < a) ? 0.0 : a;
                    else
                        a = __dmul_rn(a, 0.0);
                }
                emit(r, a, pre[u], E.pre_ptr != nullptr);
            }
        }
    }
    // the long rows, one after the other, by the whole block (fixed order of the partial results)
    __syncthreads();
    const int listed = n_long < MAX_LONG ? n_long : MAX_LONG;
    for (int q = 0; q < listed; q++) {
        const int64_t r = long_rows[q];
        const uint64_t rb = off[r], re = off[r + 1];
        double a = init;
        int k = 0;
        for (uint64_t i0 = rb + threadIdx.x; i0 < re; i0 += 4 * (uint64_t)blockDim.x) { // four entries in flight
            int64_t c4[4];
            double x4[4], s4[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint64_t i = i0 + (uint64_t)j * blockDim.x;
                c4[j] = i < re ? (int64_t)col[i] : -1;
                x4[j] = (UNIT || i >= re) ? 1.0 : val[i];
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
                s4[j] = (c4[j] >= 0 && skind != SK_NONE) ? scale_at(skind, sc, sc_ld, r, c4[j]) : 1.0;
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (c4[j] >= 0 && !(skind != SK_NONE && s4[j] == 0.0)) {
                    k++;
                    a = combine(a, skind != SK_NONE ? __dmul_rn(x4[j], s4[j]) : x4[j]);
                }
        }
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) {
            a = combine(a, shfl_xor(a, m));
            k += __shfl_xor_sync(0xffffffffu, k, m);
        }
        if (threadIdx.x % 32 == 0) {
            red_v[threadIdx.x / 32] = a;
            red_k[threadIdx.x / 32] = k;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < (int)blockDim.x / 32; w++) {
                a = combine(a, red_v[w]);
                k += red_k[w];
            }
            if (op != DB2_AGG_SUM && k < cols) { // one implicit zero takes part (AggRow.h:167-176)
                if (op == DB2_AGG_MAX)
                    a = (a < 0.0) ? 0.0 : a;
                else if (op == DB2_AGG_MIN)
                    a = (0.0 < a) ? 0.0 : a;
                else
                    a = __dmul_rn(a, 0.0);
            }
            emit(r, a, 0.0, false);
        }
        __syncthreads();
    }
    if (E.active && E.partials) {
        // block sum in a fixed order, then the last block to arrive folds the blocks' sums in block order
        __shared__ double wsum[8];
        __shared__ bool last;
        for (int d = 16; d >= 1; d >>= 1)
            local_sum = __dadd_rn(local_sum, shfl_down(local_sum, d));
        if (threadIdx.x % 32 == 0)
            wsum[threadIdx.x / 32] = local_sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < 8; w++)
                t = __dadd_rn(t, wsum[w]);
            E.partials[blockIdx.x] = t;
            __threadfence();
            last = atomicAdd(E.ticket, 1u) == gridDim.x - 1;
        }
        __syncthreads();
        if (last) { // thread t takes blocks t, t + 256, ...; then the same fixed tree as above
            __threadfence();
            double t = 0.0;
            for (unsigned b = threadIdx.x; b < gridDim.x; b += 256)
                t = __dadd_rn(t, __ldcg(E.partials + b));
            for (int d = 16; d >= 1; d >>= 1)
                t = __dadd_rn(t, shfl_down(t, d));
            __syncthreads();
            if (threadIdx.x % 32 == 0)
                wsum[threadIdx.x / 32] = t;
            __syncthreads();
            if (threadIdx.x == 0) {
                double tot = 0.0;
                for (int w = 0; w < 8; w++)
                    tot = __dadd_rn(tot, wsum[w]);
                *E.sum_out = tot;
                *E.ticket = 0;
            }
        }
    }
}

// materialisation of the product: kept entries per row, then an ordered fill
template <typename IT>
__global__ void csr_mul_count_kernel(const IT *__restrict__ col, const uint64_t *__restrict__ off, int64_t rows,
                                     int skind, const double *__restrict__ sc, int64_t sc_ld,
                                     uint64_t *__restrict__ counts) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
        uint64_t k = 0;
        for (uint64_t i = off[r]; i < off[r + 1]; i++)
            k += (scale_at(skind, sc, sc_ld, r, (int64_t)col[i]) != 0.0) ? 1 : 0;
        counts[r] = k;
    }
    if (blockIdx.x == 0 && threadIdx.x == 0)
        counts[rows] = 0;
}
template <typename IT>
__global__ void csr_mul_fill_kernel(const double *__restrict__ val, const IT *__restrict__ col,
                                    const uint64_t *__restrict__ off, int64_t rows, int skind,
                                    const double *__restrict__ sc, int64_t sc_ld, const uint64_t *__restrict__ new_off,
                                    double *__restrict__ oval, IT *__restrict__ ocol) {
    for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (int64_t)gridDim.x * blockDim.x) {
        uint64_t p = new_off[r];
        for (uint64_t i = off[r]; i < off[r + 1]; i++) {
            const double s = scale_at(skind, sc, sc_ld, r, (int64_t)col[i]);
            if (s != 0.0) {
                oval[p] = __dmul_rn(val[i], s);
                ocol[p] = col[i];
                p++;
            }
        }
    }
}

// res[r, :] = sum_i val[i] * B[col[i], :], entries in storage order (the reference's loop, Gemv.h:99-113): one warp
// per row, lanes over the dense columns
template <typename IT>
__global__ void __launch_bounds__(256)
    csr_spmm_kernel(const double *__restrict__ val, const IT *__restrict__ col, const uint64_t *__restrict__ off,
                    int64_t rows, const double *__restrict__ B, int64_t ldb, int64_t nc, double *__restrict__ out,
                    int64_t ldo) {
    const int lane = threadIdx.x % 32;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    const int64_t nwarps = (int64_t)gridDim.x * blockDim.x / 32;
    for (int64_t r = warp; r < rows; r += nwarps) {
        const uint64_t b = off[r], e = off[r + 1];
        for (int64_t j0 = 0; j0 < nc; j0 += 32) {
            const int64_t j = j0 + lane;
            double acc = 0.0;
            if (j < nc)
                for (uint64_t i = b; i < e; i++)
                    acc = __dadd_rn(acc, __dmul_rn(val[i], B[(int64_t)col[i] * ldb + j]));
            if (j < nc)
                out[r * ldo + j] = acc;
        }
    }
}

static int grid1d(int64_t n, int threads) {
    int64_t want = (n + threads - 1) / threads;
    const int64_t cap = (int64_t)sm_count() * 8;
    return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

static std::shared_ptr<DevBuf> devbuf(db2_context *ctx, size_t bytes) { return make_devbuf(ctx, bytes ? bytes : 16); }

// device placement of a host CSR (or of a deferred product)
static int csr_ensure_device(db2_csr *m);

static int scale_args(db2_csr *lhs, db2_matrix *rhs, int *skind, const double **sc, int64_t *ld) {
    DB2_TRY(ensure_device(rhs));
    if (rhs->rows == 1 && rhs->cols == lhs->cols && lhs->rows != 1)
        *skind = SK_ROWVEC;
    else if (rhs->cols == 1 && rhs->rows == lhs->rows && lhs->cols != 1)
        *skind = SK_COLVEC;
    else
        *skind = SK_MATRIX;
    if (rhs->rows == 1 && rhs->cols == 1) // 1 x 1 broadcasts both ways (rhs->get(0, 0) in the reference)
        *skind = SK_COLVEC;
    *sc = static_cast<const double *>(rhs->dev_ptr());
    *ld = (rhs->rows == 1 && rhs->cols == 1) ? 0 : rhs->dev_ld;
    return DB2_OK;
}

template <typename IT>
static int launch_agg(db2_context *ctx, int op, const db2_csr *m, int skind, const double *sc, int64_t ld,
                      double *out, const CsrEpi &epi, int *grid_out = nullptr) {
    const double *val = static_cast<const double *>(m->d_val->ptr);
    const IT *col = static_cast<const IT *>(m->d_col->ptr);
    const double avg = (double)m->nnz / (double)(m->rows > 0 ? m->rows : 1); // a view inherits its parent's count
    const int64_t rows = m->rows;
    // few lanes per row keep more rows in flight; rows far longer than the average are taken by whole blocks (see the
    // kernel), so a small group is safe on skewed graphs too
    const int lanes = avg <= 12.0 ? 2 : (avg <= 24.0 ? 4 : (avg <= 96.0 ? 8 : 32));
    // every lane group takes 4 rows per turn
    const int64_t want = (rows + (256 / lanes) * 4 - 1) / ((256 / lanes) * 4), cap = (int64_t)sm_count() * 8;
    const int grid = (int)(want < cap ? (want ? want : 1) : cap);
    if (grid_out) { // only the launch geometry is wanted (sizes the partial sums)
        *grid_out = grid;
        return DB2_OK;
    }
#define DB2_CSR_AGG3(G, UNIT, OP)                                                                                      \
    csr_agg_row_kernel<G, IT, UNIT, OP><<<grid, 256, 0, ctx->stream>>>(val, col, m->off_ptr(), rows, m->cols, skind,   \
                                                                       sc, ld, out, epi)
#define DB2_CSR_AGG2(G, UNIT)                                                                                          \
    switch (op) {                                                                                                      \
    case DB2_AGG_SUM: DB2_CSR_AGG3(G, UNIT, DB2_AGG_SUM); break;                                                       \
    case DB2_AGG_PROD: DB2_CSR_AGG3(G, UNIT, DB2_AGG_PROD); break;                                                     \
    case DB2_AGG_MIN: DB2_CSR_AGG3(G, UNIT, DB2_AGG_MIN); break;                                                       \
    default: DB2_CSR_AGG3(G, UNIT, DB2_AGG_MAX); break;                                                                \
    }
#define DB2_CSR_AGG(G)                                                                                                 \
    if (m->unit_vals) {                                                                                                \
        DB2_CSR_AGG2(G, true)                                                                                          \
    } else {                                                                                                           \
        DB2_CSR_AGG2(G, false)                                                                                         \
    }
    if (lanes == 2) {
        DB2_CSR_AGG(2)
    } else if (lanes == 4) {
        DB2_CSR_AGG(4)
    } else if (lanes == 8) {
        DB2_CSR_AGG(8)
    } else {
        DB2_CSR_AGG(32)
    }
#undef DB2_CSR_AGG
#undef DB2_CSR_AGG2
#undef DB2_CSR_AGG3
    return after_launch("csr_agg_row_kernel");
}

template <typename IT> static int materialise_product(db2_csr *m) {
    db2_context *ctx = m->ctx;
    db2_csr *lhs = m->lazy_lhs;
    DB2_TRY(csr_ensure_device(lhs));
    int skind;
    const double *sc;
    int64_t ld;
    DB2_TRY(scale_args(lhs, m->lazy_rhs, &skind, &sc, &ld));
    const int64_t rows = lhs->rows;
    auto counts = devbuf(ctx, (size_t)(rows + 1) * 8);
    auto offs = devbuf(ctx, (size_t)(rows + 1) * 8);
    const IT *col = static_cast<const IT *>(lhs->d_col->ptr);
    const double *val = static_cast<const double *>(lhs->d_val->ptr);
    csr_mul_count_kernel<IT><<<grid1d(rows, 256), 256, 0, ctx->stream>>>(col, lhs->off_ptr(), rows, skind, sc, ld,
                                                                       static_cast<uint64_t *>(counts->ptr));
    DB2_TRY(after_launch("csr_mul_count_kernel"));
    // row offsets = exclusive prefix sums of the counts: 0, then the cumulative sums (the blocked scan of AggCum)
    DB2_CUDA(cudaMemsetAsync(offs->ptr, 0, 8, ctx->stream));
    if (rows > 0) {
        const size_t tmp_bytes = db2k_agg_cum_scratch_bytes(rows, 1);
        auto tmp = devbuf(ctx, tmp_bytes);
        DB2_TRY(db2k_agg_cum(DB2_I64, DB2_AGG_SUM, counts->ptr, rows, 1, 1, static_cast<uint64_t *>(offs->ptr) + 1, 1,
                             tmp->ptr, tmp_bytes, ctx->stream));
    }
    uint64_t total = 0;
    DB2_CUDA(cudaMemcpyAsync(&total, static_cast<uint64_t *>(offs->ptr) + rows, 8, cudaMemcpyDeviceToHost,
                             ctx->stream));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    m->d_val = devbuf(ctx, (size_t)total * 8);
    m->d_col = devbuf(ctx, (size_t)total * sizeof(IT));
    m->d_off = offs;
    m->row0 = 0;
    m->nnz = (int64_t)total;
    m->idx32 = lhs->idx32;
    csr_mul_fill_kernel<IT><<<grid1d(rows, 256), 256, 0, ctx->stream>>>(
        val, col, lhs->off_ptr(), rows, skind, sc, ld, static_cast<const uint64_t *>(offs->ptr),
        static_cast<double *>(m->d_val->ptr), static_cast<IT *>(m->d_col->ptr));
    DB2_TRY(after_launch("csr_mul_fill_kernel"));
    m->dev_valid = true;
    return DB2_OK;
}

static void drop_lazy(db2_csr *m);

static int csr_ensure_device(db2_csr *m) {
    if (m->dev_valid)
        return DB2_OK;
    db2_context *ctx = m->ctx;
    bind_device(ctx);
    if (m->lazy_lhs) {
        DB2_TRY(csr_ensure_device(m->lazy_lhs));
        DB2_TRY(m->lazy_lhs->idx32 ? materialise_product<uint32_t>(m) : materialise_product<uint64_t>(m));
        drop_lazy(m);
        return DB2_OK;
    }
    DB2_CHECK(m->h_off != nullptr, DB2_EINVAL, "CSR matrix has no valid placement");
    // copy exactly the slice this handle covers and rebase nothing: offsets stay absolute, arrays are offset instead
    const uint64_t lo = m->h_off[0], hi = m->h_off[m->rows];
    const int64_t n = (int64_t)(hi - lo);
    m->idx32 = m->cols <= (int64_t)UINT32_MAX;
    {
        bool unit = n > 0;
        for (int64_t i = 0; i < n && unit; i++)
            unit = m->h_val[lo + i] == 1.0;
        m->unit_vals = unit;
    }
    m->d_val = devbuf(ctx, (size_t)n * 8);
    m->d_off = devbuf(ctx, (size_t)(m->rows + 1) * 8);
    auto wide = devbuf(ctx, (size_t)n * 8);
    DB2_CUDA(cudaMemcpyAsync(m->d_val->ptr, m->h_val + lo, (size_t)n * 8, cudaMemcpyHostToDevice, ctx->stream));
    DB2_CUDA(cudaMemcpyAsync(wide->ptr, m->h_col + lo, (size_t)n * 8, cudaMemcpyHostToDevice, ctx->stream));
    if (lo == 0) {
        DB2_CUDA(cudaMemcpyAsync(m->d_off->ptr, m->h_off, (size_t)(m->rows + 1) * 8, cudaMemcpyHostToDevice,
                                 ctx->stream));
    } else {
        std::vector<uint64_t> reb((size_t)m->rows + 1);
        for (int64_t i = 0; i <= m->rows; i++)
            reb[i] = m->h_off[i] - lo;
        DB2_CUDA(cudaMemcpyAsync(m->d_off->ptr, reb.data(), (size_t)(m->rows + 1) * 8, cudaMemcpyHostToDevice,
                                 ctx->stream));
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    if (m->idx32) {
        m->d_col = devbuf(ctx, (size_t)n * 4);
        if (n > 0) {
            narrow_idx_kernel<uint32_t><<<grid1d(n, 256), 256, 0, ctx->stream>>>(
                static_cast<const uint64_t *>(wide->ptr), static_cast<uint32_t *>(m->d_col->ptr), n);
            DB2_TRY(after_launch("narrow_idx_kernel"));
        }
    } else {
        m->d_col = wide;
    }
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.h2d_bytes += (uint64_t)n * 16 + (uint64_t)(m->rows + 1) * 8;
    }
    m->row0 = 0;
    m->nnz = n;
    m->dev_valid = true;
    return DB2_OK;
}

static void drop_lazy(db2_csr *m) {
    if (m->lazy_lhs) {
        db2_csr_decref(m->lazy_lhs);
        m->lazy_lhs = nullptr;
    }
    if (m->lazy_rhs) {
        db2_matrix_decref(m->lazy_rhs);
        m->lazy_rhs = nullptr;
    }
}

CsrSrc::CsrSrc(db2_csr *mm, int o) : m(mm), op(o) { db2_csr_incref(mm); }
CsrSrc::~CsrSrc() { db2_csr_decref(m); }

size_t csr_agg_scratch_bytes() { return (size_t)sm_count() * 8 * sizeof(double) + 64; }

int csr_agg_pass(db2_context *ctx, const CsrSrc &src, const FusedProgram &prog, double *mid_out, int mid_after,
                 double *sum_out, void *scratch, size_t scratch_bytes) {
    db2_csr *arg = src.m, *m = arg;
    int skind = SK_NONE;
    const double *sc = nullptr;
    int64_t ld = 0;
    if (arg->lazy_lhs && !arg->dev_valid) {
        m = arg->lazy_lhs;
        DB2_TRY(scale_args(m, arg->lazy_rhs, &skind, &sc, &ld));
    }
    DB2_TRY(csr_ensure_device(m));
    if (arg->rows == 0) {
        if (sum_out)
            DB2_CUDA(cudaMemsetAsync(sum_out, 0, sizeof(double), ctx->stream));
        return DB2_OK;
    }
    CsrEpi E;
    memset(&E, 0, sizeof(E));
    E.active = 1;
    E.nsteps = prog.nsteps;
    E.mid_out = mid_out;
    E.mid_after = mid_after;
    E.ew_out = static_cast<double *>(prog.ew_out);
    for (int i = 0; i < prog.nsteps; i++) {
        E.steps[i] = prog.steps[i];
        if (!E.pre_ptr && (prog.steps[i].kind == FK_MATRIX || prog.steps[i].kind == FK_COLVEC)) {
            E.pre_ptr = static_cast<const double *>(prog.steps[i].ptr);
            E.pre_ld = prog.steps[i].ld;
        }
    }
    if (sum_out) {
        int grid = 0;
        DB2_TRY(m->idx32 ? launch_agg<uint32_t>(ctx, src.op, m, skind, sc, ld, nullptr, E, &grid)
                         : launch_agg<uint64_t>(ctx, src.op, m, skind, sc, ld, nullptr, E, &grid));
        DB2_CHECK(scratch && scratch_bytes >= (size_t)grid * sizeof(double), DB2_EINVAL, "CSR pass scratch too small");
        E.partials = static_cast<double *>(scratch);
        E.sum_out = sum_out;
        E.ticket = reinterpret_cast<unsigned int *>(ctx->dev_status + 32); // zero between launches
    }
    return m->idx32 ? launch_agg<uint32_t>(ctx, src.op, m, skind, sc, ld, nullptr, E)
                    : launch_agg<uint64_t>(ctx, src.op, m, skind, sc, ld, nullptr, E);
}

} // namespace db2

using namespace db2;

extern "C" {

int db2_csr_wrap_host(db2_context *ctx, int dtype, int64_t rows, int64_t cols, const void *values,
                      const uint64_t *col_idx, const uint64_t *row_off, db2_csr **out) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && out && row_off, DB2_EINVAL, "null argument");
    DB2_CHECK(dtype == DB2_F64, DB2_EUNSUPPORTED, "CSR matrices: only double on the device");
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    std::unique_ptr<db2_csr> m(new db2_csr());
    m->ctx = ctx;
    m->rows = rows;
    m->cols = cols;
    m->h_val = static_cast<const double *>(values);
    m->h_col = col_idx;
    m->h_off = row_off;
    m->nnz = (int64_t)(row_off[rows] - row_off[0]);
    DB2_CHECK((values && col_idx) || m->nnz == 0, DB2_EINVAL, "null value/index array");
    *out = m.release();
    return DB2_OK;
    DB2_API_END
}

int db2_csr_slice_rows(db2_csr *src, int64_t r0, int64_t r1, db2_csr **view) {
    DB2_API_BEGIN
    DB2_CHECK(src && view, DB2_EINVAL, "null argument");
    // bounds checks of the reference's view constructor (CSRMatrix.h:131-148)
    DB2_CHECK(r0 < src->rows, DB2_EINVAL, "CSRMatrix: rowLowerIncl is out of bounds");
    DB2_CHECK(r1 <= src->rows, DB2_EINVAL, "CSRMatrix: rowUpperExcl is out of bounds");
    DB2_CHECK(r0 < r1 && r0 >= 0, DB2_EINVAL, "CSRMatrix: rowLowerIncl must be lower than rowUpperExcl");
    std::unique_ptr<db2_csr> m(new db2_csr());
    m->ctx = src->ctx;
    m->rows = r1 - r0;
    m->cols = src->cols;
    if (src->lazy_lhs || src->dev_valid) {
        DB2_TRY(csr_ensure_device(src));
        m->d_val = src->d_val;
        m->d_col = src->d_col;
        m->d_off = src->d_off;
        m->idx32 = src->idx32;
        m->unit_vals = src->unit_vals;
        m->row0 = src->row0 + r0;
        m->nnz = src->nnz;
        m->dev_valid = true;
    } else {
        m->h_val = src->h_val;
        m->h_col = src->h_col;
        m->h_off = src->h_off + r0;
        m->nnz = (int64_t)(m->h_off[m->rows] - m->h_off[0]);
    }
    *view = m.release();
    return DB2_OK;
    DB2_API_END
}

int db2_csr_incref(db2_csr *m) {
    DB2_CHECK(m, DB2_EINVAL, "null matrix");
    m->refs.fetch_add(1);
    return DB2_OK;
}
int db2_csr_decref(db2_csr *m) {
    if (!m)
        return DB2_OK;
    if (m->refs.fetch_sub(1) == 1) {
        drop_lazy(m);
        delete m;
    }
    return DB2_OK;
}
int db2_csr_info(db2_csr *m, int64_t *rows, int64_t *cols, int64_t *nnz) {
    DB2_API_BEGIN
    DB2_CHECK(m, DB2_EINVAL, "null matrix");
    if (rows)
        *rows = m->rows;
    if (cols)
        *cols = m->cols;
    if (nnz) {
        if (m->lazy_lhs)
            DB2_TRY(csr_ensure_device(m));
        if (m->h_off && !m->dev_valid) {
            *nnz = (int64_t)(m->h_off[m->rows] - m->h_off[0]);
        } else {
            uint64_t be[2];
            DB2_CUDA(cudaMemcpyAsync(&be[0], m->off_ptr(), 8, cudaMemcpyDeviceToHost, m->ctx->stream));
            DB2_CUDA(cudaMemcpyAsync(&be[1], m->off_ptr() + m->rows, 8, cudaMemcpyDeviceToHost, m->ctx->stream));
            DB2_CUDA(cudaStreamSynchronize(m->ctx->stream));
            *nnz = (int64_t)(be[1] - be[0]);
        }
    }
    return DB2_OK;
    DB2_API_END
}

// copies the matrix out in the reference's layout (row offsets rebased to 0); values/col_idx hold db2_csr_info's nnz
int db2_csr_to_host(db2_csr *m, void *values, uint64_t *col_idx, uint64_t *row_off) {
    DB2_API_BEGIN
    DB2_CHECK(m && row_off, DB2_EINVAL, "null argument");
    db2_context *ctx = m->ctx;
    DB2_TRY(csr_ensure_device(m));
    bind_device(ctx);
    DB2_CUDA(cudaMemcpyAsync(row_off, m->off_ptr(), (size_t)(m->rows + 1) * 8, cudaMemcpyDeviceToHost, ctx->stream));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    const uint64_t lo = row_off[0], hi = row_off[m->rows];
    const int64_t n = (int64_t)(hi - lo);
    for (int64_t i = 0; i <= m->rows; i++)
        row_off[i] -= lo;
    if (n > 0) {
        DB2_CHECK(values && col_idx, DB2_EINVAL, "null value/index array");
        DB2_CUDA(cudaMemcpyAsync(values, static_cast<const double *>(m->d_val->ptr) + lo, (size_t)n * 8,
                                 cudaMemcpyDeviceToHost, ctx->stream));
        if (m->idx32) {
            auto wide = devbuf(ctx, (size_t)n * 8);
            widen_idx_kernel<uint32_t><<<grid1d(n, 256), 256, 0, ctx->stream>>>(
                static_cast<const uint32_t *>(m->d_col->ptr) + lo, static_cast<uint64_t *>(wide->ptr), n);
            DB2_TRY(after_launch("widen_idx_kernel"));
            DB2_CUDA(cudaMemcpyAsync(col_idx, wide->ptr, (size_t)n * 8, cudaMemcpyDeviceToHost, ctx->stream));
            DB2_CUDA(cudaStreamSynchronize(ctx->stream));
        } else {
            DB2_CUDA(cudaMemcpyAsync(col_idx, static_cast<const uint64_t *>(m->d_col->ptr) + lo, (size_t)n * 8,
                                     cudaMemcpyDeviceToHost, ctx->stream));
            DB2_CUDA(cudaStreamSynchronize(ctx->stream));
        }
    }
    return DB2_OK;
    DB2_API_END
}

int db2_ewMulCsrDense(db2_context *ctx, db2_csr **res, db2_csr *lhs, db2_matrix *rhs) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && lhs && rhs, DB2_EINVAL, "null argument");
    DB2_CHECK(rhs->dtype == DB2_F64, DB2_EUNSUPPORTED, "EwBinaryMat(CSR): only double on the device");
    // shape rule of EwBinaryMat.h:259-263
    DB2_CHECK(!((lhs->rows != rhs->rows && rhs->rows != 1) || (lhs->cols != rhs->cols && rhs->cols != 1)), DB2_EINVAL,
              "EwBinaryMat(CSR) - lhs and rhs must have the same dimensions (or broadcast)");
    std::unique_ptr<db2_csr> m(new db2_csr());
    m->ctx = ctx;
    m->rows = lhs->rows;
    m->cols = lhs->cols;
    m->nnz = lhs->nnz;
    m->lazy_lhs = lhs;
    m->lazy_rhs = rhs;
    db2_csr_incref(lhs);
    db2_matrix_incref(rhs);
    if (ctx->eager) {
        DB2_TRY(csr_ensure_device(m.get()));
    }
    *res = m.release();
    return DB2_OK;
    DB2_API_END
}

int db2_aggRowCsr(db2_context *ctx, int op, db2_matrix **res, db2_csr *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    DB2_CHECK(op == DB2_AGG_SUM || op == DB2_AGG_PROD || op == DB2_AGG_MIN || op == DB2_AGG_MAX, DB2_EUNSUPPORTED,
              "aggRow(CSR): SUM, PROD, MIN and MAX are implemented on the device");
    bind_device(ctx);
    {
        bool handled = false;
        DB2_TRY(lazy_try_agg_row_csr(ctx, op, res, arg, &handled));
        if (handled)
            return DB2_OK;
    }
    const uint64_t before = g_launches.load();
    db2_csr *src = arg;
    int skind = SK_NONE;
    const double *sc = nullptr;
    int64_t ld = 0;
    if (arg->lazy_lhs && !arg->dev_valid) {
        src = arg->lazy_lhs;
        DB2_TRY(scale_args(src, arg->lazy_rhs, &skind, &sc, &ld));
    }
    DB2_TRY(csr_ensure_device(src));
    DB2_TRY(prepare_result(ctx, res, DB2_F64, arg->rows, 1));
    DB2_CHECK((*res)->dev_ld == 1, DB2_EUNSUPPORTED, "aggRow(CSR) into a strided result view");
    double *out = static_cast<double *>((*res)->dev_ptr());
    CsrEpi none;
    memset(&none, 0, sizeof(none));
    if (arg->rows > 0)
        DB2_TRY(src->idx32 ? launch_agg<uint32_t>(ctx, op, src, skind, sc, ld, out, none)
                           : launch_agg<uint64_t>(ctx, op, src, skind, sc, ld, out, none));
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load() - before;
    return DB2_OK;
    DB2_API_END
}

// res = lhs @ rhs for a CSR lhs and a dense rhs (MatMul<Dense,CSR,Dense> / Gemv<Dense,CSR,Dense>, Gemv.h:79-117)
int db2_matMulCsrDense(db2_context *ctx, db2_matrix **res, db2_csr *lhs, db2_matrix *rhs) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && lhs && rhs, DB2_EINVAL, "null argument");
    DB2_CHECK(rhs->dtype == DB2_F64, DB2_EUNSUPPORTED, "matMul(CSR, dense): only double on the device");
    DB2_CHECK(lhs->cols == rhs->rows, DB2_EINVAL, "Gemv - #cols of mat and #rows of vec must be the same");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(csr_ensure_device(lhs));
    DB2_TRY(ensure_device(rhs));
    DB2_TRY(prepare_result(ctx, res, DB2_F64, lhs->rows, rhs->cols));
    db2_matrix *r = *res;
    if (lhs->rows > 0 && rhs->cols > 0) {
        const int64_t want = (lhs->rows + 7) / 8, cap = (int64_t)sm_count() * 8;
        const int grid = (int)(want < cap ? want : cap);
        const double *val = static_cast<const double *>(lhs->d_val->ptr);
        if (lhs->idx32)
            csr_spmm_kernel<uint32_t><<<grid, 256, 0, ctx->stream>>>(
                val, static_cast<const uint32_t *>(lhs->d_col->ptr), lhs->off_ptr(), lhs->rows,
                static_cast<const double *>(rhs->dev_ptr()), rhs->dev_ld, rhs->cols,
                static_cast<double *>(r->dev_ptr()), r->dev_ld);
        else
            csr_spmm_kernel<uint64_t><<<grid, 256, 0, ctx->stream>>>(
                val, static_cast<const uint64_t *>(lhs->d_col->ptr), lhs->off_ptr(), lhs->rows,
                static_cast<const double *>(rhs->dev_ptr()), rhs->dev_ld, rhs->cols,
                static_cast<double *>(r->dev_ptr()), r->dev_ld);
        DB2_TRY(after_launch("csr_spmm_kernel"));
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load() - before;
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
