// Kernels that evaluate a deferred elementwise chain inside a consumer (see fused.cuh).
//
// Row pass (materialisation and/or up to FUSED_MAX_AGGS row aggregations in one sweep):
//   a CTA of 128 threads stages a tile of 128 rows x 32 columns in shared memory with coalesced 128-bit loads
//   (16 loads in flight per thread), then every thread walks ONE row of the tile (row pitch 33 doubles: conflict
//   free), evaluates the chain on 8 values at a time (one interpreter dispatch per step and 8 values) and feeds the
//   row trackers, so no cross-lane reduction is needed at all; results are written one row per thread (coalesced).
//   HBM traffic = every base element once + 8 or 16 bytes per row and aggregation.
// Column pass: threadIdx.x owns a packet of columns, threadIdx.y strides over rows (the mapping of agg.cu), the chain
//   is evaluated on the packet right after its load; per-CTA partials are folded by agg.cu's second stage.
//
// Division by a broadcast divisor (row vector or scalar) is the one expensive FP64 operation of the standardisation
// pipeline (B200 issues 64 FP64 instructions per SM and clock, a generic IEEE division costs about 20 of them), so it
// is computed from the divisor's correctly rounded reciprocal y = RN(1/d), staged once per column:
//   q = RN(a*y); r = a - q*d (exact, FMA); result = RN(q + r*y),
// which is the correctly rounded quotient a/d when nothing over/underflows (Markstein's theorem).  Operands outside
// a conservative exponent window, zeros, infinities, NaNs and divisors whose significand is all ones take the
// generic IEEE division instead, so the result always has the bits of a/d.
#include "fused.cuh"
#include "fused_step.cuh"
#include "ops.cuh"

namespace db2 {

constexpr int RT = 128;          // threads per CTA = rows per tile
constexpr int CK = 32;           // columns per chunk
constexpr int PITCH = CK + 1;    // doubles per tile row in shared memory
constexpr int GV = 8;            // values per interpreter dispatch
constexpr int NO_COL = 0x7fffffff;

// One row tracker per tap: running value, column of the extremum, "first element was NaN".
struct RowTracker {
    double v;
    int c;
    bool first_nan;
};
__device__ __forceinline__ void tracker_init(RowTracker &t, int kind) {
    t.c = NO_COL;
    t.first_nan = false;
    switch (kind) {
    case FT_PROD: t.v = 1.0; break;
    case FT_MIN: t.v = INFINITY; break;
    case FT_MAX: t.v = -INFINITY; break;
    default: t.v = 0.0; break;
    }
}
template <int N>
__device__ __forceinline__ void tracker_feed(RowTracker &t, int op, const double (&v)[N], int c0, int nv) {
    switch (op) {
    case FT_SUM:
    case FT_MEAN:
#pragma unroll
        for (int i = 0; i < N; i++)
            if (i < nv)
                t.v = __dadd_rn(t.v, v[i]);
        break;
    case FT_PROD:
#pragma unroll
        for (int i = 0; i < N; i++)
            if (i < nv)
                t.v = __dmul_rn(t.v, v[i]);
        break;
    case FT_MIN:
        if (c0 == 0 && v[0] != v[0])
            t.first_nan = true;
#pragma unroll
        for (int i = 0; i < N; i++)
            if (i < nv && (v[i] < t.v || (t.c == NO_COL && v[i] == t.v))) {
                t.v = v[i];
                t.c = c0 + i;
            }
        break;
    case FT_MAX:
        if (c0 == 0 && v[0] != v[0])
            t.first_nan = true;
#pragma unroll
        for (int i = 0; i < N; i++)
            if (i < nv && (v[i] > t.v || (t.c == NO_COL && v[i] == t.v))) {
                t.v = v[i];
                t.c = c0 + i;
            }
        break;
    default: break;
    }
}

template <bool ALIGNED>
__global__ void __launch_bounds__(RT)
    fused_row_kernel(const __grid_constant__ FusedProgram P) {
    extern __shared__ __align__(16) double smem[];
    double *tile = smem;             // [RT][PITCH]
    double *rvs = smem + RT * PITCH; // staged row-vector operands (+ division helpers)
    const int tid = threadIdx.x;
    const int64_t rows = P.rows, cols = P.cols;

    // stage the row-vector operands once per CTA
    for (int s = 0; s < P.nsteps; s++) {
        const FusedStep &st = P.steps[s];
        if (st.kind == FK_ROWVEC && st.smem_off >= 0) {
            const double *src = static_cast<const double *>(st.ptr);
            const bool helper = (st.op == FO_DIV && !st.reversed);
            for (int64_t c = tid; c < cols; c += RT) {
                const double d = src[c];
                rvs[st.smem_off + c] = d;
                if (helper)
                    rvs[st.smem_off + ((cols + 1) & ~(int64_t)1) + c] = div_helper(d);
            }
        }
    }
    __syncthreads();

    const double *base = static_cast<const double *>(P.base);
    const int64_t ntiles = (rows + RT - 1) / RT;
    for (int64_t tile_i = blockIdx.x; tile_i < ntiles; tile_i += gridDim.x) {
        const int64_t row0 = tile_i * RT;
        const int64_t row = row0 + tid;
        const bool live = row < rows;
        const int64_t rows_here = (rows - row0 < RT) ? (rows - row0) : RT;
        RowTracker trk[FUSED_MAX_AGGS];
#pragma unroll
        for (int a = 0; a < FUSED_MAX_AGGS; a++)
            if (a < P.ntaps)
                tracker_init(trk[a], P.taps[a].kind);

        for (int64_t cc = 0; cc < cols; cc += CK) {
            const int cw = (cols - cc < CK) ? (int)(cols - cc) : CK;
            __syncthreads(); // the previous chunk's readers are done with the tile
            if (ALIGNED && cw == CK) {
                // 16 packets of 16 bytes per row, 128 rows: 16 coalesced loads in flight per thread
                Pack<double> p[CK / 2 * RT / RT];
#pragma unroll
                for (int i = 0; i < CK / 2; i++) {
                    const int idx = tid + i * RT;
                    const int r = idx >> 4, k = idx & 15;
                    if (r < rows_here)
                        p[i] = ld_pack_stream(base + (row0 + r) * P.base_ld + cc + 2 * k);
                    else
                        p[i].v[0] = p[i].v[1] = 0.0;
                }
#pragma unroll
                for (int i = 0; i < CK / 2; i++) {
                    const int idx = tid + i * RT;
                    const int r = idx >> 4, k = idx & 15;
                    tile[r * PITCH + 2 * k] = p[i].v[0];
                    tile[r * PITCH + 2 * k + 1] = p[i].v[1];
                }
            } else {
                for (int idx = tid; idx < RT * cw; idx += RT) {
                    const int r = idx / cw, k = idx - r * cw;
                    tile[r * PITCH + k] = (r < rows_here) ? base[(row0 + r) * P.base_ld + cc + k] : 0.0;
                }
            }
            __syncthreads();

            double *myrow = tile + tid * PITCH;
            for (int k0 = 0; k0 < cw; k0 += GV) {
                const int nv = (cw - k0 < GV) ? (cw - k0) : GV;
                const int64_t c0 = cc + k0;
                double v[GV];
#pragma unroll
                for (int i = 0; i < GV; i++)
                    v[i] = (i < nv) ? myrow[k0 + i] : 0.0;
#pragma unroll
                for (int a = 0; a < FUSED_MAX_AGGS; a++)
                    if (a < P.ntaps && P.taps[a].after_step == 0)
                        tracker_feed(trk[a], P.taps[a].kind, v, (int)c0, nv);
                for (int s = 0; s < P.nsteps; s++) {
                    const FusedStep &st = P.steps[s];
                    double o[GV], y[GV];
                    if (st.kind == FK_ROWVEC) {
                        if (st.smem_off >= 0) {
                            const double *sv = rvs + st.smem_off + c0;
#pragma unroll
                            for (int i = 0; i < GV; i++)
                                o[i] = (i < nv) ? sv[i] : 1.0;
                            if (st.op == FO_DIV && !st.reversed) {
#pragma unroll
                                for (int i = 0; i < GV; i++)
                                    y[i] = (i < nv) ? sv[((cols + 1) & ~(int64_t)1) + i] : 0.0;
                            }
                        } else {
                            const double *gv = static_cast<const double *>(st.ptr) + c0;
#pragma unroll
                            for (int i = 0; i < GV; i++) {
                                o[i] = (i < nv) ? __ldg(gv + i) : 1.0;
                                y[i] = 0.0;
                            }
                        }
                    } else if (st.kind == FK_SCALAR) {
                        const double yy = (st.op == FO_DIV && !st.reversed) ? div_helper(st.imm) : 0.0;
#pragma unroll
                        for (int i = 0; i < GV; i++) {
                            o[i] = st.imm;
                            y[i] = yy;
                        }
                    } else if (st.kind == FK_COLVEC) {
                        const double x = live ? __ldg(static_cast<const double *>(st.ptr) + row * st.ld) : 1.0;
#pragma unroll
                        for (int i = 0; i < GV; i++) {
                            o[i] = x;
                            y[i] = 0.0;
                        }
                    } else if (st.kind == FK_MATRIX) {
                        const double *mp = static_cast<const double *>(st.ptr) + (live ? row : 0) * st.ld + c0;
#pragma unroll
                        for (int i = 0; i < GV; i++) {
                            o[i] = (i < nv && live) ? __ldg(mp + i) : 1.0;
                            y[i] = 0.0;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < GV; i++) {
                            o[i] = 0.0;
                            y[i] = 0.0;
                        }
                    }
                    apply_step<GV>(st.op, st.reversed != 0, v, o, y);
#pragma unroll
                    for (int a = 0; a < FUSED_MAX_AGGS; a++)
                        if (a < P.ntaps && P.taps[a].after_step == s + 1)
                            tracker_feed(trk[a], P.taps[a].kind, v, (int)c0, nv);
                }
                if (P.ew_out) {
#pragma unroll
                    for (int i = 0; i < GV; i++)
                        if (i < nv)
                            myrow[k0 + i] = v[i];
                }
            }
            if (P.ew_out) {
                __syncthreads();
                double *out = static_cast<double *>(P.ew_out);
                const bool out_vec = ALIGNED && cw == CK && ((P.ew_out_ld & 1) == 0) &&
                                     ((reinterpret_cast<uintptr_t>(out) & 15u) == 0);
                if (out_vec) {
#pragma unroll
                    for (int i = 0; i < CK / 2; i++) {
                        const int idx = tid + i * RT;
                        const int r = idx >> 4, k = idx & 15;
                        if (r < rows_here) {
                            Pack<double> q;
                            q.v[0] = tile[r * PITCH + 2 * k];
                            q.v[1] = tile[r * PITCH + 2 * k + 1];
                            st_pack_stream(out + (row0 + r) * P.ew_out_ld + cc + 2 * k, q);
                        }
                    }
                } else {
                    for (int idx = tid; idx < RT * cw; idx += RT) {
                        const int r = idx / cw, k = idx - r * cw;
                        if (r < rows_here)
                            out[(row0 + r) * P.ew_out_ld + cc + k] = tile[r * PITCH + k];
                    }
                }
            }
        }
        // one row per thread: results of consecutive rows are written by consecutive threads
        if (live) {
#pragma unroll
            for (int a = 0; a < FUSED_MAX_AGGS; a++) {
                if (a < P.ntaps) {
                    const FusedTap &tp = P.taps[a];
                    RowTracker t = trk[a];
                    if ((tp.kind == FT_MIN || tp.kind == FT_MAX) && (t.first_nan || t.c == NO_COL)) {
                        t.v = NAN; // only reachable when the first element is NaN (or every element is)
                        t.c = 0;
                    }
                    if (tp.out_idx)
                        static_cast<uint64_t *>(tp.out_idx)[row] = (uint64_t)t.c;
                    if (tp.out)
                        static_cast<double *>(tp.out)[row] =
                            (tp.kind == FT_MEAN) ? __ddiv_rn(t.v, (double)cols) : t.v;
                }
            }
        }
    }
}

int fused_row_pass_f64(const FusedProgram &prog, cudaStream_t st) {
    if (prog.rows == 0 || prog.cols == 0)
        return DB2_OK;
    const size_t smem = (size_t)(RT * PITCH + prog.smem_elems) * sizeof(double);
    bool aligned = aligned16(prog.base) && (prog.base_ld % 2 == 0);
    const int64_t ntiles = (prog.rows + RT - 1) / RT;
    // resident CTAs per SM are bounded by shared memory (about 34 KB each) and registers; 6 is a safe upper bound
    const int64_t cap = (int64_t)sm_count() * 6;
    const int grid = (int)(ntiles < cap ? ntiles : cap);
    static PerDeviceOnce attr_set[2];
    if (smem > 48 * 1024 && attr_set[aligned].need()) {
        if (aligned)
            DB2_CUDA(cudaFuncSetAttribute(fused_row_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          100 * 1024));
        else
            DB2_CUDA(cudaFuncSetAttribute(fused_row_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          100 * 1024));
        attr_set[aligned].mark();
    }
    if (aligned)
        fused_row_kernel<true><<<grid, RT, smem, st>>>(prog);
    else
        fused_row_kernel<false><<<grid, RT, smem, st>>>(prog);
    return after_launch("fused_row_kernel");
}

// ---------------------------------------------------------------------------
// flat pass: chains on column vectors (rows x 1) or on contiguous same-shape operands, one element at a time
// ---------------------------------------------------------------------------
// The row pass gives every thread one ROW, which for an n x 1 vector means one element per thread and 128 elements
// per CTA tile.  Such chains (connected components: u = max(rowMaxs(G * t(c)), c); sum(u != c)) are evaluated here
// over the n elements directly, 4 per thread and iteration.  Optional outputs of one pass: the final values
// (prog.ew_out), the values after `mid_after` steps (mid_out: a deferred matrix whose chain is a prefix), and the sum
// of the final values (per-CTA partials, added up in a fixed order by flat_sum_final_kernel).
constexpr int FLAT_THREADS = 256, FLAT_GV = 4;

bool fused_flat_eligible(const FusedProgram &P) {
    if (P.ntaps != 0)
        return false;
    if (P.cols == 1)
        return true;
    if (P.base_ld != P.cols)
        return false;
    for (int s = 0; s < P.nsteps; s++) {
        const int k = P.steps[s].kind;
        if (k == FK_ROWVEC || k == FK_COLVEC || (k == FK_MATRIX && P.steps[s].ld != P.cols))
            return false;
    }
    return true;
}

__global__ void __launch_bounds__(FLAT_THREADS)
    fused_flat_kernel(const __grid_constant__ FusedProgram P, int64_t n, int64_t stride_scale, double *mid_out,
                      int mid_after, double *partials) {
    // element i of an operand with leading dimension ld sits at i * ld for a column vector (stride_scale = 1) and at
    // i for a contiguous matrix (stride_scale = 0)
    const int64_t base_st = stride_scale ? P.base_ld : 1;
    const double *__restrict__ base = static_cast<const double *>(P.base);
    double *__restrict__ ew_out = static_cast<double *>(P.ew_out);
    const int64_t out_st = stride_scale ? P.ew_out_ld : 1;
    double sum = 0.0;
    for (int64_t i0 = ((int64_t)blockIdx.x * FLAT_THREADS + threadIdx.x) * FLAT_GV; i0 < n;
         i0 += (int64_t)gridDim.x * FLAT_THREADS * FLAT_GV) {
        const int nv = (n - i0) < FLAT_GV ? (int)(n - i0) : FLAT_GV;
        double v[FLAT_GV], o[FLAT_GV], y[FLAT_GV];
#pragma unroll
        for (int k = 0; k < FLAT_GV; k++)
            v[k] = k < nv ? base[(i0 + k) * base_st] : 0.0;
        if (mid_out && mid_after == 0) {
#pragma unroll
            for (int k = 0; k < FLAT_GV; k++)
                if (k < nv)
                    mid_out[i0 + k] = v[k];
        }
        for (int s = 0; s < P.nsteps; s++) {
            const FusedStep &st = P.steps[s];
            if (st.kind == FK_MATRIX || st.kind == FK_COLVEC) {
                const double *__restrict__ op = static_cast<const double *>(st.ptr);
                const int64_t op_st = stride_scale ? st.ld : 1;
#pragma unroll
                for (int k = 0; k < FLAT_GV; k++)
                    o[k] = k < nv ? op[(i0 + k) * op_st] : 1.0;
            } else {
                const double b = st.kind == FK_ROWVEC ? *static_cast<const double *>(st.ptr) : st.imm;
#pragma unroll
                for (int k = 0; k < FLAT_GV; k++)
                    o[k] = b;
            }
            const bool div = st.op == FO_DIV && !st.reversed;
#pragma unroll
            for (int k = 0; k < FLAT_GV; k++)
                y[k] = div ? div_helper(o[k]) : 0.0;
            apply_step<FLAT_GV>(st.op, st.reversed != 0, v, o, y);
            if (mid_out && mid_after == s + 1) {
#pragma unroll
                for (int k = 0; k < FLAT_GV; k++)
                    if (k < nv)
                        mid_out[i0 + k] = v[k];
            }
        }
        if (ew_out) {
#pragma unroll
            for (int k = 0; k < FLAT_GV; k++)
                if (k < nv)
                    ew_out[(i0 + k) * out_st] = v[k];
        }
#pragma unroll
        for (int k = 0; k < FLAT_GV; k++)
            if (k < nv)
                sum = __dadd_rn(sum, v[k]);
    }
    if (partials) {
        __shared__ double wsum[FLAT_THREADS / 32];
        for (int d = 16; d >= 1; d >>= 1)
            sum = __dadd_rn(sum, shfl_down(sum, d));
        if (threadIdx.x % 32 == 0)
            wsum[threadIdx.x / 32] = sum;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0.0;
            for (int w = 0; w < FLAT_THREADS / 32; w++)
                t = __dadd_rn(t, wsum[w]);
            partials[blockIdx.x] = t;
        }
    }
}

__global__ void flat_sum_final_kernel(const double *__restrict__ partials, int n, double *__restrict__ out) {
    __shared__ double sh[256];
    double t = 0.0;
    for (int i = threadIdx.x; i < n; i += 256)
        t = __dadd_rn(t, partials[i]);
    sh[threadIdx.x] = t;
    __syncthreads();
    for (int d = 128; d >= 1; d >>= 1) {
        if ((int)threadIdx.x < d)
            sh[threadIdx.x] = __dadd_rn(sh[threadIdx.x], sh[threadIdx.x + d]);
        __syncthreads();
    }
    if (threadIdx.x == 0)
        *out = sh[0];
}

size_t fused_flat_scratch_bytes() { return ((size_t)sm_count() * 8 + 8) * sizeof(double); }

// sum_out (device, may be null): sum of the final values; scratch holds the per-CTA partials behind it
int fused_flat_pass_f64(const FusedProgram &prog, void *mid_out, int mid_after, double *sum_out, void *scratch,
                        size_t scratch_bytes, cudaStream_t st) {
    const int64_t n = prog.rows * prog.cols;
    if (n == 0) {
        if (sum_out)
            DB2_CUDA(cudaMemsetAsync(sum_out, 0, sizeof(double), st));
        return DB2_OK;
    }
    int64_t grid = (n + FLAT_THREADS * FLAT_GV - 1) / (FLAT_THREADS * FLAT_GV);
    const int64_t cap = (int64_t)sm_count() * 8;
    grid = grid < cap ? grid : cap;
    DB2_CHECK(!sum_out || (scratch && scratch_bytes >= (size_t)grid * sizeof(double)), DB2_EINVAL,
              "flat pass scratch too small");
    fused_flat_kernel<<<(unsigned)grid, FLAT_THREADS, 0, st>>>(prog, n, prog.cols == 1 ? 1 : 0,
                                                             static_cast<double *>(mid_out), mid_after,
                                                             sum_out ? static_cast<double *>(scratch) : nullptr);
    DB2_TRY(after_launch("fused_flat_kernel"));
    if (sum_out) {
        flat_sum_final_kernel<<<1, 256, 0, st>>>(static_cast<const double *>(scratch), (int)grid, sum_out);
        DB2_TRY(after_launch("flat_sum_final_kernel"));
    }
    return DB2_OK;
}

// ---------------------------------------------------------------------------
// column pass
// ---------------------------------------------------------------------------
constexpr int CT = 256;
enum { CK_SUM = 0, CK_PROD = 1, CK_MIN = 2, CK_MAX = 3 };
constexpr int64_t POS_NONE = INT64_MAX; // no element seen yet
constexpr int64_t POS_FIRST_NAN = -1;   // row 0 holds a NaN: the sequential scan of the reference never leaves it

// does candidate (b at row q) replace the current extremum (a at row p)?  Lowest row wins ties.
template <int KIND> __device__ __forceinline__ bool col_better(double b, int64_t q, double a, int64_t p) {
    if (q == POS_NONE || p == POS_FIRST_NAN)
        return false;
    if (p == POS_NONE || q == POS_FIRST_NAN)
        return true;
    return (KIND == CK_MIN) ? (b < a || (b == a && q < p)) : (b > a || (b == a && q < p));
}

template <int KIND>
__global__ void __launch_bounds__(CT)
    fused_col_kernel(const __grid_constant__ FusedProgram P, double *__restrict__ part_v,
                     int64_t *__restrict__ part_i) {
    extern __shared__ __align__(16) double csm[];
    if (P.run_if && *P.run_if == 0)
        return;
    double *sv = csm;                                          // [TY][TX*2]
    int64_t *si = reinterpret_cast<int64_t *>(csm + CT * 2);   // same shape
    const int tx = threadIdx.x, ty = threadIdx.y, TX = blockDim.x, TY = blockDim.y;
    const int64_t rows = P.rows, cols = P.cols;
    const int64_t c0 = ((int64_t)blockIdx.y * TX + tx) * 2;
    const int nv = (c0 + 2 <= cols) ? 2 : ((c0 < cols) ? 1 : 0);
    double acc[2];
    int64_t pos[2];
#pragma unroll
    for (int k = 0; k < 2; k++) {
        acc[k] = (KIND == CK_SUM) ? 0.0 : (KIND == CK_PROD) ? 1.0 : (KIND == CK_MIN) ? INFINITY : -INFINITY;
        pos[k] = POS_NONE;
    }
    const double *base = static_cast<const double *>(P.base);
    const bool vec = (P.base_ld % 2 == 0) && aligned16(base) && nv == 2;
    if (nv > 0) {
        // row-vector operands are invariant per thread (fixed columns): fetched through L1 on every use
        const int64_t row_stride = (int64_t)gridDim.x * TY;
        for (int64_t r = (int64_t)blockIdx.x * TY + ty; r < rows; r += row_stride) {
            double v[2];
            if (vec) {
                const Pack<double> p = ld_pack_stream(base + r * P.base_ld + c0);
                v[0] = p.v[0];
                v[1] = p.v[1];
            } else {
                v[0] = base[r * P.base_ld + c0];
                v[1] = (nv == 2) ? base[r * P.base_ld + c0 + 1] : 0.0;
            }
            for (int s = 0; s < P.nsteps; s++) {
                const FusedStep &st = P.steps[s];
                double o[2], y[2];
                if (st.kind == FK_ROWVEC) {
                    const double *gv = static_cast<const double *>(st.ptr) + c0;
                    o[0] = __ldg(gv);
                    o[1] = (nv == 2) ? __ldg(gv + 1) : 1.0;
                    if (st.op == FO_DIV && !st.reversed) {
                        y[0] = div_helper(o[0]);
                        y[1] = div_helper(o[1]);
                    } else
                        y[0] = y[1] = 0.0;
                } else if (st.kind == FK_SCALAR) {
                    o[0] = o[1] = st.imm;
                    y[0] = y[1] = (st.op == FO_DIV && !st.reversed) ? div_helper(st.imm) : 0.0;
                } else if (st.kind == FK_COLVEC) {
                    o[0] = o[1] = __ldg(static_cast<const double *>(st.ptr) + r * st.ld);
                    y[0] = y[1] = 0.0;
                } else if (st.kind == FK_MATRIX) {
                    const double *mp = static_cast<const double *>(st.ptr) + r * st.ld + c0;
                    o[0] = __ldg(mp);
                    o[1] = (nv == 2) ? __ldg(mp + 1) : 1.0;
                    y[0] = y[1] = 0.0;
                } else {
                    o[0] = o[1] = y[0] = y[1] = 0.0;
                }
                apply_step<2>(st.op, st.reversed != 0, v, o, y);
            }
#pragma unroll
            for (int k = 0; k < 2; k++) {
                if (KIND == CK_SUM)
                    acc[k] = __dadd_rn(acc[k], v[k]);
                else if (KIND == CK_PROD)
                    acc[k] = __dmul_rn(acc[k], v[k]);
                else {
                    if (r == 0 && v[k] != v[k]) {
                        acc[k] = v[k];
                        pos[k] = POS_FIRST_NAN;
                    } else if (v[k] == v[k] && col_better<KIND>(v[k], r, acc[k], pos[k])) {
                        acc[k] = v[k];
                        pos[k] = r;
                    }
                }
            }
        }
    }
#pragma unroll
    for (int k = 0; k < 2; k++) {
        sv[(ty * TX + tx) * 2 + k] = acc[k];
        si[(ty * TX + tx) * 2 + k] = pos[k];
    }
    __syncthreads();
    for (int k = ty; k < 2; k += TY) {
        if (c0 + k < cols) {
            double a = sv[tx * 2 + k];
            int64_t p = si[tx * 2 + k];
            for (int yv = 1; yv < TY; yv++) {
                const double b = sv[(yv * TX + tx) * 2 + k];
                const int64_t q = si[(yv * TX + tx) * 2 + k];
                if (KIND == CK_SUM)
                    a = __dadd_rn(a, b);
                else if (KIND == CK_PROD)
                    a = __dmul_rn(a, b);
                else if (col_better<KIND>(b, q, a, p)) {
                    a = b;
                    p = q;
                }
            }
            part_v[(int64_t)blockIdx.x * cols + c0 + k] = a;
            part_i[(int64_t)blockIdx.x * cols + c0 + k] = p;
        }
    }
}

// second stage for the chain column pass: folds the per-CTA partials in order and applies the epilogue
template <int KIND>
__global__ void fused_col_final_kernel(const double *__restrict__ part_v, const int64_t *__restrict__ part_i,
                                       int nparts, int64_t cols, int64_t count, int out_mode, void *__restrict__ res,
                                       const int32_t *__restrict__ run_if) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols || (run_if && *run_if == 0))
        return;
    double a = part_v[c];
    int64_t p = part_i[c];
    for (int i = 1; i < nparts; i++) {
        const double b = part_v[(int64_t)i * cols + c];
        const int64_t q = part_i[(int64_t)i * cols + c];
        if (KIND == CK_SUM)
            a = __dadd_rn(a, b);
        else if (KIND == CK_PROD)
            a = __dmul_rn(a, b);
        else if (col_better<KIND>(b, q, a, p)) {
            a = b;
            p = q;
        }
    }
    if (out_mode == 1)
        static_cast<uint64_t *>(res)[c] = (p == POS_NONE || p == POS_FIRST_NAN) ? 0 : (uint64_t)p;
    else if (out_mode == 2)
        static_cast<double *>(res)[c] = __ddiv_rn(a, (double)count);
    else
        static_cast<double *>(res)[c] = ((KIND == CK_MIN || KIND == CK_MAX) && p == POS_NONE) ? (double)NAN : a;
}

size_t fused_col_scratch_bytes(int64_t cols) { return (size_t)sm_count() * 8 * cols * 16 + 256; }

template <int KIND>
static int fused_col_launch(const FusedProgram &prog, int out_mode, void *res, void *scratch, cudaStream_t st) {
    const int64_t packets = (prog.cols + 1) / 2;
    int tx = next_pow2(packets);
    if (tx > 32)
        tx = 32;
    const int ty = CT / tx;
    const int gy = (int)((packets + tx - 1) / tx);
    int64_t cap = ((int64_t)sm_count() * 8 + gy - 1) / gy;
    int64_t want = (prog.rows + (int64_t)ty * 4 - 1) / ((int64_t)ty * 4);
    if (want < 1)
        want = 1;
    const int gx = (int)(want < cap ? want : cap);
    double *part_v = static_cast<double *>(scratch);
    int64_t *part_i = reinterpret_cast<int64_t *>(part_v + (size_t)gx * prog.cols);
    fused_col_kernel<KIND><<<dim3(gx, gy), dim3(tx, ty), CT * 2 * 16, st>>>(prog, part_v, part_i);
    DB2_TRY(after_launch("fused_col_kernel"));
    fused_col_final_kernel<KIND>
        <<<(unsigned)((prog.cols + 127) / 128), 128, 0, st>>>(part_v, part_i, gx, prog.cols, prog.rows, out_mode, res,
                                                              prog.run_if);
    return after_launch("fused_col_final_kernel");
}

int fused_col_pass_f64(const FusedProgram &prog, int agg_op, void *res, void *scratch, size_t scratch_bytes,
                       cudaStream_t st) {
    if (prog.cols == 0)
        return DB2_OK;
    DB2_CHECK(prog.rows > 0, DB2_EINVAL, "aggCol on a matrix without rows");
    DB2_CHECK(scratch && scratch_bytes >= fused_col_scratch_bytes(prog.cols), DB2_EINVAL, "scratch too small");
    switch (agg_op) {
    case DB2_AGG_SUM: return fused_col_launch<CK_SUM>(prog, 0, res, scratch, st);
    case DB2_AGG_MEAN: return fused_col_launch<CK_SUM>(prog, 2, res, scratch, st);
    case DB2_AGG_PROD: return fused_col_launch<CK_PROD>(prog, 0, res, scratch, st);
    case DB2_AGG_MIN: return fused_col_launch<CK_MIN>(prog, 0, res, scratch, st);
    case DB2_AGG_MAX: return fused_col_launch<CK_MAX>(prog, 0, res, scratch, st);
    case DB2_AGG_IDXMIN: return fused_col_launch<CK_MIN>(prog, 1, res, scratch, st);
    case DB2_AGG_IDXMAX: return fused_col_launch<CK_MAX>(prog, 1, res, scratch, st);
    default: return set_error(DB2_EUNSUPPORTED, "AggOpCode %d has no fused column pass", agg_op);
    }
}

} // namespace db2
