// Aggregation kernels: per row, per column, full.
//
// All are HBM-bound (every input element is read exactly once per pass; results are tiny), so the design goal is
// coalesced 128-bit loads with enough packets in flight, and reductions that never serialise on one thread:
//   * rows:    a group of G = 1..32 lanes owns one row (G = packets per row rounded up to a power of two), partial
//              results are combined with warp shuffles inside the group; very wide rows use one CTA per row;
//   * columns: threadIdx.x owns a packet of columns, threadIdx.y strides over rows; column partials are combined
//              across threadIdx.y through shared memory, written per CTA to scratch, and reduced in a fixed order by
//              a second small kernel (deterministic; no floating-point atomics anywhere);
//   * full:    grid-stride packets, warp shuffle + shared memory per CTA, then the same two-stage scheme.
// MIN/MAX/IDXMIN/IDXMAX carry (value, position) pairs and resolve ties to the lowest position, which reproduces
// the reference's sequential scans bit for bit (strict comparisons in AggRow.h:71-96 and AggCol.h:70-121, std::min/
// std::max in EwBinarySca.h:156-157), including their treatment of NaN (a NaN is only ever returned when it is the
// first element) and of signed zeros.
// MEAN/VAR/STDDEV follow the reference's two-pass population formulas (AggRow.h:118-158, AggCol.h:146-173,
// AggAll.h:161-192).
#include "ops.cuh"

#include <mutex>

namespace db2 {

constexpr int AGG_THREADS = 256;
constexpr int64_t NO_IDX = INT64_MAX;

enum AggKind { K_SUM = 0, K_PROD = 1, K_MIN = 2, K_MAX = 3, K_SQDEV = 4 };

// accumulator: value (+ position for MIN/MAX kinds)
template <typename VT, int KIND> struct Acc {
    VT v;
    int64_t i;
    __device__ __forceinline__ void init() {
        if constexpr (KIND == K_SUM || KIND == K_SQDEV)
            v = (VT)0;
        else if constexpr (KIND == K_PROD)
            v = (VT)1;
        else if constexpr (KIND == K_MIN)
            v = pos_inf_or_max<VT>();
        else
            v = neg_inf_or_min<VT>();
        i = NO_IDX;
    }
    // fold one element x at position p (mean only used by K_SQDEV)
    __device__ __forceinline__ void add(VT x, int64_t p, VT mean) {
        if constexpr (KIND == K_SUM)
            v = op_add(v, x);
        else if constexpr (KIND == K_PROD)
            v = op_mul(v, x);
        else if constexpr (KIND == K_SQDEV) {
            const VT d = op_sub(x, mean);
            v = op_add(v, op_mul(d, d));
        } else if constexpr (KIND == K_MIN) {
            if (x < v || (x == v && p < i)) {
                v = x;
                i = p;
            }
        } else {
            if (x > v || (x == v && p < i)) {
                v = x;
                i = p;
            }
        }
    }
    __device__ __forceinline__ void merge(const Acc &o) {
        if constexpr (KIND == K_SUM || KIND == K_SQDEV)
            v = op_add(v, o.v);
        else if constexpr (KIND == K_PROD)
            v = op_mul(v, o.v);
        else if constexpr (KIND == K_MIN) {
            if (o.i != NO_IDX && (o.v < v || (o.v == v && o.i < i) || i == NO_IDX)) {
                v = o.v;
                i = o.i;
            }
        } else {
            if (o.i != NO_IDX && (o.v > v || (o.v == v && o.i < i) || i == NO_IDX)) {
                v = o.v;
                i = o.i;
            }
        }
    }
};

template <typename VT, int KIND> __device__ __forceinline__ Acc<VT, KIND> shfl_xor_acc(Acc<VT, KIND> a, int m) {
    Acc<VT, KIND> o;
    o.v = shfl_xor(a.v, m);
    if constexpr (KIND == K_MIN || KIND == K_MAX)
        o.i = shfl_xor(a.i, m);
    else
        o.i = NO_IDX;
    return o;
}

// op code -> first-pass kind
static inline int kind_of(int op) {
    switch (op) {
    case DB2_AGG_SUM:
    case DB2_AGG_MEAN:
    case DB2_AGG_STDDEV:
    case DB2_AGG_VAR:
        return K_SUM;
    case DB2_AGG_PROD:
        return K_PROD;
    case DB2_AGG_MIN:
    case DB2_AGG_IDXMIN:
        return K_MIN;
    case DB2_AGG_MAX:
    case DB2_AGG_IDXMAX:
        return K_MAX;
    default:
        return -1;
    }
}

// the reference divides by a size_t count: floating point -> ordinary division, int64 -> unsigned division
template <typename VT> __device__ __forceinline__ VT div_count(VT s, int64_t n) {
    if constexpr (std::is_integral_v<VT>)
        return (VT)((uint64_t)s / (uint64_t)n);
    else
        return op_div(s, (VT)n);
}
template <typename VT> __device__ __forceinline__ VT sqrt_vt(VT x) {
    if constexpr (std::is_same_v<VT, float>)
        return __fsqrt_rn(x);
    else if constexpr (std::is_same_v<VT, double>)
        return __dsqrt_rn(x);
    else
        return (VT)__dsqrt_rn((double)x);
}

// ---------------------------------------------------------------------------
// rows
// ---------------------------------------------------------------------------
// One group of G lanes per row.  OP is the AggOpCode.  VEC = Pack<VT>::N when rows are 16-byte aligned, else 1.
template <typename VT, int OP, int G, int VEC>
__global__ void __launch_bounds__(AGG_THREADS)
    agg_row_kernel(const VT *__restrict__ arg, int64_t rows, int64_t cols, int64_t ld, void *__restrict__ res,
                   int64_t res_ld) {
    constexpr int KIND = (OP == DB2_AGG_PROD)                            ? K_PROD
                         : (OP == DB2_AGG_MIN || OP == DB2_AGG_IDXMIN) ? K_MIN
                         : (OP == DB2_AGG_MAX || OP == DB2_AGG_IDXMAX) ? K_MAX
                                                                       : K_SUM;
    constexpr int ROWS_PER_CTA = AGG_THREADS / G;
    const int lane = threadIdx.x % G;
    const int grp = threadIdx.x / G;
    const int64_t row_stride = (int64_t)gridDim.x * ROWS_PER_CTA;
    const int64_t rows_padded = (rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA * ROWS_PER_CTA; // keep groups converged
    for (int64_t r = (int64_t)blockIdx.x * ROWS_PER_CTA + grp; r < rows_padded; r += row_stride) {
        const bool live = r < rows;
        const VT *row = arg + (live ? r : 0) * ld;
        Acc<VT, KIND> acc;
        acc.init();
        if (live) {
            for (int64_t c0 = (int64_t)lane * VEC; c0 < cols; c0 += (int64_t)G * VEC) {
                if constexpr (VEC > 1) {
                    if (c0 + VEC <= cols) {
                        const Pack<VT> p = ld_pack_stream(row + c0);
#pragma unroll
                        for (int k = 0; k < VEC; k++)
                            acc.add(p.v[k], c0 + k, (VT)0);
                    } else {
                        for (int64_t c = c0; c < cols; c++)
                            acc.add(row[c], c, (VT)0);
                    }
                } else
                    acc.add(row[c0], c0, (VT)0);
            }
        }
#pragma unroll
        for (int m = G / 2; m >= 1; m >>= 1)
            acc.merge(shfl_xor_acc<VT, KIND>(acc, m));
        // every lane of the group now holds the row's aggregate
        if constexpr (OP == DB2_AGG_STDDEV || OP == DB2_AGG_VAR) {
            const VT mean = div_count(acc.v, cols);
            Acc<VT, K_SQDEV> sq;
            sq.init();
            if (live) {
                for (int64_t c0 = (int64_t)lane * VEC; c0 < cols; c0 += (int64_t)G * VEC) {
                    const int64_t ce = (c0 + VEC <= cols) ? c0 + VEC : cols;
                    for (int64_t c = c0; c < ce; c++)
                        sq.add(row[c], c, mean);
                }
            }
#pragma unroll
            for (int m = G / 2; m >= 1; m >>= 1)
                sq.merge(shfl_xor_acc<VT, K_SQDEV>(sq, m));
            if (live && lane == 0) {
                VT var = div_count(sq.v, cols);
                static_cast<VT *>(res)[r * res_ld] = (OP == DB2_AGG_STDDEV) ? sqrt_vt(var) : var;
            }
        } else if (live && lane == 0) {
            if constexpr (KIND == K_MIN || KIND == K_MAX) {
                const VT first = row[0];
                const bool first_nan = first != first;
                if (first_nan || acc.i == NO_IDX) {
                    acc.v = first;
                    acc.i = 0;
                }
                if constexpr (OP == DB2_AGG_IDXMIN || OP == DB2_AGG_IDXMAX)
                    static_cast<uint64_t *>(res)[r * res_ld] = (uint64_t)acc.i;
                else
                    static_cast<VT *>(res)[r * res_ld] = acc.v;
            } else if constexpr (OP == DB2_AGG_MEAN)
                static_cast<VT *>(res)[r * res_ld] = div_count(acc.v, cols);
            else
                static_cast<VT *>(res)[r * res_ld] = acc.v;
        }
    }
}

// One CTA per row (wide rows, few rows).
template <typename VT, int OP>
__global__ void __launch_bounds__(AGG_THREADS)
    agg_row_wide_kernel(const VT *__restrict__ arg, int64_t rows, int64_t cols, int64_t ld, void *__restrict__ res,
                        int64_t res_ld) {
    constexpr int KIND = (OP == DB2_AGG_PROD)                            ? K_PROD
                         : (OP == DB2_AGG_MIN || OP == DB2_AGG_IDXMIN) ? K_MIN
                         : (OP == DB2_AGG_MAX || OP == DB2_AGG_IDXMAX) ? K_MAX
                                                                       : K_SUM;
    __shared__ VT sv[AGG_THREADS / 32];
    __shared__ int64_t si[AGG_THREADS / 32];
    __shared__ VT s_mean;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const VT *row = arg + r * ld;
        Acc<VT, KIND> acc;
        acc.init();
        for (int64_t c = threadIdx.x; c < cols; c += AGG_THREADS)
            acc.add(row[c], c, (VT)0);
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1)
            acc.merge(shfl_xor_acc<VT, KIND>(acc, m));
        __syncthreads();
        if (lane == 0) {
            sv[warp] = acc.v;
            si[warp] = acc.i;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            Acc<VT, KIND> t;
            t.v = sv[0];
            t.i = si[0];
            for (int w = 1; w < AGG_THREADS / 32; w++) {
                Acc<VT, KIND> o;
                o.v = sv[w];
                o.i = si[w];
                t.merge(o);
            }
            if constexpr (KIND == K_MIN || KIND == K_MAX) {
                const VT first = row[0];
                if (first != first || t.i == NO_IDX) {
                    t.v = first;
                    t.i = 0;
                }
                if constexpr (OP == DB2_AGG_IDXMIN || OP == DB2_AGG_IDXMAX)
                    static_cast<uint64_t *>(res)[r * res_ld] = (uint64_t)t.i;
                else
                    static_cast<VT *>(res)[r * res_ld] = t.v;
            } else if constexpr (OP == DB2_AGG_MEAN)
                static_cast<VT *>(res)[r * res_ld] = div_count(t.v, cols);
            else if constexpr (OP == DB2_AGG_STDDEV || OP == DB2_AGG_VAR)
                s_mean = div_count(t.v, cols);
            else
                static_cast<VT *>(res)[r * res_ld] = t.v;
        }
        if constexpr (OP == DB2_AGG_STDDEV || OP == DB2_AGG_VAR) {
            __syncthreads();
            const VT mean = s_mean;
            Acc<VT, K_SQDEV> sq;
            sq.init();
            for (int64_t c = threadIdx.x; c < cols; c += AGG_THREADS)
                sq.add(row[c], c, mean);
#pragma unroll
            for (int m = 16; m >= 1; m >>= 1)
                sq.merge(shfl_xor_acc<VT, K_SQDEV>(sq, m));
            __syncthreads();
            if (lane == 0)
                sv[warp] = sq.v;
            __syncthreads();
            if (threadIdx.x == 0) {
                VT t = sv[0];
                for (int w = 1; w < AGG_THREADS / 32; w++)
                    t = op_add(t, sv[w]);
                VT var = div_count(t, cols);
                static_cast<VT *>(res)[r * res_ld] = (OP == DB2_AGG_STDDEV) ? sqrt_vt(var) : var;
            }
        }
    }
}

template <typename VT, int OP>
static int agg_row_launch(const VT *arg, int64_t rows, int64_t cols, int64_t ld, void *res, int64_t res_ld,
                          cudaStream_t st) {
    constexpr int N = Pack<VT>::N;
    const int cap = sm_count() * 8;
    if (cols >= 8192 && rows < (int64_t)cap * 4) {
        int grid = (int)(rows < cap ? rows : cap);
        agg_row_wide_kernel<VT, OP><<<grid, AGG_THREADS, 0, st>>>(arg, rows, cols, ld, res, res_ld);
        return after_launch("agg_row_wide_kernel");
    }
    const bool vec_ok = aligned16(arg) && ((ld * (int64_t)sizeof(VT)) % 16 == 0);
    const int vec = vec_ok ? N : 1;
    int g = next_pow2((cols + vec - 1) / vec);
    if (g > 32)
        g = 32;
    const int rows_per_cta = AGG_THREADS / g;
    int64_t want = (rows + rows_per_cta - 1) / rows_per_cta;
    int grid = (int)(want < cap ? want : cap);
#define LAUNCH_G(GG)                                                                                                   \
    case GG:                                                                                                           \
        if (vec_ok)                                                                                                    \
            agg_row_kernel<VT, OP, GG, N><<<grid, AGG_THREADS, 0, st>>>(arg, rows, cols, ld, res, res_ld);             \
        else                                                                                                           \
            agg_row_kernel<VT, OP, GG, 1><<<grid, AGG_THREADS, 0, st>>>(arg, rows, cols, ld, res, res_ld);             \
        break;
    switch (g) {
        LAUNCH_G(1)
        LAUNCH_G(2)
        LAUNCH_G(4)
        LAUNCH_G(8)
        LAUNCH_G(16)
        LAUNCH_G(32)
    }
#undef LAUNCH_G
    return after_launch("agg_row_kernel");
}

// ---------------------------------------------------------------------------
// columns
// ---------------------------------------------------------------------------
// blockDim = (TX, AGG_THREADS / TX).  blockIdx.y selects a chunk of TX*VEC columns, blockIdx.x strides over rows.
// Writes one partial per (blockIdx.x, column): part_v[blockIdx.x * cols + c] (+ part_i for MIN/MAX kinds).
template <typename VT, int KIND, int VEC>
__global__ void __launch_bounds__(AGG_THREADS)
    agg_col_partial_kernel(const VT *__restrict__ arg, int64_t rows, int64_t cols, int64_t ld,
                           const VT *__restrict__ mean, VT *__restrict__ part_v, int64_t *__restrict__ part_i) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tx = threadIdx.x, ty = threadIdx.y, TX = blockDim.x, TY = blockDim.y;
    const int64_t c0 = ((int64_t)blockIdx.y * TX + tx) * VEC;
    Acc<VT, KIND> acc[VEC];
    VT mu[VEC];
#pragma unroll
    for (int k = 0; k < VEC; k++) {
        acc[k].init();
        mu[k] = (KIND == K_SQDEV && c0 + k < cols) ? mean[c0 + k] : (VT)0;
    }
    if (c0 < cols) {
        const int64_t row_stride = (int64_t)gridDim.x * TY;
        int64_t r = (int64_t)blockIdx.x * TY + ty;
        if (VEC > 1 && c0 + VEC <= cols) {
            // two rows in flight per thread
            for (; r + row_stride < rows; r += 2 * row_stride) {
                const Pack<VT> p0 = ld_pack_stream(arg + r * ld + c0);
                const Pack<VT> p1 = ld_pack_stream(arg + (r + row_stride) * ld + c0);
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    acc[k].add(p0.v[k], r, mu[k]);
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    acc[k].add(p1.v[k], r + row_stride, mu[k]);
            }
            for (; r < rows; r += row_stride) {
                const Pack<VT> p0 = ld_pack_stream(arg + r * ld + c0);
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    acc[k].add(p0.v[k], r, mu[k]);
            }
        } else {
            for (; r < rows; r += row_stride) {
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    if (c0 + k < cols)
                        acc[k].add(arg[r * ld + c0 + k], r, mu[k]);
            }
        }
    }
    // combine across ty through shared memory
    VT *sv = reinterpret_cast<VT *>(smem_raw);                                         // [TY][TX*VEC]
    int64_t *si = reinterpret_cast<int64_t *>(smem_raw + sizeof(VT) * AGG_THREADS * VEC); // same shape
#pragma unroll
    for (int k = 0; k < VEC; k++) {
        sv[(ty * TX + tx) * VEC + k] = acc[k].v;
        if constexpr (KIND == K_MIN || KIND == K_MAX)
            si[(ty * TX + tx) * VEC + k] = acc[k].i;
    }
    __syncthreads();
    // thread (tx, ty) with ty < VEC finishes column c0 + ty
    for (int k = ty; k < VEC; k += TY) {
        if (c0 + k < cols) {
            Acc<VT, KIND> t;
            t.v = sv[(0 * TX + tx) * VEC + k];
            t.i = (KIND == K_MIN || KIND == K_MAX) ? si[(0 * TX + tx) * VEC + k] : NO_IDX;
            for (int y = 1; y < TY; y++) {
                Acc<VT, KIND> o;
                o.v = sv[(y * TX + tx) * VEC + k];
                o.i = (KIND == K_MIN || KIND == K_MAX) ? si[(y * TX + tx) * VEC + k] : NO_IDX;
                t.merge(o);
            }
            part_v[(int64_t)blockIdx.x * cols + c0 + k] = t.v;
            if constexpr (KIND == K_MIN || KIND == K_MAX)
                part_i[(int64_t)blockIdx.x * cols + c0 + k] = t.i;
        }
    }
}

// Second stage: one thread per column folds the `nparts` partials in order and applies the op's epilogue.
// OUT: 0 = value, 1 = index (uint64), 2 = value / count (MEAN, or mean for the variance's first pass),
//      3 = value / count (VAR), 4 = sqrt(value / count) (STDDEV).
template <typename VT, int KIND>
__global__ void agg_col_final_kernel(const VT *__restrict__ part_v, const int64_t *__restrict__ part_i, int nparts,
                                     int64_t cols, int64_t count, const VT *__restrict__ first_row, int out_mode,
                                     void *__restrict__ res) {
    // one warp per column: lane l folds partials l, l + 32, ... in order, then a fixed shuffle tree
    const int lane = threadIdx.x % 32;
    const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    if (c >= cols)
        return;
    Acc<VT, KIND> t;
    t.init();
    for (int p = lane; p < nparts; p += 32) {
        Acc<VT, KIND> o;
        o.v = part_v[(int64_t)p * cols + c];
        o.i = (KIND == K_MIN || KIND == K_MAX) ? part_i[(int64_t)p * cols + c] : NO_IDX;
        t.merge(o); // lanes start from the neutral element
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1)
        t.merge(shfl_xor_acc<VT, KIND>(t, m));
    if (lane != 0)
        return;
    if constexpr (KIND == K_MIN || KIND == K_MAX) {
        const VT first = first_row[c];
        if (first != first || t.i == NO_IDX) {
            t.v = first;
            t.i = 0;
        }
    }
    if (out_mode == 1)
        static_cast<uint64_t *>(res)[c] = (uint64_t)t.i;
    else if (out_mode == 0)
        static_cast<VT *>(res)[c] = t.v;
    else if (out_mode == 2 || out_mode == 3)
        static_cast<VT *>(res)[c] = div_count(t.v, count);
    else
        static_cast<VT *>(res)[c] = sqrt_vt(div_count(t.v, count));
}

struct ColPlan {
    int vec, tx, ty, gx, gy;
    size_t smem;
};
template <typename VT> static ColPlan col_plan(const void *arg, int64_t rows, int64_t cols, int64_t ld) {
    constexpr int N = Pack<VT>::N;
    ColPlan p;
    const bool vec_ok = aligned16(arg) && ((ld * (int64_t)sizeof(VT)) % 16 == 0) && cols >= N;
    p.vec = vec_ok ? N : 1;
    const int64_t packets = (cols + p.vec - 1) / p.vec;
    p.tx = next_pow2(packets);
    if (p.tx > 32)
        p.tx = 32; // a warp covers 512 contiguous bytes of a row; wider matrices use blockIdx.y
    p.ty = AGG_THREADS / p.tx;
    p.gy = (int)((packets + p.tx - 1) / p.tx);
    int64_t cap = ((int64_t)sm_count() * 8 + p.gy - 1) / p.gy;
    int64_t want = (rows + (int64_t)p.ty * 4 - 1) / ((int64_t)p.ty * 4); // >= 4 rows per thread before adding CTAs
    if (want < 1)
        want = 1;
    p.gx = (int)(want < cap ? want : cap);
    p.smem = (sizeof(VT) + sizeof(int64_t)) * AGG_THREADS * N;
    return p;
}
// upper bound over both alignments, so that the size query needs no pointer
static size_t col_scratch_bytes(int64_t cols, size_t vt_size) {
    const int64_t max_parts = (int64_t)sm_count() * 8;
    return (size_t)max_parts * cols * (vt_size + 8) + (size_t)cols * vt_size + 256;
}

template <typename VT, int KIND>
static int agg_col_pass(const VT *arg, int64_t rows, int64_t cols, int64_t ld, const VT *mean, int out_mode,
                        int64_t count, void *res, void *scratch, cudaStream_t st) {
    ColPlan p = col_plan<VT>(arg, rows, cols, ld);
    VT *part_v = static_cast<VT *>(scratch);
    int64_t *part_i = reinterpret_cast<int64_t *>(static_cast<char *>(scratch) +
                                                  (((size_t)p.gx * cols * sizeof(VT) + 15) & ~(size_t)15));
    dim3 block(p.tx, p.ty), grid(p.gx, p.gy);
    if (p.vec > 1)
        agg_col_partial_kernel<VT, KIND, Pack<VT>::N>
            <<<grid, block, p.smem, st>>>(arg, rows, cols, ld, mean, part_v, part_i);
    else
        agg_col_partial_kernel<VT, KIND, 1><<<grid, block, p.smem, st>>>(arg, rows, cols, ld, mean, part_v, part_i);
    DB2_TRY(after_launch("agg_col_partial_kernel"));
    const int fb = 256; // 8 columns (warps) per block
    agg_col_final_kernel<VT, KIND>
        <<<(unsigned)((cols * 32 + fb - 1) / fb), fb, 0, st>>>(part_v, part_i, p.gx, cols, count, arg, out_mode, res);
    return after_launch("agg_col_final_kernel");
}

template <typename VT>
static int agg_col_impl(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, void *res, void *scratch,
                        size_t scratch_bytes, cudaStream_t st) {
    if (cols == 0)
        return DB2_OK;
    DB2_CHECK(rows > 0, DB2_EINVAL, "aggCol on a matrix without rows");
    DB2_CHECK(scratch && scratch_bytes >= col_scratch_bytes(cols, sizeof(VT)), DB2_EINVAL,
              "aggCol scratch too small: %zu < %zu", scratch_bytes, col_scratch_bytes(cols, sizeof(VT)));
    switch (op) {
    case DB2_AGG_SUM:
        return agg_col_pass<VT, K_SUM>(arg, rows, cols, ld, nullptr, 0, rows, res, scratch, st);
    case DB2_AGG_PROD:
        return agg_col_pass<VT, K_PROD>(arg, rows, cols, ld, nullptr, 0, rows, res, scratch, st);
    case DB2_AGG_MIN:
        return agg_col_pass<VT, K_MIN>(arg, rows, cols, ld, nullptr, 0, rows, res, scratch, st);
    case DB2_AGG_MAX:
        return agg_col_pass<VT, K_MAX>(arg, rows, cols, ld, nullptr, 0, rows, res, scratch, st);
    case DB2_AGG_IDXMIN:
        return agg_col_pass<VT, K_MIN>(arg, rows, cols, ld, nullptr, 1, rows, res, scratch, st);
    case DB2_AGG_IDXMAX:
        return agg_col_pass<VT, K_MAX>(arg, rows, cols, ld, nullptr, 1, rows, res, scratch, st);
    case DB2_AGG_MEAN:
        return agg_col_pass<VT, K_SUM>(arg, rows, cols, ld, nullptr, 2, rows, res, scratch, st);
    case DB2_AGG_VAR:
    case DB2_AGG_STDDEV: {
        // the mean lives at the end of the scratch area
        VT *mean = reinterpret_cast<VT *>(static_cast<char *>(scratch) +
                                          ((scratch_bytes - (size_t)cols * sizeof(VT)) & ~(size_t)15));
        DB2_TRY((agg_col_pass<VT, K_SUM>(arg, rows, cols, ld, nullptr, 2, rows, mean, scratch, st)));
        return agg_col_pass<VT, K_SQDEV>(arg, rows, cols, ld, mean, op == DB2_AGG_VAR ? 3 : 4, rows, res, scratch,
                                         st);
    }
    default:
        return set_error(DB2_EUNSUPPORTED, "unsupported AggOpCode %d", op);
    }
}

// ---------------------------------------------------------------------------
// full aggregation
// ---------------------------------------------------------------------------
template <typename VT, int KIND> __device__ __forceinline__ VT block_reduce_value(VT v, VT *sh) {
    // value-only reduce (MIN/MAX here compare values only: the full aggregate returns no position)
    auto comb = [](VT a, VT b) -> VT {
        if constexpr (KIND == K_SUM || KIND == K_SQDEV)
            return op_add(a, b);
        else if constexpr (KIND == K_PROD)
            return op_mul(a, b);
        else if constexpr (KIND == K_MIN)
            return (b < a) ? b : a;
        else
            return (a < b) ? b : a;
    };
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1)
        v = comb(v, shfl_xor(v, m));
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    __syncthreads();
    if (lane == 0)
        sh[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        VT t = sh[0];
        for (int w = 1; w < (int)(blockDim.x / 32); w++)
            t = comb(t, sh[w]);
        sh[0] = t;
    }
    __syncthreads();
    return sh[0];
}

template <typename VT, int KIND> __device__ __forceinline__ VT neutral_value() {
    if constexpr (KIND == K_SUM || KIND == K_SQDEV)
        return (VT)0;
    else if constexpr (KIND == K_PROD)
        return (VT)1;
    else if constexpr (KIND == K_MIN)
        return pos_inf_or_max<VT>();
    else
        return neg_inf_or_min<VT>();
}
template <typename VT, int KIND> __device__ __forceinline__ VT fold_value(VT a, VT x, VT mean) {
    if constexpr (KIND == K_SUM)
        return op_add(a, x);
    else if constexpr (KIND == K_PROD)
        return op_mul(a, x);
    else if constexpr (KIND == K_SQDEV) {
        const VT d = op_sub(x, mean);
        return op_add(a, op_mul(d, d));
    } else if constexpr (KIND == K_MIN)
        return (x < a) ? x : a;
    else
        return (a < x) ? x : a;
}

// rows x cols with leading dimension ld; contiguous input is passed as 1 x n.
template <typename VT, int KIND, int VEC>
__global__ void __launch_bounds__(AGG_THREADS)
    agg_all_partial_kernel(const VT *__restrict__ arg, int64_t rows, int64_t cols, int64_t ld,
                           const VT *__restrict__ mean_ptr, VT *__restrict__ part) {
    __shared__ VT sh[AGG_THREADS / 32];
    const VT mean = (KIND == K_SQDEV) ? *mean_ptr : (VT)0;
    VT a0 = neutral_value<VT, KIND>(), a1 = a0, a2 = a0, a3 = a0;
    const int64_t pk_per_row = cols / VEC;
    if (rows == 1 || ld == cols) {
        const int64_t n = rows * cols;
        const int64_t npk = n / VEC;
        const int64_t stride = (int64_t)gridDim.x * AGG_THREADS;
        int64_t i = (int64_t)blockIdx.x * AGG_THREADS + threadIdx.x;
        if constexpr (VEC > 1) {
            for (; i + 3 * stride < npk; i += 4 * stride) {
                const Pack<VT> p0 = ld_pack_stream(arg + i * VEC);
                const Pack<VT> p1 = ld_pack_stream(arg + (i + stride) * VEC);
                const Pack<VT> p2 = ld_pack_stream(arg + (i + 2 * stride) * VEC);
                const Pack<VT> p3 = ld_pack_stream(arg + (i + 3 * stride) * VEC);
#pragma unroll
                for (int k = 0; k < VEC; k++) {
                    a0 = fold_value<VT, KIND>(a0, p0.v[k], mean);
                    a1 = fold_value<VT, KIND>(a1, p1.v[k], mean);
                    a2 = fold_value<VT, KIND>(a2, p2.v[k], mean);
                    a3 = fold_value<VT, KIND>(a3, p3.v[k], mean);
                }
            }
            for (; i < npk; i += stride) {
                const Pack<VT> p0 = ld_pack_stream(arg + i * VEC);
#pragma unroll
                for (int k = 0; k < VEC; k++)
                    a0 = fold_value<VT, KIND>(a0, p0.v[k], mean);
            }
            const int64_t t = npk * VEC + (int64_t)blockIdx.x * AGG_THREADS + threadIdx.x;
            if (t < n)
                a1 = fold_value<VT, KIND>(a1, arg[t], mean);
        } else {
            for (; i < n; i += stride)
                a0 = fold_value<VT, KIND>(a0, arg[i], mean);
        }
    } else {
        // strided view: a warp walks one row at a time
        const int lane = threadIdx.x % 32;
        const int64_t warp_id = ((int64_t)blockIdx.x * AGG_THREADS + threadIdx.x) / 32;
        const int64_t nwarps = (int64_t)gridDim.x * AGG_THREADS / 32;
        for (int64_t r = warp_id; r < rows; r += nwarps)
            for (int64_t c = lane; c < cols; c += 32)
                a0 = fold_value<VT, KIND>(a0, arg[r * ld + c], mean);
        (void)pk_per_row;
    }
    VT v;
    if constexpr (KIND == K_SQDEV || KIND == K_SUM)
        v = op_add(op_add(a0, a1), op_add(a2, a3));
    else if constexpr (KIND == K_PROD)
        v = op_mul(op_mul(a0, a1), op_mul(a2, a3));
    else
        v = fold_value<VT, KIND>(fold_value<VT, KIND>(a0, a1, mean), fold_value<VT, KIND>(a2, a3, mean), mean);
    v = block_reduce_value<VT, KIND>(v, sh);
    if (threadIdx.x == 0)
        part[blockIdx.x] = v;
}

// out_mode: 0 value, 2 value/count, 3 value/count (VAR), 4 sqrt(value/count)
template <typename VT, int KIND>
__global__ void __launch_bounds__(AGG_THREADS)
    agg_all_final_kernel(const VT *__restrict__ part, int nparts, int64_t count, int out_mode, VT *__restrict__ res) {
    __shared__ VT sh[AGG_THREADS / 32];
    VT a = neutral_value<VT, KIND>();
    constexpr int K2 = (KIND == K_SQDEV) ? K_SUM : KIND;
    for (int i = threadIdx.x; i < nparts; i += AGG_THREADS)
        a = fold_value<VT, K2>(a, part[i], (VT)0);
    a = block_reduce_value<VT, K2>(a, sh);
    if (threadIdx.x == 0) {
        if (out_mode == 0)
            *res = a;
        else if (out_mode == 2 || out_mode == 3)
            *res = div_count(a, count);
        else
            *res = sqrt_vt(div_count(a, count));
    }
}

static size_t all_scratch_bytes(size_t vt_size) { return (size_t)sm_count() * 8 * vt_size + 64; }

template <typename VT, int KIND>
static int agg_all_pass(const VT *arg, int64_t rows, int64_t cols, int64_t ld, const VT *mean, int out_mode,
                        VT *res, VT *part, cudaStream_t st) {
    constexpr int N = Pack<VT>::N;
    const int64_t n = rows * cols;
    const bool contiguous = rows == 1 || ld == cols;
    const int64_t per_block = (int64_t)AGG_THREADS * N * 4;
    int64_t want = (n + per_block - 1) / per_block;
    const int64_t cap = (int64_t)sm_count() * 8;
    int grid = (int)(want < 1 ? 1 : (want < cap ? want : cap));
    if (contiguous && aligned16(arg))
        agg_all_partial_kernel<VT, KIND, N><<<grid, AGG_THREADS, 0, st>>>(arg, rows, cols, ld, mean, part);
    else
        agg_all_partial_kernel<VT, KIND, 1><<<grid, AGG_THREADS, 0, st>>>(arg, rows, cols, ld, mean, part);
    DB2_TRY(after_launch("agg_all_partial_kernel"));
    agg_all_final_kernel<VT, KIND><<<1, AGG_THREADS, 0, st>>>(part, grid, n, out_mode, res);
    return after_launch("agg_all_final_kernel");
}

template <typename VT>
static int agg_all_impl(int op, const VT *arg, int64_t rows, int64_t cols, int64_t ld, VT *res, void *scratch,
                        size_t scratch_bytes, cudaStream_t st) {
    DB2_CHECK(scratch && scratch_bytes >= all_scratch_bytes(sizeof(VT)), DB2_EINVAL,
              "aggAll scratch too small: %zu < %zu", scratch_bytes, all_scratch_bytes(sizeof(VT)));
    VT *part = static_cast<VT *>(scratch);
    switch (op) {
    case DB2_AGG_SUM:
        return agg_all_pass<VT, K_SUM>(arg, rows, cols, ld, nullptr, 0, res, part, st);
    case DB2_AGG_PROD:
        return agg_all_pass<VT, K_PROD>(arg, rows, cols, ld, nullptr, 0, res, part, st);
    case DB2_AGG_MIN:
        return agg_all_pass<VT, K_MIN>(arg, rows, cols, ld, nullptr, 0, res, part, st);
    case DB2_AGG_MAX:
        return agg_all_pass<VT, K_MAX>(arg, rows, cols, ld, nullptr, 0, res, part, st);
    case DB2_AGG_MEAN:
        return agg_all_pass<VT, K_SUM>(arg, rows, cols, ld, nullptr, 2, res, part, st);
    case DB2_AGG_VAR:
    case DB2_AGG_STDDEV: {
        VT *mean = reinterpret_cast<VT *>(static_cast<char *>(scratch) + ((scratch_bytes - sizeof(VT)) & ~(size_t)15));
        DB2_TRY((agg_all_pass<VT, K_SUM>(arg, rows, cols, ld, nullptr, 2, mean, part, st)));
        return agg_all_pass<VT, K_SQDEV>(arg, rows, cols, ld, mean, op == DB2_AGG_VAR ? 3 : 4, res, part, st);
    }
    default:
        return set_error(DB2_EUNSUPPORTED, "unsupported AggOpCode %d for a full aggregation", op);
    }
}

} // namespace db2

using namespace db2;

#define DB2_DISPATCH_AGGOP(op, OP, ...)                                                                                \
    switch (op) {                                                                                                      \
    case DB2_AGG_SUM: { constexpr int OP = DB2_AGG_SUM; __VA_ARGS__; } break;                                          \
    case DB2_AGG_PROD: { constexpr int OP = DB2_AGG_PROD; __VA_ARGS__; } break;                                        \
    case DB2_AGG_MIN: { constexpr int OP = DB2_AGG_MIN; __VA_ARGS__; } break;                                          \
    case DB2_AGG_MAX: { constexpr int OP = DB2_AGG_MAX; __VA_ARGS__; } break;                                          \
    case DB2_AGG_IDXMIN: { constexpr int OP = DB2_AGG_IDXMIN; __VA_ARGS__; } break;                                    \
    case DB2_AGG_IDXMAX: { constexpr int OP = DB2_AGG_IDXMAX; __VA_ARGS__; } break;                                    \
    case DB2_AGG_MEAN: { constexpr int OP = DB2_AGG_MEAN; __VA_ARGS__; } break;                                        \
    case DB2_AGG_STDDEV: { constexpr int OP = DB2_AGG_STDDEV; __VA_ARGS__; } break;                                    \
    case DB2_AGG_VAR: { constexpr int OP = DB2_AGG_VAR; __VA_ARGS__; } break;                                          \
    default:                                                                                                           \
        return ::db2::set_error(DB2_EUNSUPPORTED, "unknown AggOpCode %d", (int)(op));                                  \
    }

extern "C" int db2k_agg_row(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                            int64_t res_ld, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    if (rows == 0)
        return DB2_OK;
    DB2_CHECK(cols > 0, DB2_EINVAL, "aggRow on a matrix without columns");
    DB2_CHECK(arg && res, DB2_EINVAL, "null operand");
    DB2_DISPATCH_DTYPE(dtype, VT,
                       DB2_DISPATCH_AGGOP(op, OP, return (agg_row_launch<VT, OP>((const VT *)arg, rows, cols, ld, res,
                                                                                 res_ld, as_stream(stream)))));
    return DB2_OK;
}

extern "C" size_t db2k_agg_col_scratch_bytes(int dtype, int op, int64_t rows, int64_t cols) {
    (void)op;
    (void)rows;
    return col_scratch_bytes(cols, dtype_size(dtype));
}

extern "C" int db2k_agg_col(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                            void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    DB2_CHECK((arg && res) || cols == 0, DB2_EINVAL, "null operand");
    DB2_DISPATCH_DTYPE(dtype, VT, return (agg_col_impl<VT>(op, (const VT *)arg, rows, cols, ld, res, scratch,
                                                           scratch_bytes, as_stream(stream))));
    return DB2_OK;
}

// ---------------------------------------------------------------------------
// column aggregation without any allocation
// ---------------------------------------------------------------------------
// Scratch for db2k_agg_col_static: one fixed array in device memory per GPU that loads this library.  Host code only
// ever uses its address as returned by cudaGetSymbolAddress (the bare name is a host-side stand-in for the symbol).
#define DB2_STATIC_SCRATCH_BYTES (4u << 20)
static __device__ __align__(256) unsigned char g_agg_col_static_scratch[DB2_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_mu;
void *g_static_ptr[64] = {nullptr};

// Looks the array's device address up once per device (with that device current) and remembers it.
int static_scratch(void **out) {
    int dev = -1;
    DB2_CUDA(cudaGetDevice(&dev));
    DB2_CHECK(dev >= 0 && dev < 64, DB2_EINVAL, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        DB2_CUDA(cudaGetSymbolAddress(&p, g_agg_col_static_scratch));
        DB2_CHECK(p != nullptr, DB2_ECUDA, "cudaGetSymbolAddress returned a null address");
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return DB2_OK;
}
} // namespace

extern "C" size_t db2k_agg_col_static_max_bytes(void) { return DB2_STATIC_SCRATCH_BYTES; }

extern "C" int db2k_agg_col_static(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld,
                                   void *res, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    DB2_CHECK((arg && res) || cols == 0, DB2_EINVAL, "null operand");
    const size_t need = col_scratch_bytes(cols, dtype_size(dtype));
    DB2_CHECK(need <= (size_t)DB2_STATIC_SCRATCH_BYTES, DB2_EINVAL,
              "db2k_agg_col_static: %lld columns need %zu bytes of scratch, the built-in array holds %zu; use "
              "db2k_agg_col with caller-provided scratch for wider matrices",
              (long long)cols, need, (size_t)DB2_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    DB2_TRY(static_scratch(&scratch));
    DB2_DISPATCH_DTYPE(dtype, VT, return (agg_col_impl<VT>(op, (const VT *)arg, rows, cols, ld, res, scratch,
                                                           (size_t)DB2_STATIC_SCRATCH_BYTES, as_stream(stream))));
    return DB2_OK;
}

extern "C" size_t db2k_agg_all_scratch_bytes(int dtype, int op, int64_t rows, int64_t cols) {
    (void)op;
    (void)rows;
    (void)cols;
    return all_scratch_bytes(dtype_size(dtype));
}

extern "C" int db2k_agg_all(int dtype, int op, const void *arg, int64_t rows, int64_t cols, int64_t ld, void *res,
                            void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    DB2_CHECK(rows * cols > 0, DB2_EINVAL, "aggAll on an empty matrix");
    DB2_CHECK(arg && res, DB2_EINVAL, "null operand");
    DB2_DISPATCH_DTYPE(dtype, VT, return (agg_all_impl<VT>(op, (const VT *)arg, rows, cols, ld, (VT *)res, scratch,
                                                           scratch_bytes, as_stream(stream))));
    return DB2_OK;
}
