// Compile-time specialisations of the fused passes (fused.cuh) for the chains the benchmark pipelines produce.
//
// The interpreter in fused.cu spends most of its instructions on decoding; for a chain known at compile time the
// per-element work shrinks to the arithmetic itself, which is what lets the standardisation pass run at HBM speed
// on a part whose FP64 rate is only 64 instructions per SM and clock.  A chain is spelled as a type list
// (Chain<S<op, operand kind>...>, Taps<T<position, tracker kind>...>); the runtime matches the signature string of a
// recorded program against the table at the end of this file and falls back to the interpreter otherwise.  Adding a
// pattern is one table line.
//
// Row pass layout: every warp works on its own: a warp owns tiles of 32 rows and walks them in chunks of 32 columns.
// A chunk is brought into the warp's shared memory with 16-byte cp.async copies (no register staging) into an
// XOR-swizzled layout -- 16-byte slot p of row r lives at slot p ^ (r & 15) -- so that the cooperative (coalesced)
// fill and the one-row-per-lane walk are both bank-conflict free without padding.  Each warp has two chunk buffers:
// the copies of its next chunk are in flight while it evaluates the current one, so an SM always has 8 KB per warp
// outstanding and no warp ever waits at a block-wide barrier.  Every lane walks its row with 128-bit shared loads,
// applies the chain and feeds its row trackers; results leave one row per lane (coalesced).  No cross-lane
// reduction exists.
#include "fused.cuh"
#include "ops.cuh"

#include <cstring>
#include <type_traits>

#include "fused_ct_dev.cuh"

namespace db2 {
namespace ct {

template <typename ChainT, typename TapsT, bool EW> static int launch_row(const FusedProgram &prog, cudaStream_t st) {
    const size_t smem = (size_t)(WARPS * 2 * WR * CK + prog.smem_elems + 2 * FUSED_MAX_STEPS) * sizeof(double) + 256; // + run-time chain tables, alignment slack
    const int64_t nblocks = ((prog.rows + WR - 1) / WR + WARPS - 1) / WARPS;
    const int64_t cap = (int64_t)sm_count() * RowCtasPerSm<ChainT>::value;
    const int grid = (int)(nblocks < cap ? nblocks : cap);
    static PerDeviceOnce attr;
    if (attr.need()) {
        DB2_CUDA(cudaFuncSetAttribute(fused_row_ct_kernel<ChainT, TapsT, EW>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024));
        attr.mark();
    }
    fused_row_ct_kernel<ChainT, TapsT, EW><<<grid, RT, smem, st>>>(prog);
    return after_launch("fused_row_ct_kernel");
}

// ---------------------------------------------------------------------------
// column pass with a compile-time chain (SUM only: the squared-deviation and plain column sums)
// ---------------------------------------------------------------------------
constexpr int CT_THREADS = 256;

template <typename ChainT, int I = 0>
__device__ __forceinline__ void load_rowvec_regs(double (&rv)[ChainT::n > 0 ? ChainT::n : 1][2],
                                                 double (&ry)[ChainT::n > 0 ? ChainT::n : 1][2],
                                                 const FusedProgram &P, int64_t c0) {
    if constexpr (I < ChainT::n) {
        using St = typename At<I, ChainT>::type;
        rv[I][0] = rv[I][1] = ry[I][0] = ry[I][1] = 0.0;
        if constexpr (St::kind == FK_ROWVEC) {
            const double *src = static_cast<const double *>(P.steps[I].ptr) + c0;
            rv[I][0] = src[0];
            rv[I][1] = src[1];
            if constexpr (St::op == FO_DIV && !St::rev) {
                ry[I][0] = div_helper(rv[I][0]);
                ry[I][1] = div_helper(rv[I][1]);
            }
        } else if constexpr (St::kind == FK_SCALAR) {
            rv[I][0] = rv[I][1] = P.steps[I].imm;
            if constexpr (St::op == FO_DIV && !St::rev)
                ry[I][0] = ry[I][1] = div_helper(P.steps[I].imm);
        }
        load_rowvec_regs<ChainT, I + 1>(rv, ry, P, c0);
    }
}
template <typename ChainT, int I = 0>
__device__ __forceinline__ double col_chain(double v, int k, const double (&rv)[ChainT::n > 0 ? ChainT::n : 1][2],
                                            const double (&ry)[ChainT::n > 0 ? ChainT::n : 1][2],
                                            const FusedProgram &P, int64_t r, int64_t c) {
    if constexpr (I < ChainT::n) {
        using St = typename At<I, ChainT>::type;
        double o = rv[I][k], y = ry[I][k];
        if constexpr (St::kind == FK_COLVEC)
            o = __ldg(static_cast<const double *>(P.steps[I].ptr) + r * P.steps[I].ld);
        else if constexpr (St::kind == FK_MATRIX)
            o = __ldg(static_cast<const double *>(P.steps[I].ptr) + r * P.steps[I].ld + c);
        v = apply<St::op, St::rev>(v, o, y);
        return col_chain<ChainT, I + 1>(v, k, rv, ry, P, r, c);
    } else
        return v;
}

// blockDim = (TX, 256 / TX); requires even cols, 16-byte aligned base and even ld
template <typename ChainT>
__global__ void __launch_bounds__(CT_THREADS)
    fused_col_sum_ct_kernel(const __grid_constant__ FusedProgram P, double *__restrict__ part) {
    __shared__ double sv[CT_THREADS * 2];
    if (P.run_if && *P.run_if == 0)
        return;
    const int tx = threadIdx.x, ty = threadIdx.y, TX = blockDim.x, TY = blockDim.y;
    const int64_t rows = P.rows, cols = P.cols;
    const int64_t c0 = ((int64_t)blockIdx.y * TX + tx) * 2;
    double a0 = 0.0, a1 = 0.0, b0 = 0.0, b1 = 0.0;
    if (c0 < cols) {
        double rv[ChainT::n > 0 ? ChainT::n : 1][2], ry[ChainT::n > 0 ? ChainT::n : 1][2];
        load_rowvec_regs<ChainT>(rv, ry, P, c0);
        const double *base = static_cast<const double *>(P.base);
        const int64_t stride = (int64_t)gridDim.x * TY;
        int64_t r = (int64_t)blockIdx.x * TY + ty;
        // four rows in flight per thread (the pass is bound by memory latency); the adds keep the row order
        for (; r + 3 * stride < rows; r += 4 * stride) {
            Pack<double> p[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                p[u] = ld_pack_stream(base + (r + u * stride) * P.base_ld + c0);
            double v0[4], v1[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                v0[u] = col_chain<ChainT>(p[u].v[0], 0, rv, ry, P, r + u * stride, c0);
                v1[u] = col_chain<ChainT>(p[u].v[1], 1, rv, ry, P, r + u * stride, c0 + 1);
            }
            a0 = __dadd_rn(a0, v0[0]);
            a1 = __dadd_rn(a1, v1[0]);
            b0 = __dadd_rn(b0, v0[1]);
            b1 = __dadd_rn(b1, v1[1]);
            a0 = __dadd_rn(a0, v0[2]);
            a1 = __dadd_rn(a1, v1[2]);
            b0 = __dadd_rn(b0, v0[3]);
            b1 = __dadd_rn(b1, v1[3]);
        }
        for (; r + stride < rows; r += 2 * stride) {
            const Pack<double> p = ld_pack_stream(base + r * P.base_ld + c0);
            const Pack<double> q = ld_pack_stream(base + (r + stride) * P.base_ld + c0);
            a0 = __dadd_rn(a0, col_chain<ChainT>(p.v[0], 0, rv, ry, P, r, c0));
            a1 = __dadd_rn(a1, col_chain<ChainT>(p.v[1], 1, rv, ry, P, r, c0 + 1));
            b0 = __dadd_rn(b0, col_chain<ChainT>(q.v[0], 0, rv, ry, P, r + stride, c0));
            b1 = __dadd_rn(b1, col_chain<ChainT>(q.v[1], 1, rv, ry, P, r + stride, c0 + 1));
        }
        for (; r < rows; r += stride) {
            const Pack<double> p = ld_pack_stream(base + r * P.base_ld + c0);
            a0 = __dadd_rn(a0, col_chain<ChainT>(p.v[0], 0, rv, ry, P, r, c0));
            a1 = __dadd_rn(a1, col_chain<ChainT>(p.v[1], 1, rv, ry, P, r, c0 + 1));
        }
    }
    sv[(ty * TX + tx) * 2] = __dadd_rn(a0, b0);
    sv[(ty * TX + tx) * 2 + 1] = __dadd_rn(a1, b1);
    __syncthreads();
    for (int k = ty; k < 2; k += TY) {
        if (c0 + k < cols) {
            double a = sv[tx * 2 + k];
            for (int y = 1; y < TY; y++)
                a = __dadd_rn(a, sv[(y * TX + tx) * 2 + k]);
            part[(int64_t)blockIdx.x * cols + c0 + k] = a;
        }
    }
}

__global__ void col_sum_final_kernel(const double *__restrict__ part, int nparts, int64_t cols, int64_t count,
                                     int mean, double *__restrict__ res, const int32_t *__restrict__ run_if) {
    if (run_if && *run_if == 0)
        return;
    // one warp per column: lane l adds partials l, l + 32, ... in order, then a fixed shuffle tree (deterministic)
    const int lane = threadIdx.x % 32;
    const int64_t c = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / 32;
    if (c >= cols)
        return;
    double a = 0.0;
    for (int i = lane; i < nparts; i += 32)
        a = (i == lane) ? part[(int64_t)i * cols + c] : __dadd_rn(a, part[(int64_t)i * cols + c]);
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1)
        a = __dadd_rn(a, shfl_xor(a, m));
    if (lane == 0)
        res[c] = mean ? __ddiv_rn(a, (double)count) : a;
}

template <typename ChainT>
static int launch_col_sum(const FusedProgram &prog, int mean, void *res, void *scratch, cudaStream_t st) {
    const int64_t packets = prog.cols / 2;
    int tx = next_pow2(packets);
    if (tx > 32)
        tx = 32;
    const int ty = CT_THREADS / tx;
    const int gy = (int)((packets + tx - 1) / tx);
    int64_t cap = ((int64_t)sm_count() * 8 + gy - 1) / gy;
    int64_t want = (prog.rows + (int64_t)ty * 8 - 1) / ((int64_t)ty * 8);
    if (want < 1)
        want = 1;
    const int gx = (int)(want < cap ? want : cap);
    double *part = static_cast<double *>(scratch);
    fused_col_sum_ct_kernel<ChainT><<<dim3(gx, gy), dim3(tx, ty), 0, st>>>(prog, part);
    DB2_TRY(after_launch("fused_col_sum_ct_kernel"));
    col_sum_final_kernel<<<(unsigned)((prog.cols * 32 + 255) / 256), 256, 0, st>>>(part, gx, prog.cols, prog.rows, mean,
                                                                            static_cast<double *>(res), prog.run_if);
    return after_launch("col_sum_final_kernel");
}

// ---------------------------------------------------------------------------
// the table of specialised programs
// ---------------------------------------------------------------------------
using SubR = S<FO_SUB, FK_ROWVEC>;
using DivR = S<FO_DIV, FK_ROWVEC>;
using AddR = S<FO_ADD, FK_ROWVEC>;
using AddC = S<FO_ADD, FK_COLVEC>;
using MulS = S<FO_MUL, FK_SCALAR>;
using SqS = S<FO_SQUARE, FK_SCALAR>;

struct RowEntry {
    const char *sig;
    int (*launch)(const FusedProgram &, cudaStream_t);
};
static const RowEntry ROW_TABLE[] = {
    // column standardisation: Z = (X - mu) / sd; rowSums(Z^2), rowMaxs(Z), idxMax(Z) in one sweep, and its parts
    {"SUB.R|DIV.R|SQ.S#MAX@2,SUM@3", &launch_row<Chain<SubR, DivR, SqS>, Taps<T<2, FT_MAX>, T<3, FT_SUM>>, false>},
    {"SUB.R|DIV.R|SQ.S#SUM@3", &launch_row<Chain<SubR, DivR, SqS>, Taps<T<3, FT_SUM>>, false>},
    {"SUB.R|DIV.R#MAX@2", &launch_row<Chain<SubR, DivR>, Taps<T<2, FT_MAX>>, false>},
    {"SUB.R|DIV.R#+EW", &launch_row<Chain<SubR, DivR>, Taps<>, true>},
    {"SUB.R|DIV.R#MAX@2+EW", &launch_row<Chain<SubR, DivR>, Taps<T<2, FT_MAX>>, true>},
    // plain row aggregations of a matrix
    {"#SUM@0", &launch_row<Chain<>, Taps<T<0, FT_SUM>>, false>},
    {"#MIN@0", &launch_row<Chain<>, Taps<T<0, FT_MIN>>, false>},
    {"#MAX@0", &launch_row<Chain<>, Taps<T<0, FT_MAX>>, false>},
    {"#MEAN@0", &launch_row<Chain<>, Taps<T<0, FT_MEAN>>, false>},
    {"#SUM@0,MAX@0", &launch_row<Chain<>, Taps<T<0, FT_SUM>, T<0, FT_MAX>>, false>},
    {"#MIN@0,MAX@0", &launch_row<Chain<>, Taps<T<0, FT_MIN>, T<0, FT_MAX>>, false>},
    {"SQ.S#SUM@1", &launch_row<Chain<SqS>, Taps<T<1, FT_SUM>>, false>},
    // k-means distances: D = (X @ t(C)) * -2 + rowSums(X^2) + t(rowSums(C^2)); argmin per row
    {"MUL.S|ADD.C|ADD.R#MIN@3", &launch_row<Chain<MulS, AddC, AddR>, Taps<T<3, FT_MIN>>, false>},
    {"MUL.S|ADD.R#MIN@2", &launch_row<Chain<MulS, AddR>, Taps<T<2, FT_MIN>>, false>},
};

struct ColEntry {
    const char *sig;
    int (*launch)(const FusedProgram &, int, void *, void *, cudaStream_t);
};
static const ColEntry COL_TABLE[] = {
    {"SUB.R|SQ.S#", &launch_col_sum<Chain<SubR, SqS>>}, // column sums of squared deviations (variance)
    {"SQ.S#", &launch_col_sum<Chain<SqS>>},
    {"MUL.C#", &launch_col_sum<Chain<S<FO_MUL, FK_COLVEC>>>}, // t(X) y as column sums of X .* y
    {"#", &launch_col_sum<Chain<>>},
};

} // namespace ct

static bool ct_layout_ok(const FusedProgram &P) {
    if (!aligned16(P.base) || (P.base_ld & 1) || (P.cols & 1) || P.rows <= 0 || P.cols <= 0)
        return false;
    for (int i = 0; i < P.nsteps; i++)
        if (P.steps[i].kind == FK_ROWVEC && P.steps[i].smem_off < 0)
            return false; // row vectors too large to stage
    return true;
}

bool fused_row_pass_ct(const FusedProgram &P, const char *signature, cudaStream_t st, int *rc) {
    if (!ct_layout_ok(P))
        return false;
    if (P.ew_out && (!aligned16(P.ew_out) || (P.ew_out_ld & 1)))
        return false;
    for (const auto &e : ct::ROW_TABLE)
        if (strcmp(e.sig, signature) == 0) {
            *rc = e.launch(P, st);
            return true;
        }
    // not in the table: the kernel compiled for this chain at run time, once that exists (fused_rtc.cu) ...
    if (fused_row_pass_rtc(P, st, rc))
        return true;
    // ... and until then the same kernel with the chain read at run time
    *rc = P.ew_out ? ct::launch_row<ct::AnyChain, ct::AnyTaps, true>(P, st)
                   : ct::launch_row<ct::AnyChain, ct::AnyTaps, false>(P, st);
    return true;
}

bool fused_col_pass_ct(const FusedProgram &P, const char *signature, int agg_op, void *res, void *scratch,
                       size_t scratch_bytes, cudaStream_t st, int *rc) {
    if (agg_op != DB2_AGG_SUM && agg_op != DB2_AGG_MEAN)
        return false;
    if (!ct_layout_ok(P) || scratch_bytes < fused_col_scratch_bytes(P.cols))
        return false;
    for (const auto &e : ct::COL_TABLE)
        if (strcmp(e.sig, signature) == 0) {
            *rc = e.launch(P, agg_op == DB2_AGG_MEAN ? 1 : 0, res, scratch, st);
            return true;
        }
    return false;
}

} // namespace db2
