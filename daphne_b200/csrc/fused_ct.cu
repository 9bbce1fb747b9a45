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

} // namespace ct

// launch geometry of the column pass: blockDim = (tx, 256 / tx), grid = (gx row slices, gy column slices)
void fused_col_geometry(const FusedProgram &prog, unsigned (&grid)[2], unsigned (&block)[2]) {
    const int64_t packets = prog.cols / 2;
    int tx = next_pow2(packets);
    if (tx > 32)
        tx = 32;
    const int ty = ct::CT_THREADS / tx;
    const int gy = (int)((packets + tx - 1) / tx);
    int64_t cap = ((int64_t)sm_count() * 8 + gy - 1) / gy;
    int64_t want = (prog.rows + (int64_t)ty * 8 - 1) / ((int64_t)ty * 8);
    if (want < 1)
        want = 1;
    grid[0] = (unsigned)(want < cap ? want : cap);
    grid[1] = (unsigned)gy;
    block[0] = (unsigned)tx;
    block[1] = (unsigned)ty;
}
// the partial sums of `parts` row slices (scratch) -> res
int fused_col_finish(const FusedProgram &prog, unsigned parts, int mean, void *res, void *scratch, cudaStream_t st) {
    ct::col_sum_final_kernel<<<(unsigned)((prog.cols * 32 + 255) / 256), 256, 0, st>>>(
        static_cast<const double *>(scratch), (int)parts, prog.cols, prog.rows, mean, static_cast<double *>(res),
        prog.run_if);
    return after_launch("col_sum_final_kernel");
}

namespace ct {

template <typename ChainT>
static int launch_col_sum(const FusedProgram &prog, int mean, void *res, void *scratch, cudaStream_t st) {
    unsigned grid[2], block[2];
    fused_col_geometry(prog, grid, block);
    fused_col_sum_ct_kernel<ChainT><<<dim3(grid[0], grid[1]), dim3(block[0], block[1]), 0, st>>>(
        prog, static_cast<double *>(scratch));
    DB2_TRY(after_launch("fused_col_sum_ct_kernel"));
    return fused_col_finish(prog, grid[0], mean, res, scratch, st);
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

static bool ct_staged(const FusedProgram &P) {
    if (P.rows <= 0 || P.cols <= 0)
        return false;
    for (int i = 0; i < P.nsteps; i++)
        if (P.steps[i].kind == FK_ROWVEC && P.steps[i].smem_off < 0)
            return false; // row vectors too large to stage
    return true;
}
// rows start on 16-byte boundaries and hold an even number of values: the 16-byte copies of the compiled-in kernels
static bool ct_layout_ok(const FusedProgram &P) {
    return ct_staged(P) && aligned16(P.base) && !(P.base_ld & 1) && !(P.cols & 1);
}

bool fused_row_pass_ct(const FusedProgram &P, const char *signature, cudaStream_t st, int *rc) {
    if (!ct_staged(P))
        return false;
    if (!ct_layout_ok(P) || (P.ew_out && (!aligned16(P.ew_out) || (P.ew_out_ld & 1)))) {
        // any other layout (odd number of columns, odd leading dimension, a view that starts at an odd column): the
        // kernel compiled at run time in its copy-by-element form; until that exists, the general interpreter
        return (reinterpret_cast<uintptr_t>(P.base) & 7) == 0 && fused_row_pass_rtc(P, false, st, rc);
    }
    for (const auto &e : ct::ROW_TABLE)
        if (strcmp(e.sig, signature) == 0) {
            *rc = e.launch(P, st);
            return true;
        }
    // not in the table: the kernel compiled for this chain at run time, once that exists (fused_rtc.cu) ...
    if (fused_row_pass_rtc(P, true, st, rc))
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
    // not in the table: the kernel compiled for this chain at run time, once it exists; until then the general pass
    return fused_col_pass_rtc(P, agg_op == DB2_AGG_MEAN ? 1 : 0, res, scratch, st, rc);
}

} // namespace db2
