// Compile-time specialisations of the fused passes (fused.cuh) for the chains the benchmark pipelines produce.
//
// The interpreter in fused.cu spends most of its instructions on decoding; for a chain known at compile time the
// per-element work shrinks to the arithmetic itself, which is what lets the standardisation pass run at HBM speed
// on a part whose FP64 rate is only 64 instructions per SM and clock.  A chain is spelled as a type list
// (Chain<S<op, operand kind>...>, Taps<T<position, tracker kind>...>); the runtime matches the signature string of a
// recorded program against the table at the end of this file and falls back to the interpreter otherwise.  Adding a
// pattern is one table line.
//
// Row pass layout: CTA = 128 threads = 128 rows per tile, 32 columns per chunk.  The tile is brought into shared
// memory with 16-byte cp.async copies (no register staging) into an XOR-swizzled layout -- 16-byte slot p of row r
// lives at slot p ^ (r & 15) -- so that the cooperative (coalesced) fill and the one-row-per-thread walk are both
// bank-conflict free without padding.  Every thread then walks its row with 128-bit shared loads, applies the chain
// and feeds its row trackers; results leave one row per thread (coalesced).  No cross-lane reduction exists.
#include "fused.cuh"
#include "ops.cuh"

#include <cstring>

namespace db2 {
namespace ct {

constexpr int RT = 128;
constexpr int CK = 32;
constexpr int NO_COL = 0x7fffffff;

template <int OP, int KIND, bool REV = false> struct S {
    static constexpr int op = OP, kind = KIND;
    static constexpr bool rev = REV;
};
template <typename... Ss> struct Chain {
    static constexpr int n = sizeof...(Ss);
};
template <int AFTER, int TK> struct T {
    static constexpr int after = AFTER, kind = TK;
};
template <typename... Ts> struct Taps {
    static constexpr int n = sizeof...(Ts);
};
template <int I, typename L> struct At;
template <int I, template <typename...> class L, typename H, typename... R> struct At<I, L<H, R...>> {
    using type = typename At<I - 1, L<R...>>::type;
};
template <template <typename...> class L, typename H, typename... R> struct At<0, L<H, R...>> {
    using type = H;
};

__device__ __forceinline__ bool safe_divisor(double d) {
    const unsigned hi = (unsigned)__double2hiint(d), lo = (unsigned)__double2loint(d);
    const int e = (hi >> 20) & 0x7ff;
    const bool all_ones = ((hi & 0xfffffu) == 0xfffffu) && (lo == 0xffffffffu);
    return e > 923 && e < 1123 && !all_ones;
}
__device__ __forceinline__ double div_helper(double d) { return safe_divisor(d) ? __drcp_rn(d) : 0.0; }
// a / d from the staged reciprocal y = RN(1/d) (0.0 = not applicable); see fused.cu for the argument
__device__ __forceinline__ double fast_div(double a, double d, double y) {
    const int ea = (__double2hiint(a) >> 20) & 0x7ff;
    if (y != 0.0) {
        if (ea > 123 && ea < 1923) {
            const double q = __dmul_rn(a, y);
            const double r = __fma_rn(-q, d, a);
            return __fma_rn(r, y, q);
        }
        if (a == 0.0)
            return __dmul_rn(a, y);
    }
    return __ddiv_rn(a, d);
}

template <int OP, bool REV> __device__ __forceinline__ double apply(double a, double b, double y) {
    const double l = REV ? b : a, r = REV ? a : b;
    if constexpr (OP == FO_ADD) return __dadd_rn(l, r);
    else if constexpr (OP == FO_SUB) return __dsub_rn(l, r);
    else if constexpr (OP == FO_MUL) return __dmul_rn(l, r);
    else if constexpr (OP == FO_DIV) return REV ? __ddiv_rn(l, r) : fast_div(a, b, y);
    else if constexpr (OP == FO_SQUARE) return __dmul_rn(a, a);
    else if constexpr (OP == FO_EQ) return (double)(l == r);
    else if constexpr (OP == FO_NEQ) return (double)(l != r);
    else if constexpr (OP == FO_LT) return (double)(l < r);
    else if constexpr (OP == FO_LE) return (double)(l <= r);
    else if constexpr (OP == FO_GT) return (double)(l > r);
    else if constexpr (OP == FO_GE) return (double)(l >= r);
    else if constexpr (OP == FO_MIN) return (r < l) ? r : l;
    else if constexpr (OP == FO_MAX) return (l < r) ? r : l;
    else if constexpr (OP == FO_NEG) return -a;
    else if constexpr (OP == FO_ABS) return fabs(a);
    else return a;
}

// per-thread state of a chain: aux[i] = reciprocal helper of a SCALAR divisor, or the row's COLVEC operand
template <typename ChainT> struct ChainState {
    double aux[ChainT::n > 0 ? ChainT::n : 1];
};
template <typename TapsT> struct TapState {
    double v[TapsT::n > 0 ? TapsT::n : 1];
    double first[TapsT::n > 0 ? TapsT::n : 1];
    int c[TapsT::n > 0 ? TapsT::n : 1];
};

template <typename TapsT, int AFTER, int J = 0>
__device__ __forceinline__ void feed(TapState<TapsT> &ts, double v, int c) {
    if constexpr (J < TapsT::n) {
        using Tp = typename At<J, TapsT>::type;
        if constexpr (Tp::after == AFTER) {
            if constexpr (Tp::kind == FT_SUM || Tp::kind == FT_MEAN)
                ts.v[J] = __dadd_rn(ts.v[J], v);
            else if constexpr (Tp::kind == FT_PROD)
                ts.v[J] = __dmul_rn(ts.v[J], v);
            else {
                if (c == 0)
                    ts.first[J] = v;
                const bool better = (Tp::kind == FT_MIN) ? (v < ts.v[J]) : (v > ts.v[J]);
                if (better) {
                    ts.v[J] = v;
                    ts.c[J] = c;
                }
            }
        }
        feed<TapsT, AFTER, J + 1>(ts, v, c);
    }
}

template <typename ChainT, typename TapsT, int I = 0>
__device__ __forceinline__ double run_chain(double v, const FusedProgram &P, const ChainState<ChainT> &cs,
                                            TapState<TapsT> &ts, const double *rvs, int64_t row, int64_t c) {
    if constexpr (I == 0)
        feed<TapsT, 0>(ts, v, (int)c);
    if constexpr (I < ChainT::n) {
        using St = typename At<I, ChainT>::type;
        const FusedStep &fs = P.steps[I];
        double o = 0.0, y = 0.0;
        if constexpr (St::kind == FK_ROWVEC) {
            o = rvs[fs.smem_off + c];
            if constexpr (St::op == FO_DIV && !St::rev)
                y = rvs[fs.smem_off + P.cols + c];
        } else if constexpr (St::kind == FK_SCALAR) {
            o = fs.imm;
            y = cs.aux[I];
        } else if constexpr (St::kind == FK_COLVEC) {
            o = cs.aux[I];
        } else if constexpr (St::kind == FK_MATRIX) {
            o = __ldg(static_cast<const double *>(fs.ptr) + row * fs.ld + c);
        }
        v = apply<St::op, St::rev>(v, o, y);
        feed<TapsT, I + 1>(ts, v, (int)c);
        return run_chain<ChainT, TapsT, I + 1>(v, P, cs, ts, rvs, row, c);
    } else
        return v;
}

template <typename ChainT, int I = 0>
__device__ __forceinline__ void init_scalar_aux(ChainState<ChainT> &cs, const FusedProgram &P) {
    if constexpr (I < ChainT::n) {
        using St = typename At<I, ChainT>::type;
        cs.aux[I] = 0.0;
        if constexpr (St::kind == FK_SCALAR && St::op == FO_DIV && !St::rev)
            cs.aux[I] = div_helper(P.steps[I].imm);
        init_scalar_aux<ChainT, I + 1>(cs, P);
    }
}
template <typename ChainT, int I = 0>
__device__ __forceinline__ void load_colvec_aux(ChainState<ChainT> &cs, const FusedProgram &P, int64_t row) {
    if constexpr (I < ChainT::n) {
        using St = typename At<I, ChainT>::type;
        if constexpr (St::kind == FK_COLVEC)
            cs.aux[I] = __ldg(static_cast<const double *>(P.steps[I].ptr) + row * P.steps[I].ld);
        load_colvec_aux<ChainT, I + 1>(cs, P, row);
    }
}
template <typename TapsT, int J = 0> __device__ __forceinline__ void init_taps(TapState<TapsT> &ts) {
    if constexpr (J < TapsT::n) {
        using Tp = typename At<J, TapsT>::type;
        ts.v[J] = (Tp::kind == FT_PROD) ? 1.0 : (Tp::kind == FT_MIN) ? INFINITY : (Tp::kind == FT_MAX) ? -INFINITY : 0.0;
        ts.first[J] = 0.0;
        ts.c[J] = NO_COL;
        init_taps<TapsT, J + 1>(ts);
    }
}
template <typename TapsT, int J = 0>
__device__ __forceinline__ void write_taps(const TapState<TapsT> &ts, const FusedProgram &P, int64_t row) {
    if constexpr (J < TapsT::n) {
        using Tp = typename At<J, TapsT>::type;
        double v = ts.v[J];
        int c = ts.c[J];
        if constexpr (Tp::kind == FT_MIN || Tp::kind == FT_MAX) {
            // the reference's scan starts from element 0 and only moves on a strict improvement: when nothing
            // improved on the start value (or element 0 is a NaN) the answer is element 0
            if (c == NO_COL || ts.first[J] != ts.first[J]) {
                v = ts.first[J];
                c = 0;
            }
            if (P.taps[J].out_idx)
                static_cast<uint64_t *>(P.taps[J].out_idx)[row] = (uint64_t)c;
        }
        if constexpr (Tp::kind == FT_MEAN)
            v = __ddiv_rn(v, (double)P.cols);
        if (P.taps[J].out)
            static_cast<double *>(P.taps[J].out)[row] = v;
        write_taps<TapsT, J + 1>(ts, P, row);
    }
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

template <typename ChainT, typename TapsT, bool EW>
__global__ void __launch_bounds__(RT, 5) fused_row_ct_kernel(const __grid_constant__ FusedProgram P) {
    extern __shared__ __align__(16) double smem[];
    double *tile = smem;           // [RT][CK], 16-byte slots swizzled by row
    double *rvs = smem + RT * CK;  // staged row-vector operands (+ reciprocal helpers)
    const int tid = threadIdx.x;
    const int64_t rows = P.rows, cols = P.cols;
    for (int s = 0; s < P.nsteps; s++) {
        const FusedStep &st = P.steps[s];
        if (st.kind == FK_ROWVEC) {
            const double *src = static_cast<const double *>(st.ptr);
            const bool helper = (st.op == FO_DIV && !st.reversed);
            for (int64_t c = tid; c < cols; c += RT) {
                const double d = src[c];
                rvs[st.smem_off + c] = d;
                if (helper)
                    rvs[st.smem_off + cols + c] = div_helper(d);
            }
        }
    }
    ChainState<ChainT> cs;
    init_scalar_aux<ChainT>(cs, P);
    __syncthreads();

    const double *base = static_cast<const double *>(P.base);
    const int64_t ntiles = (rows + RT - 1) / RT;
    const int swz = tid & 15;
    for (int64_t tile_i = blockIdx.x; tile_i < ntiles; tile_i += gridDim.x) {
        const int64_t row0 = tile_i * RT;
        const int64_t row = row0 + tid;
        const bool live = row < rows;
        const int rows_here = (rows - row0 < RT) ? (int)(rows - row0) : RT;
        TapState<TapsT> ts;
        init_taps<TapsT>(ts);
        if (live)
            load_colvec_aux<ChainT>(cs, P, row);
        for (int64_t cc = 0; cc < cols; cc += CK) {
            const int cw = (cols - cc < CK) ? (int)(cols - cc) : CK;
            __syncthreads(); // every reader of the previous chunk is done
#pragma unroll
            for (int i = 0; i < CK / 2; i++) {
                const int idx = tid + i * RT;
                const int r = idx >> 4, p = idx & 15;
                if (r < rows_here && 2 * p < cw)
                    cp_async16(tile + (r * 16 + (p ^ (r & 15))) * 2, base + (row0 + r) * P.base_ld + cc + 2 * p);
            }
            cp_async_wait_all();
            __syncthreads();
            if (live) {
#pragma unroll
                for (int p = 0; p < CK / 2; p++) {
                    if (2 * p < cw) {
                        double2 *slot = reinterpret_cast<double2 *>(tile + (tid * 16 + (p ^ swz)) * 2);
                        double2 xy = *slot;
                        xy.x = run_chain<ChainT, TapsT>(xy.x, P, cs, ts, rvs, row, cc + 2 * p);
                        xy.y = run_chain<ChainT, TapsT>(xy.y, P, cs, ts, rvs, row, cc + 2 * p + 1);
                        if constexpr (EW)
                            *slot = xy;
                    }
                }
            }
            if constexpr (EW) {
                __syncthreads();
                double *out = static_cast<double *>(P.ew_out);
#pragma unroll
                for (int i = 0; i < CK / 2; i++) {
                    const int idx = tid + i * RT;
                    const int r = idx >> 4, p = idx & 15;
                    if (r < rows_here && 2 * p < cw) {
                        const double2 q = *reinterpret_cast<const double2 *>(tile + (r * 16 + (p ^ (r & 15))) * 2);
                        __stcs(reinterpret_cast<double2 *>(out + (row0 + r) * P.ew_out_ld + cc + 2 * p), q);
                    }
                }
            }
        }
        if (live)
            write_taps<TapsT>(ts, P, row);
    }
}

template <typename ChainT, typename TapsT, bool EW> static int launch_row(const FusedProgram &prog, cudaStream_t st) {
    const size_t smem = (size_t)(RT * CK + prog.smem_elems) * sizeof(double);
    const int64_t ntiles = (prog.rows + RT - 1) / RT;
    const int64_t cap = (int64_t)sm_count() * 5;
    const int grid = (int)(ntiles < cap ? ntiles : cap);
    static bool attr = false;
    if (!attr) {
        DB2_CUDA(cudaFuncSetAttribute(fused_row_ct_kernel<ChainT, TapsT, EW>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
        attr = true;
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
                                     int mean, double *__restrict__ res) {
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
                                                                            static_cast<double *>(res));
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
    return false;
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
