// Device code of the row pass with a chain known at compile time (see fused_ct.cu for the layout): the chain and
// tap type lists, the per-step arithmetic, the run-time chain interpreter and the kernel template itself.  Included
// by fused_ct.cu for the specialisations that are compiled into the library, and handed as text to the run-time
// compiler for every other chain (fused_rtc.cu) -- so it includes nothing but fused_types.cuh.
#pragma once

#include "fused_types.cuh"

namespace db2 {
namespace ct {

constexpr int RT = 128;        // threads per CTA
constexpr int WR = 32;         // rows of a warp's tile = lanes
constexpr int WARPS = RT / 32;
constexpr int CK = 32;         // columns per chunk
constexpr int GR = 8;          // elements of a row evaluated together
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
template <typename A, typename B> struct same {
    static constexpr bool value = false;
};
template <typename A> struct same<A, A> {
    static constexpr bool value = true;
};

__device__ __forceinline__ bool safe_divisor(double d) {
    const unsigned hi = (unsigned)__double2hiint(d), lo = (unsigned)__double2loint(d);
    const int e = (hi >> 20) & 0x7ff;
    const bool all_ones = ((hi & 0xfffffu) == 0xfffffu) && (lo == 0xffffffffu);
    return e > 923 && e < 1123 && !all_ones;
}
// RN(1/d) for a divisor fast_div may use, NaN = "take the generic division"
__device__ __forceinline__ double div_helper(double d) {
    return safe_divisor(d) ? __drcp_rn(d) : __longlong_as_double(0x7ff8000000000000ll);
}
// a / d from the staged helper y.  The three-instruction quotient (see fused.cu for the argument) is computed
// unconditionally and accepted when its exponent lies in [2^-750, 2^750): with |d| in [2^-99, 2^100) that can only
// happen for |a| in (2^-850, 2^851), inside the window in which no intermediate over- or underflows; zeros,
// infinities, NaNs, a NaN helper and everything near the ends of the range fail the one test and are divided
// generically.  One integer test on the result replaces the tests on both operands.
constexpr unsigned FAST_DIV_WINDOW = 1500u << 20;
__device__ __forceinline__ unsigned fast_div_window_pos(double q1) {
    return ((unsigned)__double2hiint(q1) & 0x7ff00000u) - (273u << 20);
}
__device__ __forceinline__ bool in_fast_div_window(double q1) { return fast_div_window_pos(q1) < FAST_DIV_WINDOW; }
__device__ __forceinline__ double fast_div(double a, double d, double y) {
    const double q = __dmul_rn(a, y);
    const double r = __fma_rn(-q, d, a);
    const double q1 = __fma_rn(r, y, q);
    if (in_fast_div_window(q1))
        return q1;
    if (a == 0.0 && y == y)
        return __dmul_rn(a, y); // signed zero
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
    else if constexpr (OP == FO_AND) return (double)((l != 0.0) && (r != 0.0));
    else if constexpr (OP == FO_OR) return (double)((l != 0.0) || (r != 0.0));
    else if constexpr (OP == FO_NEG) return -a;
    else if constexpr (OP == FO_ABS) return fabs(a);
    else if constexpr (OP == FO_SIGN) return (a == 0) ? 0.0 : ((a < 0) ? -1.0 : ((a > 0) ? 1.0 : (double)NAN));
    else if constexpr (OP == FO_FLOOR) return floor(a);
    else if constexpr (OP == FO_CEIL) return ceil(a);
    else if constexpr (OP == FO_ROUND) return round(a);
    else if constexpr (OP == FO_ISNAN) return (double)(a != a);
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

// C0: the element may be column 0 of its row (only then is the scan's start value recorded)
template <typename TapsT, int AFTER, bool C0, int J = 0>
__device__ __forceinline__ void feed(TapState<TapsT> &ts, double v, int c) {
    if constexpr (J < TapsT::n) {
        using Tp = typename At<J, TapsT>::type;
        if constexpr (Tp::after == AFTER) {
            if constexpr (Tp::kind == FT_SUM || Tp::kind == FT_MEAN)
                ts.v[J] = __dadd_rn(ts.v[J], v);
            else if constexpr (Tp::kind == FT_PROD)
                ts.v[J] = __dmul_rn(ts.v[J], v);
            else {
                if constexpr (C0)
                    if (c == 0)
                        ts.first[J] = v;
                const bool better = (Tp::kind == FT_MIN) ? (v < ts.v[J]) : (v > ts.v[J]);
                if (better) {
                    ts.v[J] = v;
                    ts.c[J] = c;
                }
            }
        }
        feed<TapsT, AFTER, C0, J + 1>(ts, v, c);
    }
}

// ---- chains that have no entry in the table: same kernel, steps and taps read from the program at run time ----
// The data movement, the grouping and the division are those of the compiled chains; what is interpreted is the
// operand kind and the opcode, once per step and group of G elements (not per element).
struct AnyChain {
    static constexpr int n = 0; // no per-thread chain state: scalar helpers sit behind the staged row vectors
};
struct AnyTaps {
    static constexpr int n = FUSED_MAX_AGGS;
};

__device__ __forceinline__ void init_taps_rt(TapState<AnyTaps> &ts, const FusedProgram &P) {
#pragma unroll
    for (int a = 0; a < FUSED_MAX_AGGS; a++) {
        const int kind = a < P.ntaps ? P.taps[a].kind : FT_SUM;
        ts.v[a] = (kind == FT_PROD) ? 1.0 : (kind == FT_MIN) ? INFINITY : (kind == FT_MAX) ? -INFINITY : 0.0;
        ts.first[a] = 0.0;
        ts.c[a] = NO_COL;
    }
}
__device__ __forceinline__ void write_taps_rt(const TapState<AnyTaps> &ts, const FusedProgram &P, int64_t row) {
#pragma unroll
    for (int a = 0; a < FUSED_MAX_AGGS; a++) {
        if (a < P.ntaps) {
            const int kind = P.taps[a].kind;
            double v = ts.v[a];
            int c = ts.c[a];
            if (kind == FT_MIN || kind == FT_MAX) {
                if (c == NO_COL || ts.first[a] != ts.first[a]) { // see write_taps
                    v = ts.first[a];
                    c = 0;
                }
                if (P.taps[a].out_idx)
                    static_cast<uint64_t *>(P.taps[a].out_idx)[row] = (uint64_t)c;
            }
            if (kind == FT_MEAN)
                v = __ddiv_rn(v, (double)P.cols);
            if (P.taps[a].out)
                static_cast<double *>(P.taps[a].out)[row] = v;
        }
    }
}

// The chain on G consecutive elements of one row, step by step: G independent dependency chains for the scheduler to
// interleave (an element at a time, the latency of the FP64 pipe would be exposed on every step).  The division's
// range test is folded over the group, so the rare generic division costs one branch per group instead of a branch
// per element that would fence the chains off from one another.  Taps are fed in element order.
template <typename TapsT, int AFTER, bool C0, int G>
__device__ __forceinline__ void feed_group(TapState<TapsT> &ts, const double (&v)[G], int c0) {
    if constexpr (TapsT::n > 0) {
        feed<TapsT, AFTER, C0>(ts, v[0], c0);
#pragma unroll
        for (int i = 1; i < G; i++)
            feed<TapsT, AFTER, false>(ts, v[i], c0 + i);
    }
}
template <typename ChainT, typename TapsT, bool C0, int G, int I = 0>
__device__ __forceinline__ void run_group(double (&v)[G], const FusedProgram &P, const ChainState<ChainT> &cs,
                                          TapState<TapsT> &ts, const double *rvs, int64_t row, int64_t c) {
    {
    if constexpr (I == 0)
        feed_group<TapsT, 0, C0, G>(ts, v, (int)c);
    if constexpr (I < ChainT::n) {
        using St = typename At<I, ChainT>::type;
        const FusedStep &fs = P.steps[I];
        double o[G], y[G];
        if constexpr (St::kind == FK_ROWVEC && G == 1) { // the last column of a row with an odd number of columns
            o[0] = rvs[fs.smem_off + c];
            y[0] = 0.0;
            if constexpr (St::op == FO_DIV && !St::rev)
                y[0] = rvs[fs.smem_off + ((P.cols + 1) & ~(int64_t)1) + c];
        } else if constexpr (St::kind == FK_ROWVEC) {
            // staged operands: offsets and c are even, so pairs are 16-byte aligned
            const double2 *ov = reinterpret_cast<const double2 *>(rvs + fs.smem_off + c);
            const double2 *yv = reinterpret_cast<const double2 *>(rvs + fs.smem_off + ((P.cols + 1) & ~(int64_t)1) + c);
#pragma unroll
            for (int i = 0; i < G / 2; i++) {
                const double2 t = ov[i];
                o[2 * i] = t.x;
                o[2 * i + 1] = t.y;
                y[2 * i] = y[2 * i + 1] = 0.0;
                if constexpr (St::op == FO_DIV && !St::rev) {
                    const double2 u = yv[i];
                    y[2 * i] = u.x;
                    y[2 * i + 1] = u.y;
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < G; i++) {
                o[i] = 0.0;
                y[i] = 0.0;
                if constexpr (St::kind == FK_SCALAR) {
                    o[i] = fs.imm;
                    y[i] = cs.aux[I];
                } else if constexpr (St::kind == FK_COLVEC) {
                    o[i] = cs.aux[I];
                } else if constexpr (St::kind == FK_MATRIX) {
                    o[i] = __ldg(static_cast<const double *>(fs.ptr) + row * fs.ld + c + i);
                }
            }
        }
        // a reciprocal helper is staged for row-vector and scalar divisors only; any other divisor is divided by
        constexpr bool HELPED = St::op == FO_DIV && !St::rev && (St::kind == FK_ROWVEC || St::kind == FK_SCALAR);
        if constexpr (St::op == FO_DIV && !St::rev && !HELPED) {
#pragma unroll
            for (int i = 0; i < G; i++)
                v[i] = __ddiv_rn(v[i], o[i]);
        } else if constexpr (HELPED) {
            double q1[G];
            unsigned worst = 0; // the largest distance from the window's lower end, as an unsigned number
#pragma unroll
            for (int i = 0; i < G; i++) {
                const double q = __dmul_rn(v[i], y[i]);
                const double r = __fma_rn(-q, o[i], v[i]);
                q1[i] = __fma_rn(r, y[i], q);
                worst = max(worst, fast_div_window_pos(q1[i]));
            }
            if (worst < FAST_DIV_WINDOW) {
#pragma unroll
                for (int i = 0; i < G; i++)
                    v[i] = q1[i];
            } else {
#pragma unroll
                for (int i = 0; i < G; i++)
                    v[i] = fast_div(v[i], o[i], y[i]);
            }
        } else {
#pragma unroll
            for (int i = 0; i < G; i++)
                v[i] = apply<St::op, St::rev>(v[i], o[i], y[i]);
        }
        feed_group<TapsT, I + 1, C0, G>(ts, v, (int)c);
        run_group<ChainT, TapsT, C0, G, I + 1>(v, P, cs, ts, rvs, row, c);
    }
    } // compiled chain
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

__device__ __forceinline__ void cp_async16(unsigned smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::: "memory"); }
__device__ __forceinline__ double2 lds128(unsigned a) {
    double2 v;
    asm volatile("ld.shared.v2.f64 {%0, %1}, [%2];\n" : "=d"(v.x), "=d"(v.y) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void sts128(unsigned a, double x, double y) {
    asm volatile("st.shared.v2.f64 [%0], {%1, %2};\n" ::"r"(a), "d"(x), "d"(y) : "memory");
}

// A chunk buffer holds WR rows of 256 bytes and starts on a 256-byte boundary; 16-byte slot p of row r lives at slot
// p ^ (r & 15).  With the buffer aligned, both address patterns below reduce to one XOR with an immediate:
//   cooperative (fill, store): lane -> rows r0 + 2 i (r0 = lane / 16), slot p = lane % 16:
//       address = ((buf + 256 r0 + 16 (p ^ r0)) ^ (16 (2 i % 16))) + 512 i
//   walk: lane = row, slot p:  address = (buf + 256 lane + 16 (lane % 16)) ^ (16 p)
__device__ __forceinline__ unsigned coop_addr(unsigned coop0, int i) {
    return (coop0 ^ (unsigned)(((2 * i) & 15) << 4)) + (unsigned)(512 * i);
}

// copies of one chunk (rows_here x cw of the WR x CK window at src) by one warp
template <bool FULL>
__device__ __forceinline__ void issue_chunk(unsigned coop0, const double *src, int64_t ld, int rows_here, int cw,
                                            int lane) {
    const int r0 = lane >> 4, p = lane & 15;
    const double *s = src + r0 * ld + 2 * p;
#pragma unroll
    for (int i = 0; i < CK / 2; i++)
        if (FULL || (r0 + 2 * i < rows_here && 2 * p < cw))
            cp_async16(coop_addr(coop0, i), s + (int64_t)(2 * i) * ld);
}

// The same chunk for a source whose rows do not start on 16-byte boundaries (odd leading dimension, odd number of
// columns, or a base that is only 8-byte aligned): one 8-byte copy per element, lane = column, so that a row of the
// chunk is still one 256-byte request; element (r, c) lands where the 16-byte form puts it.
__device__ __forceinline__ void cp_async8(unsigned smem_dst, const void *gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ unsigned elem_addr(unsigned buf, int r, int lane) {
    return buf + (unsigned)(256 * r + ((((lane >> 1) ^ r) & 15) << 4) + ((lane & 1) << 3));
}
template <bool FULL>
__device__ __forceinline__ void issue_chunk_by_element(unsigned buf, const double *src, int64_t ld, int rows_here, int cw,
                                                       int lane) {
    const double *s = src + lane;
#pragma unroll
    for (int r = 0; r < WR; r++)
        if (FULL || (r < rows_here && lane < cw))
            cp_async8(elem_addr(buf, r, lane), s + (int64_t)r * ld);
}

// one lane walks its row of a chunk (FULL: all CK columns are there)
template <typename ChainT, typename TapsT, bool EW, bool FULL>
__device__ __forceinline__ void walk_row(unsigned walk0, const FusedProgram &P, const ChainState<ChainT> &cs,
                                         TapState<TapsT> &ts, const double *rvs, int64_t row, int64_t cc, int cw) {
#pragma unroll
    for (int g = 0; g < CK / GR; g++) {
        if (FULL || g * GR < cw) { // a group that straddles the end loads padding it never uses
            double v[GR];
#pragma unroll
            for (int j = 0; j < GR / 2; j++) {
                const double2 xy = lds128(walk0 ^ (unsigned)((g * (GR / 2) + j) << 4));
                v[2 * j] = xy.x;
                v[2 * j + 1] = xy.y;
            }
            if (FULL || g * GR + GR <= cw) {
                if (g == 0)
                    run_group<ChainT, TapsT, true, GR>(v, P, cs, ts, rvs, row, cc);
                else
                    run_group<ChainT, TapsT, false, GR>(v, P, cs, ts, rvs, row, cc + g * GR);
            } else { // ragged end of the last chunk: pairs
#pragma unroll
                for (int j = 0; j < GR / 2; j++) {
                    if (g * GR + 2 * j + 1 < cw) {
                        double w[2] = {v[2 * j], v[2 * j + 1]};
                        if (g == 0 && j == 0)
                            run_group<ChainT, TapsT, true, 2>(w, P, cs, ts, rvs, row, cc);
                        else
                            run_group<ChainT, TapsT, false, 2>(w, P, cs, ts, rvs, row, cc + g * GR + 2 * j);
                        v[2 * j] = w[0];
                        v[2 * j + 1] = w[1];
                    } else if (g * GR + 2 * j < cw) { // the last column of a row with an odd number of columns
                        double w[1] = {v[2 * j]};
                        if (g == 0 && j == 0)
                            run_group<ChainT, TapsT, true, 1>(w, P, cs, ts, rvs, row, cc);
                        else
                            run_group<ChainT, TapsT, false, 1>(w, P, cs, ts, rvs, row, cc + g * GR + 2 * j);
                        v[2 * j] = w[0];
                    }
                }
            }
            if constexpr (EW) {
#pragma unroll
                for (int j = 0; j < GR / 2; j++)
                    if (FULL || g * GR + 2 * j < cw)
                        sts128(walk0 ^ (unsigned)((g * (GR / 2) + j) << 4), v[2 * j], v[2 * j + 1]);
            }
        }
    }
}

// ---- run-time chains: one lane applies the steps to its row of a chunk IN PLACE, step by step ----
// The row's CK elements sit in the warp's chunk buffer in shared memory.  A step is a function of its own per
// (opcode, operand order, operand kind): it reads the row 8 elements at a time, applies the operation and writes
// the row back, so nothing is live in registers from one step to the next and no two steps share code paths that
// would have to agree on registers.  (Holding the row in registers through one `switch` per step cost 48
// instructions per element, 14 of them register moves where the cases meet; this form costs a third of that.)
// A step's description -- opcode, operand kind, operand address -- is decoded once per CK elements.  Scalar helpers
// and tap masks sit behind the staged row vectors:
//   rvs[smem_elems + s]                    division helper of step s (SCALAR operands)
//   rvs[smem_elems + FUSED_MAX_STEPS + s]  (as bits) mask of the taps that follow s steps
struct RtOperand {
    unsigned vec;       // ROWVEC: shared-memory address of the staged operand at this chunk's first column (its
                        // division helpers follow `cols` elements further on)
    const double *mat;  // MATRIX: this row's operand at the chunk's first column
    double scal, yscal; // SCALAR / COLVEC operand and its division helper
    int64_t cols;
    int cw; // columns of the chunk that exist (even)
};

// one group of GR elements of the row; WHOLE: all of them exist (no column tests)
template <int OP, bool REV, int KIND, bool WHOLE>
__device__ __forceinline__ void rt_step_group(unsigned walk0, const RtOperand &so, int g) {
    double v[GR], o[GR], y[GR];
#pragma unroll
    for (int j = 0; j < GR / 2; j++) {
        const double2 xy = lds128(walk0 ^ (unsigned)((g * (GR / 2) + j) << 4));
        v[2 * j] = xy.x;
        v[2 * j + 1] = xy.y;
    }
    if constexpr (KIND == FK_ROWVEC) {
#pragma unroll
        for (int j = 0; j < GR / 2; j++) {
            o[2 * j] = o[2 * j + 1] = y[2 * j] = y[2 * j + 1] = 0.0;
            if (WHOLE || g * GR + 2 * j < so.cw) {
                const double2 t = lds128(so.vec + (unsigned)((g * GR + 2 * j) * 8));
                o[2 * j] = t.x;
                o[2 * j + 1] = t.y;
                if constexpr (OP == FO_DIV && !REV) {
                    const double2 u = lds128(so.vec + (unsigned)((so.cols + g * GR + 2 * j) * 8));
                    y[2 * j] = u.x;
                    y[2 * j + 1] = u.y;
                }
            }
        }
    } else if constexpr (KIND == FK_MATRIX) {
#pragma unroll
        for (int i = 0; i < GR; i++) {
            o[i] = (WHOLE || g * GR + i < so.cw) ? __ldg(so.mat + g * GR + i) : 0.0;
            y[i] = __longlong_as_double(0x7ff8000000000000ll); // no helper: generic division
        }
    } else {
#pragma unroll
        for (int i = 0; i < GR; i++) {
            o[i] = so.scal;
            y[i] = so.yscal;
        }
    }
    if constexpr (OP == FO_DIV && !REV) {
        double q1[GR];
        unsigned worst = 0;
#pragma unroll
        for (int i = 0; i < GR; i++) {
            const double q = __dmul_rn(v[i], y[i]);
            const double r = __fma_rn(-q, o[i], v[i]);
            q1[i] = __fma_rn(r, y[i], q);
            worst = max(worst, fast_div_window_pos(q1[i]));
        }
        if (worst < FAST_DIV_WINDOW) {
#pragma unroll
            for (int i = 0; i < GR; i++)
                v[i] = q1[i];
        } else {
#pragma unroll
            for (int i = 0; i < GR; i++)
                v[i] = fast_div(v[i], o[i], y[i]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < GR; i++)
            v[i] = apply<OP, REV>(v[i], o[i], 0.0);
    }
#pragma unroll
    for (int j = 0; j < GR / 2; j++)
        sts128(walk0 ^ (unsigned)((g * (GR / 2) + j) << 4), v[2 * j], v[2 * j + 1]);
}

template <int OP, bool REV, int KIND>
__device__ __noinline__ void rt_step(unsigned walk0, const RtOperand so) {
    if (so.cw == CK) { // the usual case: all columns of the chunk exist
#pragma unroll
        for (int g = 0; g < CK / GR; g++)
            rt_step_group<OP, REV, KIND, true>(walk0, so, g);
    } else {
#pragma unroll 1
        for (int g = 0; g * GR < so.cw; g++) // a group that straddles the end works on padding nobody reads
            rt_step_group<OP, REV, KIND, false>(walk0, so, g);
    }
}

template <int OP, bool REV>
__device__ __forceinline__ void rt_step_kind(int kind, unsigned walk0, const RtOperand &so) {
    if (kind == FK_ROWVEC)
        rt_step<OP, REV, FK_ROWVEC>(walk0, so);
    else if (kind == FK_MATRIX)
        rt_step<OP, REV, FK_MATRIX>(walk0, so);
    else
        rt_step<OP, REV, FK_SCALAR>(walk0, so); // SCALAR, or COLVEC: this row's value
}
template <int OP> __device__ __forceinline__ void rt_step_rev(bool rev, int kind, unsigned walk0, const RtOperand &so) {
    if (rev)
        rt_step_kind<OP, true>(kind, walk0, so);
    else
        rt_step_kind<OP, false>(kind, walk0, so);
}

__device__ __forceinline__ void rt_dispatch(int op, bool rev, int kind, unsigned walk0, const RtOperand &so) {
    switch (op) {
    // the order of the operands does not matter
    case FO_ADD: rt_step_kind<FO_ADD, false>(kind, walk0, so); break;
    case FO_MUL: rt_step_kind<FO_MUL, false>(kind, walk0, so); break;
    case FO_EQ: rt_step_kind<FO_EQ, false>(kind, walk0, so); break;
    case FO_NEQ: rt_step_kind<FO_NEQ, false>(kind, walk0, so); break;
    case FO_AND: rt_step_kind<FO_AND, false>(kind, walk0, so); break;
    case FO_OR: rt_step_kind<FO_OR, false>(kind, walk0, so); break;
    // it does (for MIN and MAX: which operand a NaN or a signed zero comes from)
    case FO_SUB: rt_step_rev<FO_SUB>(rev, kind, walk0, so); break;
    case FO_DIV: rt_step_rev<FO_DIV>(rev, kind, walk0, so); break;
    case FO_LT: rt_step_rev<FO_LT>(rev, kind, walk0, so); break;
    case FO_LE: rt_step_rev<FO_LE>(rev, kind, walk0, so); break;
    case FO_GT: rt_step_rev<FO_GT>(rev, kind, walk0, so); break;
    case FO_GE: rt_step_rev<FO_GE>(rev, kind, walk0, so); break;
    case FO_MIN: rt_step_rev<FO_MIN>(rev, kind, walk0, so); break;
    case FO_MAX: rt_step_rev<FO_MAX>(rev, kind, walk0, so); break;
    // no operand
    case FO_SQUARE: rt_step<FO_SQUARE, false, FK_UNARY>(walk0, so); break;
    case FO_NEG: rt_step<FO_NEG, false, FK_UNARY>(walk0, so); break;
    case FO_ABS: rt_step<FO_ABS, false, FK_UNARY>(walk0, so); break;
    case FO_SIGN: rt_step<FO_SIGN, false, FK_UNARY>(walk0, so); break;
    case FO_FLOOR: rt_step<FO_FLOOR, false, FK_UNARY>(walk0, so); break;
    case FO_CEIL: rt_step<FO_CEIL, false, FK_UNARY>(walk0, so); break;
    case FO_ROUND: rt_step<FO_ROUND, false, FK_UNARY>(walk0, so); break;
    case FO_ISNAN: rt_step<FO_ISNAN, false, FK_UNARY>(walk0, so); break;
    default: break;
    }
}

// the taps that see the row as it stands now (bit a of mask = tap a), fed in element order; FULL: all CK columns exist
template <bool FULL>
__device__ __forceinline__ void rt_feed_chunk(unsigned walk0, TapState<AnyTaps> &ts, const FusedProgram &P,
                                              unsigned mask, int cc, int cw) {
    double v[CK];
#pragma unroll
    for (int j = 0; j < CK / 2; j++) {
        const double2 xy = lds128(walk0 ^ (unsigned)(j << 4));
        v[2 * j] = xy.x;
        v[2 * j + 1] = xy.y;
    }
#pragma unroll
    for (int a = 0; a < FUSED_MAX_AGGS; a++) {
        if (mask & (1u << a)) {
            const int kind = P.taps[a].kind;
            if (kind == FT_SUM || kind == FT_MEAN) {
                double acc = ts.v[a];
#pragma unroll
                for (int i = 0; i < CK; i++)
                    if (FULL || i < cw)
                        acc = __dadd_rn(acc, v[i]);
                ts.v[a] = acc;
            } else if (kind == FT_PROD) {
                double acc = ts.v[a];
#pragma unroll
                for (int i = 0; i < CK; i++)
                    if (FULL || i < cw)
                        acc = __dmul_rn(acc, v[i]);
                ts.v[a] = acc;
            } else {
                if (cc == 0)
                    ts.first[a] = v[0];
                double best = ts.v[a];
                int bc = ts.c[a];
                if (kind == FT_MAX) {
#pragma unroll
                    for (int i = 0; i < CK; i++) {
                        const bool better = (FULL || i < cw) && (v[i] > best);
                        best = better ? v[i] : best;
                        bc = better ? cc + i : bc;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < CK; i++) {
                        const bool better = (FULL || i < cw) && (v[i] < best);
                        best = better ? v[i] : best;
                        bc = better ? cc + i : bc;
                    }
                }
                ts.v[a] = best;
                ts.c[a] = bc;
            }
        }
    }
}
__device__ __forceinline__ void rt_feed(unsigned walk0, TapState<AnyTaps> &ts, const FusedProgram &P, unsigned mask,
                                        int cc, int cw) {
    if (mask == 0)
        return;
    if (cw == CK)
        rt_feed_chunk<true>(walk0, ts, P, mask, cc, cw);
    else
        rt_feed_chunk<false>(walk0, ts, P, mask, cc, cw);
}

__device__ __forceinline__ void walk_row_rt(unsigned walk0, const FusedProgram &P, TapState<AnyTaps> &ts,
                                            const double *rvs, int64_t row, int64_t cc, int cw) {
    static_assert(CK % GR == 0, "a chunk is a whole number of groups");
    const unsigned *masks = reinterpret_cast<const unsigned *>(rvs + P.smem_elems + FUSED_MAX_STEPS);
    rt_feed(walk0, ts, P, masks[0], (int)cc, cw);
#pragma unroll 1
    for (int s = 0; s < P.nsteps; s++) {
        const FusedStep &fs = P.steps[s];
        const int kind = fs.kind;
        RtOperand so;
        so.vec = kind == FK_ROWVEC ? (unsigned)__cvta_generic_to_shared(rvs + fs.smem_off + cc) : 0u;
        so.mat = kind == FK_MATRIX ? static_cast<const double *>(fs.ptr) + row * fs.ld + cc : nullptr;
        so.scal = fs.imm;
        so.yscal = rvs[P.smem_elems + s]; // helper of a SCALAR divisor (staged once per CTA)
        if (kind == FK_COLVEC) {
            so.scal = __ldg(static_cast<const double *>(fs.ptr) + row * fs.ld);
            so.yscal = (fs.op == FO_DIV && !fs.reversed) ? div_helper(so.scal) : 0.0;
        }
        so.cols = (P.cols + 1) & ~(int64_t)1; // where the helpers of a staged divisor start
        so.cw = cw;
        rt_dispatch(fs.op, fs.reversed != 0, kind, walk0, so);
        rt_feed(walk0, ts, P, masks[s + 1], (int)cc, cw);
    }
}

// resident CTAs per SM: a run-time chain holds a whole chunk row in registers and gets the larger register budget
template <typename ChainT> struct RowCtasPerSm {
    static constexpr int value = 3;
};

// AL: rows of the base (and of the stored result) start on 16-byte boundaries and have an even number of columns
template <typename ChainT, typename TapsT, bool EW, bool AL = true>
__global__ void __launch_bounds__(RT, RowCtasPerSm<ChainT>::value) fused_row_ct_kernel(const __grid_constant__ FusedProgram P) {
    extern __shared__ __align__(16) double smem_raw[];
    // the chunk buffers start on a 256-byte boundary (the launch reserves the slack)
    const unsigned raw_s = (unsigned)__cvta_generic_to_shared(smem_raw);
    const unsigned pad = ((raw_s + 255u) & ~255u) - raw_s;
    double *smem = smem_raw + pad / 8;
    double *rvs = smem + WARPS * 2 * WR * CK; // staged row-vector operands (+ reciprocal helpers)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned bufs_s = raw_s + pad + (unsigned)(warp * 2 * WR * CK * 8); // this warp's two chunk buffers
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
                    rvs[st.smem_off + ((cols + 1) & ~(int64_t)1) + c] = div_helper(d);
            }
        }
    }
    if constexpr (same<ChainT, AnyChain>::value) {
        if (tid < P.nsteps) // NaN: no helper, the generic division
            rvs[P.smem_elems + tid] = P.steps[tid].kind == FK_SCALAR ? div_helper(P.steps[tid].imm)
                                                                      : __longlong_as_double(0x7ff8000000000000ll);
        if (tid <= P.nsteps) { // which taps follow `tid` steps
            unsigned mask = 0;
            for (int a = 0; a < P.ntaps; a++)
                if (P.taps[a].after_step == tid)
                    mask |= 1u << a;
            reinterpret_cast<unsigned *>(rvs + P.smem_elems + FUSED_MAX_STEPS)[tid] = mask;
        }
    }
    ChainState<ChainT> cs;
    init_scalar_aux<ChainT>(cs, P);
    __syncthreads(); // the only block-wide barrier: from here on every warp runs on its own

    const double *base = static_cast<const double *>(P.base);
    const int64_t ntiles = (rows + WR - 1) / WR;
    const int nchunks = (int)((cols + CK - 1) / CK);
    const int64_t wstride = (int64_t)gridDim.x * WARPS;
    constexpr unsigned BUF_BYTES = WR * CK * 8;
    const unsigned coop_off = (unsigned)((lane >> 4) * 256 + (((lane & 15) ^ (lane >> 4)) << 4));
    const unsigned walk_off = (unsigned)(lane * 256 + ((lane & 15) << 4));
    int64_t t = (int64_t)blockIdx.x * WARPS + warp;
    int ch = 0;
    unsigned b = 0;
    if (t < ntiles) {
        const int64_t row0 = t * WR;
        const int rh = (rows - row0 < WR) ? (int)(rows - row0) : WR, cw = (cols < CK) ? (int)cols : CK;
        if constexpr (AL) {
            if (rh == WR && cw == CK)
                issue_chunk<true>(bufs_s + coop_off, base + row0 * P.base_ld, P.base_ld, rh, cw, lane);
            else
                issue_chunk<false>(bufs_s + coop_off, base + row0 * P.base_ld, P.base_ld, rh, cw, lane);
        } else {
            if (rh == WR && cw == CK)
                issue_chunk_by_element<true>(bufs_s, base + row0 * P.base_ld, P.base_ld, rh, cw, lane);
            else
                issue_chunk_by_element<false>(bufs_s, base + row0 * P.base_ld, P.base_ld, rh, cw, lane);
        }
    }
    cp_async_commit();
    TapState<TapsT> ts;
    while (t < ntiles) {
        // the next chunk of this warp is on its way while this one is evaluated
        int64_t tn = t;
        int chn = ch + 1;
        if (chn == nchunks) {
            chn = 0;
            tn = t + wstride;
        }
        if (tn < ntiles) {
            const int64_t row0n = tn * WR, ccn = (int64_t)chn * CK;
            const int rh = (rows - row0n < WR) ? (int)(rows - row0n) : WR, cw = (cols - ccn < CK) ? (int)(cols - ccn) : CK;
            const double *src = base + row0n * P.base_ld + ccn;
            if constexpr (AL) {
                if (rh == WR && cw == CK)
                    issue_chunk<true>(bufs_s + (b ^ BUF_BYTES) + coop_off, src, P.base_ld, rh, cw, lane);
                else
                    issue_chunk<false>(bufs_s + (b ^ BUF_BYTES) + coop_off, src, P.base_ld, rh, cw, lane);
            } else {
                if (rh == WR && cw == CK)
                    issue_chunk_by_element<true>(bufs_s + (b ^ BUF_BYTES), src, P.base_ld, rh, cw, lane);
                else
                    issue_chunk_by_element<false>(bufs_s + (b ^ BUF_BYTES), src, P.base_ld, rh, cw, lane);
            }
        }
        cp_async_commit();
        cp_async_wait_but_one();
        __syncwarp();

        const unsigned tile_s = bufs_s + b;
        const int64_t row0 = t * WR, row = row0 + lane, cc = (int64_t)ch * CK;
        const int rows_here = (rows - row0 < WR) ? (int)(rows - row0) : WR;
        const int cw = (cols - cc < CK) ? (int)(cols - cc) : CK;
        const bool live = lane < rows_here;
        if (ch == 0) {
            if constexpr (same<TapsT, AnyTaps>::value)
                init_taps_rt(ts, P);
            else
                init_taps<TapsT>(ts);
            if (live)
                load_colvec_aux<ChainT>(cs, P, row);
        }
        if constexpr (same<ChainT, AnyChain>::value) {
            if (live) // in place: the elementwise result, if wanted, is the tile itself
                walk_row_rt(tile_s + walk_off, P, ts, rvs, row, cc, cw);
        } else {
            if (rows_here == WR && cw == CK)
                walk_row<ChainT, TapsT, EW, true>(tile_s + walk_off, P, cs, ts, rvs, row, cc, cw);
            else if (live)
                walk_row<ChainT, TapsT, EW, false>(tile_s + walk_off, P, cs, ts, rvs, row, cc, cw);
        }
        if constexpr (EW && !AL) { // one 8-byte store per element, lane = column
            __syncwarp();
            double *out = static_cast<double *>(P.ew_out) + row0 * P.ew_out_ld + cc + lane;
            if (lane < cw) {
#pragma unroll 4
                for (int r = 0; r < WR; r++)
                    if (r < rows_here) {
                        double q;
                        asm volatile("ld.shared.f64 %0, [%1];\n" : "=d"(q) : "r"(elem_addr(tile_s, r, lane)) : "memory");
                        __stcs(out + (int64_t)r * P.ew_out_ld, q);
                    }
            }
        } else if constexpr (EW) {
            __syncwarp();
            const int r0 = lane >> 4, p = lane & 15;
            double *out = static_cast<double *>(P.ew_out) + (row0 + r0) * P.ew_out_ld + cc + 2 * p;
            const bool full = rows_here == WR && cw == CK;
#pragma unroll
            for (int i = 0; i < CK / 2; i++) {
                if (full || (r0 + 2 * i < rows_here && 2 * p < cw)) {
                    const double2 q = lds128(coop_addr(tile_s + coop_off, i));
                    __stcs(reinterpret_cast<double2 *>(out + (int64_t)(2 * i) * P.ew_out_ld), q);
                }
            }
        }
        if (ch == nchunks - 1 && live) {
            if constexpr (same<TapsT, AnyTaps>::value)
                write_taps_rt(ts, P, row);
            else
                write_taps<TapsT>(ts, P, row);
        }
        __syncwarp(); // every lane is done with this buffer before the next iteration refills it
        t = tn;
        ch = chn;
        b ^= BUF_BYTES;
    }
}

// ---------------------------------------------------------------------------
// column pass with a compile-time chain (SUM only: the squared-deviation and plain column sums)
// ---------------------------------------------------------------------------
constexpr int CT_THREADS = 256;
// streaming load of two neighbouring values: read once, not kept in L1
__device__ __forceinline__ double2 ld_pair_stream(const double *p) { return __ldcs(reinterpret_cast<const double2 *>(p)); }

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
        if constexpr (St::op == FO_DIV && !St::rev && St::kind != FK_ROWVEC && St::kind != FK_SCALAR)
            v = __ddiv_rn(v, o); // no reciprocal helper exists for a column-vector or matrix divisor
        else
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
            double2 p[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                p[u] = ld_pair_stream(base + (r + u * stride) * P.base_ld + c0);
            double v0[4], v1[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                v0[u] = col_chain<ChainT>(p[u].x, 0, rv, ry, P, r + u * stride, c0);
                v1[u] = col_chain<ChainT>(p[u].y, 1, rv, ry, P, r + u * stride, c0 + 1);
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
            const double2 p = ld_pair_stream(base + r * P.base_ld + c0);
            const double2 q = ld_pair_stream(base + (r + stride) * P.base_ld + c0);
            a0 = __dadd_rn(a0, col_chain<ChainT>(p.x, 0, rv, ry, P, r, c0));
            a1 = __dadd_rn(a1, col_chain<ChainT>(p.y, 1, rv, ry, P, r, c0 + 1));
            b0 = __dadd_rn(b0, col_chain<ChainT>(q.x, 0, rv, ry, P, r + stride, c0));
            b1 = __dadd_rn(b1, col_chain<ChainT>(q.y, 1, rv, ry, P, r + stride, c0 + 1));
        }
        for (; r < rows; r += stride) {
            const double2 p = ld_pair_stream(base + r * P.base_ld + c0);
            a0 = __dadd_rn(a0, col_chain<ChainT>(p.x, 0, rv, ry, P, r, c0));
            a1 = __dadd_rn(a1, col_chain<ChainT>(p.y, 1, rv, ry, P, r, c0 + 1));
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

} // namespace ct
} // namespace db2
