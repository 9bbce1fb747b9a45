// Tall-skinny FP64 product  D = A @ op(B)  with a fused row epilogue:  A is n x K (n large, K <= 128, row-major),
// op(B) is K x N with N <= 64.  This is the distance step of k-means,  X @ t(C)  (MatMul.cpp:284-288 in the reference:
// one dgemm writing the n x k matrix), followed there by three elementwise kernels and a row idxMin.
//
// One persistent CTA of 16 warps per SM keeps op(B) in shared memory for the whole launch.  Every WARP owns a private
// 16-row tile buffer and walks its own sequence of tiles -- copy (16-byte cp.async, zero fill), DMMAs
// (mma.sync m16n8k16 f64), epilogue -- without block-wide barriers, so the warps of an SM drift apart and the FP64 pipe
// (which the DMMAs and the epilogue's scalar FP64 arithmetic share) always finds a warp with DMMAs to issue.  A warp's
// 16 rows x all N columns sit in its accumulators with a row's values in the four lanes of a quad: the recorded
// elementwise chain (scalar, column-vector and row-vector operands) is applied in registers, the row minimum / maximum
// and its position are reduced with two shuffles, and the n x N product itself is only written if somebody asked for it.
#include "fused.cuh"
#include "runtime.h"

namespace db2 {

constexpr int SK_WARPS = 16, SK_WROWS = 16, SK_THREADS = SK_WARPS * 32, SK_MAXN = 64, SK_MAXK = 128;
constexpr int SK_VEC_SLOTS = 4; // row-vector and column-vector operands of a fused chain (each kind)

__device__ __forceinline__ void sk_dmma(double (&c)[4], const double (&a)[8], const double (&b)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7,%8,%9,%10,%11}, "
                 "{%12,%13,%14,%15}, {%0,%1,%2,%3};\n"
                 : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
                 : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(a[4]), "d"(a[5]), "d"(a[6]), "d"(a[7]), "d"(b[0]),
                   "d"(b[1]), "d"(b[2]), "d"(b[3]));
}

// value (op) operand on NV values with the exactly rounded semantics of the elementwise kernels; the opcode is
// dispatched once per step, not per value (the epilogue must stay small: it runs once per 128-row tile)
template <int NV>
__device__ __forceinline__ void sk_apply(int op, bool rev, double (&v)[NV], const double (&o)[NV]) {
#define DB2_SK_STEP(FWD, REV)                                                                                          \
    if (!rev) {                                                                                                        \
        _Pragma("unroll") for (int i = 0; i < NV; i++) { const double a = v[i], b = o[i]; (void)b; v[i] = (FWD); }     \
    } else {                                                                                                           \
        _Pragma("unroll") for (int i = 0; i < NV; i++) { const double a = v[i], b = o[i]; (void)b; v[i] = (REV); }     \
    }                                                                                                                  \
    break;
    switch (op) {
    case FO_ADD: DB2_SK_STEP(__dadd_rn(a, b), __dadd_rn(b, a))
    case FO_SUB: DB2_SK_STEP(__dsub_rn(a, b), __dsub_rn(b, a))
    case FO_MUL: DB2_SK_STEP(__dmul_rn(a, b), __dmul_rn(b, a))
    case FO_DIV: DB2_SK_STEP(__ddiv_rn(a, b), __ddiv_rn(b, a))
    case FO_SQUARE: DB2_SK_STEP(__dmul_rn(a, a), __dmul_rn(a, a))
    case FO_MIN: DB2_SK_STEP(((b < a) ? b : a), ((a < b) ? a : b))
    case FO_MAX: DB2_SK_STEP(((a < b) ? b : a), ((b < a) ? a : b))
    case FO_NEG: DB2_SK_STEP(-a, -a)
    case FO_ABS: DB2_SK_STEP(fabs(a), fabs(a))
    default: break;
    }
#undef DB2_SK_STEP
}
bool skinny_op_supported(int op) {
    return op == FO_ADD || op == FO_SUB || op == FO_MUL || op == FO_DIV || op == FO_SQUARE || op == FO_MIN ||
           op == FO_MAX || op == FO_NEG || op == FO_ABS;
}

// KPT: the contraction length rounded up to 16 as a compile-time constant (0: taken from the arguments).  With it every
// fragment address is one base register plus an immediate; the general form spends most of its instructions on
// address arithmetic.
template <int NT, bool TB, int KPT>
__global__ void __launch_bounds__(SK_THREADS, 1) skinny_gemm_kernel(const __grid_constant__ SkinnyArgs s) {
    extern __shared__ __align__(16) double sm[];
    const int KP = KPT ? KPT : (s.K + 15) / 16 * 16, PA = KP + 4; // pitch = 4 mod 16 doubles: conflict-free fragments
    const int PB = TB ? KP + 4 : NT * 8 + 4;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32, g = lane / 4, t = lane % 4;
    double *Bs = sm;                                 // TB: [NT*8][PB] (k contiguous);  else [KP][PB]
    double *rv = Bs + (TB ? NT * 8 * PB : KP * PB);   // row-vector operands: [slot][64]
    double *At = rv + SK_VEC_SLOTS * SK_MAXN + (size_t)warp * (SK_WROWS * PA + SK_VEC_SLOTS * SK_WROWS);
    double *cv = At + SK_WROWS * PA;                  // this warp's column-vector operands: [slot][16]
    const FusedProgram &P = s.prog;

    // op(B), zero padded to NT*8 columns and KP rows of k
    if (TB) {
        for (int e = tid; e < NT * 8 * KP; e += SK_THREADS) {
            const int n = e / KP, k = e % KP;
            Bs[n * PB + k] = (n < s.N && k < s.K) ? s.B[(int64_t)n * s.ldb + k] : 0.0;
        }
    } else {
        for (int e = tid; e < KP * NT * 8; e += SK_THREADS) {
            const int k = e / (NT * 8), n = e % (NT * 8);
            Bs[k * PB + n] = (n < s.N && k < s.K) ? s.B[(int64_t)k * s.ldb + n] : 0.0;
        }
    }
    for (int st = 0; st < P.nsteps; st++)
        if (P.steps[st].kind == FK_ROWVEC)
            for (int c = tid; c < SK_MAXN; c += SK_THREADS)
                rv[P.steps[st].smem_off * SK_MAXN + c] = c < s.N ? static_cast<const double *>(P.steps[st].ptr)[c] : 0.0;
    __syncthreads(); // the only block-wide barrier: from here on every warp runs on its own

    // Every warp walks its own sequence of 16-row tiles: copy (cp.async), DMMAs, epilogue.  The 16 warps of the SM
    // drift apart, so while one waits for its copy or works through its epilogue the others keep the FP64 pipe busy.
    const int64_t ntiles = (s.n + SK_WROWS - 1) / SK_WROWS;
    const int packets = KP / 2; // 16-byte packets per row
    const int dr = 32 / packets, dp = 32 % packets;
    for (int64_t tile = (int64_t)blockIdx.x * SK_WARPS + warp; tile < ntiles; tile += (int64_t)gridDim.x * SK_WARPS) {
        const int64_t r0 = tile * SK_WROWS;
        {
            int r = lane / packets, p = lane % packets;
            for (int e = lane; e < SK_WROWS * packets; e += 32) {
                const int64_t row = r0 + r;
                const int k = 2 * p;
                int bytes = 0;
                if (row < s.n && k < s.K)
                    bytes = (s.K - k >= 2) ? 16 : 8;
                const unsigned d = (unsigned)__cvta_generic_to_shared(At + r * PA + k);
                const double *src = bytes ? s.A + row * s.lda + k : s.A;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
                r += dr;
                p += dp;
                if (p >= packets) {
                    p -= packets;
                    r++;
                }
            }
            if (lane < SK_WROWS)
                for (int st = 0; st < P.nsteps; st++)
                    if (P.steps[st].kind == FK_COLVEC) {
                        const int64_t row = r0 + lane;
                        const double *base = static_cast<const double *>(P.steps[st].ptr);
                        const unsigned d = (unsigned)__cvta_generic_to_shared(cv + P.steps[st].smem_off * SK_WROWS + lane);
                        const int bytes = row < s.n ? 8 : 0;
                        const double *src = bytes ? base + row * P.steps[st].ld : base;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
                    }
            asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
            __syncwarp();
        }

        double acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                acc[nt][e] = 0.0;
        for (int ks = 0; ks < KP; ks += 16) {
            double af[8];
#pragma unroll
            for (int i = 0; i < 8; i++)
                af[i] = At[(g + 8 * (i & 1)) * PA + ks + t + 4 * (i >> 1)];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                double bf[4];
#pragma unroll
                for (int i = 0; i < 4; i++)
                    bf[i] = TB ? Bs[(nt * 8 + g) * PB + ks + t + 4 * i] : Bs[(ks + t + 4 * i) * PB + nt * 8 + g];
                sk_dmma(acc[nt], af, bf);
            }
        }

        // ---- epilogue: chain, outputs, row extremum, for the thread's two rows g and g + 8 ----
        constexpr int NV = NT * 2; // value 2 * nt + e is column 8 * nt + 2 * t + e
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int64_t r = r0 + g + 8 * h;
            double v[NV];
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                v[2 * nt] = acc[nt][2 * h];
                v[2 * nt + 1] = acc[nt][2 * h + 1];
            }
#pragma unroll 1
            for (int st = 0; st < P.nsteps; st++) {
                const FusedStep &fs = P.steps[st];
                double o[NV];
                if (fs.kind == FK_ROWVEC) {
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        const double2 two = *reinterpret_cast<const double2 *>(rv + fs.smem_off * SK_MAXN + nt * 8 + 2 * t);
                        o[2 * nt] = two.x;
                        o[2 * nt + 1] = two.y;
                    }
                } else {
                    const double colv = fs.kind == FK_COLVEC ? cv[fs.smem_off * SK_WROWS + g + 8 * h] : fs.imm;
#pragma unroll
                    for (int i = 0; i < NV; i++)
                        o[i] = colv;
                }
                sk_apply<NV>(fs.op, fs.reversed != 0, v, o);
            }
            if (P.ew_out && r < s.n) {
                double *out = static_cast<double *>(P.ew_out) + r * P.ew_out_ld;
#pragma unroll
                for (int i = 0; i < NV; i++) {
                    const int c = (i >> 1) * 8 + 2 * t + (i & 1);
                    if (c < s.N)
                        out[c] = v[i];
                }
            }
#pragma unroll 1
            for (int tp = 0; tp < P.ntaps; tp++) {
                // First extremum in column order; the maximum is the minimum of the negated values.  The reference's
                // scan (AggRow.h:71-96) starts from column 0 and uses strict comparisons: a NaN never replaces the
                // running extremum, and a NaN in column 0 stays.  Here NaNs and the padding columns take part as
                // +inf: they can only "win" a row whose every real value is +inf or NaN, and such a row's answer is
                // column 0 anyway.  Block tournament (depth 4): slot i of a round stands for the slots [i, i + w);
                // every column of the left block is lower than every column of the right block, so keeping the left
                // candidate on ties keeps the first extremum.  Only the two cross-lane rounds need a column tie-break.
                const bool want_max = P.taps[tp].kind == FT_MAX;
                double x[16];
                int c[16];
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int col = (i >> 1) * 8 + 2 * t + (i & 1);
                    const double val = i < NV ? v[i < NV ? i : 0] : 0.0;
                    x[i] = (i < NV && col < s.N) ? fmin(want_max ? -val : val, (double)INFINITY) : (double)INFINITY;
                    c[i] = col;
                }
#pragma unroll
                for (int w = 1; w <= 8; w <<= 1)
#pragma unroll
                    for (int i = 0; i < 16; i += 2 * w) {
                        const bool right = x[i + w] < x[i];
                        x[i] = right ? x[i + w] : x[i];
                        c[i] = right ? c[i + w] : c[i];
                    }
                double best = x[0];
                int bi = c[0];
#pragma unroll
                for (int m = 1; m <= 2; m <<= 1) {
                    const double ob = __shfl_xor_sync(0xffffffffu, best, m);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
                    const bool take = ob < best || (ob == best && oi < bi);
                    best = take ? ob : best;
                    bi = take ? oi : bi;
                }
                const double v0 = __shfl_sync(0xffffffffu, v[0], lane & ~3); // column 0 lives in lane t = 0
                if (r < s.n && t == 0) {
                    double val = want_max ? -best : best;
                    int pos = bi;
                    if (best == (double)INFINITY) { // nothing below +inf: the scan never left column 0
                        val = v0;
                        pos = 0;
                    }
                    if (P.taps[tp].out)
                        static_cast<double *>(P.taps[tp].out)[r] = val;
                    if (P.taps[tp].out_idx)
                        static_cast<uint64_t *>(P.taps[tp].out_idx)[r] = (uint64_t)pos;
                }
            }
        }
        __syncwarp(); // every lane is done with this tile's shared memory before the next copy overwrites it
    }
}

static size_t skinny_smem(int K, int nt, bool tb) {
    const int KP = (K + 15) / 16 * 16, PA = KP + 4, PB = tb ? KP + 4 : nt * 8 + 4;
    return ((size_t)(tb ? nt * 8 * PB : KP * PB) + SK_VEC_SLOTS * SK_MAXN +
            (size_t)SK_WARPS * (SK_WROWS * PA + SK_VEC_SLOTS * SK_WROWS)) * sizeof(double);
}

bool skinny_shape_ok(int64_t n, int64_t K, int64_t N, const void *A, int64_t lda) {
    return n >= 4096 && K >= 1 && K <= SK_MAXK && N >= 1 && N <= SK_MAXN && aligned16(A) && lda % 2 == 0 &&
           skinny_smem((int)K, (int)((N + 7) / 8), true) <= 220 * 1024 &&
           skinny_smem((int)K, (int)((N + 7) / 8), false) <= 220 * 1024;
}

template <int NT, bool TB, int KPT> static int launch_skinny_k(const SkinnyArgs &a, cudaStream_t st) {
    const size_t smem = skinny_smem(a.K, NT, TB);
    static bool attr = false;
    if (!attr) {
        DB2_CUDA(cudaFuncSetAttribute(skinny_gemm_kernel<NT, TB, KPT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      220 * 1024));
        attr = true;
    }
    const int64_t ctas = ((a.n + SK_WROWS - 1) / SK_WROWS + SK_WARPS - 1) / SK_WARPS;
    const int grid = (int)(ctas < sm_count() ? ctas : sm_count());
    skinny_gemm_kernel<NT, TB, KPT><<<grid, SK_THREADS, smem, st>>>(a);
    return after_launch("skinny_gemm_kernel");
}
template <int NT, bool TB> static int launch_skinny(const SkinnyArgs &a, cudaStream_t st) {
    switch ((a.K + 15) / 16 * 16) { // the common contraction lengths get their own instantiation
    case 16: return launch_skinny_k<NT, TB, 16>(a, st);
    case 32: return launch_skinny_k<NT, TB, 32>(a, st);
    case 64: return launch_skinny_k<NT, TB, 64>(a, st);
    default: return launch_skinny_k<NT, TB, 0>(a, st);
    }
}

int skinny_vec_slots() { return SK_VEC_SLOTS; }

int skinny_gemm(const SkinnyArgs &args, cudaStream_t st) {
    if (args.n == 0 || args.N == 0)
        return DB2_OK;
    SkinnyArgs a = args;
    int rows = 0, cols = 0; // shared-memory slot of every vector operand
    for (int i = 0; i < a.prog.nsteps; i++) {
        if (a.prog.steps[i].kind == FK_ROWVEC)
            a.prog.steps[i].smem_off = rows++;
        else if (a.prog.steps[i].kind == FK_COLVEC)
            a.prog.steps[i].smem_off = cols++;
    }
    DB2_CHECK(rows <= SK_VEC_SLOTS && cols <= SK_VEC_SLOTS, DB2_EINVAL, "skinny product: too many vector operands");
    const int nt = (a.N + 7) / 8;
#define DB2_SK(NTV)                                                                                                    \
    case NTV: return a.tb ? launch_skinny<NTV, true>(a, st) : launch_skinny<NTV, false>(a, st);
    switch (nt) {
        DB2_SK(1) DB2_SK(2) DB2_SK(3) DB2_SK(4) DB2_SK(5) DB2_SK(6) DB2_SK(7) DB2_SK(8)
    default: return set_error(DB2_EINVAL, "skinny product: more than 64 columns");
    }
#undef DB2_SK
}

} // namespace db2
