// Tall-skinny FP64 product  D = A @ op(B)  with a fused row epilogue:  A is n x K (n large, K <= 128, row-major),
// op(B) is K x N with N <= 64.  This is the distance step of k-means,  X @ t(C)  (MatMul.cpp:284-288 in the reference:
// one dgemm writing the n x k matrix), followed there by three elementwise kernels and a row idxMin.
//
// One persistent CTA of 16 warps per SM keeps op(B) in shared memory for the whole launch.  Every WARP owns a private
// 16-row tile buffer and walks its own sequence of tiles -- copy (16-byte cp.async, zero fill), DMMAs
// (mma.sync m8n8k4 f64), epilogue -- without block-wide barriers, so the warps of an SM drift apart and the FP64 pipe
// (which the DMMAs and the epilogue's scalar FP64 arithmetic share) always finds a warp with DMMAs to issue.  A warp's
// 16 rows x all N columns sit in its accumulators with a row's values in the four lanes of a quad: the recorded
// elementwise chain (scalar, column-vector and row-vector operands) is applied in registers, the row minimum / maximum
// and its position are reduced with two shuffles, and the n x N product itself is only written if somebody asked for it.
#include "fused.cuh"
#include "runtime.h"

namespace db2 {

constexpr int SK_WARPS = 16, SK_WROWS = 16, SK_THREADS = SK_WARPS * 32, SK_MAXN = 64, SK_MAXK = 128;
constexpr int SK_VEC_SLOTS = 4; // row-vector and column-vector operands of a fused chain (each kind)

// one hardware DMMA: an 8 x 8 tile of C += A (8 x 4) * B (4 x 8); lane (g, t) holds A[g][t], B[t][g], C[g][2t..2t+1]
__device__ __forceinline__ void sk_dmma(double &c0, double &c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}
__device__ __forceinline__ double2 sk_lds128(unsigned a) {
    double2 v;
    asm volatile("ld.shared.v2.f64 {%0, %1}, [%2];\n" : "=d"(v.x), "=d"(v.y) : "r"(a) : "memory");
    return v;
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

// KPT: the contraction length rounded up to 16 as a compile-time constant (0: taken from the arguments).
// CH:  the fused chain as a compile-time constant: 1 = (* scalar, + column vector, + row vector), 2 = (* scalar, + row
//      vector) -- the distance step of k-means with and without the rowSums(X^2) term; 0 = interpreted.
//
// The FP64 pipe issues one DMMA per 16 cycles and scheduler, and every other instruction of the four warps that share
// a scheduler costs an issue slot in between, so the kernel is written to keep everything that is not a DMMA short:
//  * within each block of 16 k the four lanes of a quad take k = 4 t + j (j = 0..3) instead of t + 4 j -- A and B
//    agree, so the product is the same sum in a different (fixed) order -- which makes a lane's four k values
//    contiguous: two 128-bit shared loads per fragment instead of four 64-bit ones.  Row pitch = 2 mod 4 doubles: the
//    eight lanes of a load phase then hit eight different 16-byte columns.
//  * the tile copy has a fast path for full tiles (no bounds tests, one pointer increment per copy);
//  * the k-means chains are compiled in; the extremum tournament carries slot numbers (immediates), tests validity
//    only where padding columns can be, and looks for NaNs once per row instead of once per value.
template <int NT, int KPT, int CH>
__global__ void __launch_bounds__(SK_THREADS, 1) skinny_gemm_kernel(const __grid_constant__ SkinnyArgs s) {
    extern __shared__ __align__(16) double sm[];
    const int KP = KPT ? KPT : (s.K + 15) / 16 * 16, PA = KP + 2, PB = KP + 2;
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32, g = lane / 4, t = lane % 4;
    double *Bs = sm;                          // [NT*8][PB]: op(B) transposed, k contiguous
    double *rv = Bs + NT * 8 * PB;            // row-vector operands: [slot][64]
    double *At = rv + SK_VEC_SLOTS * SK_MAXN + (size_t)warp * (SK_WROWS * PA + SK_VEC_SLOTS * SK_WROWS);
    double *cv = At + SK_WROWS * PA;          // this warp's column-vector operands: [slot][16]
    const FusedProgram &P = s.prog;

    // op(B) transposed, zero padded to NT*8 columns and KP values of k
    for (int e = tid; e < NT * 8 * KP; e += SK_THREADS) {
        int n, k;
        if (s.tb) {
            n = e / KP;
            k = e % KP;
        } else {
            k = e / (NT * 8);
            n = e % (NT * 8);
        }
        double b = 0.0;
        if (n < s.N && k < s.K)
            b = s.tb ? s.B[(int64_t)n * s.ldb + k] : s.B[(int64_t)k * s.ldb + n];
        Bs[n * PB + k] = b;
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
    bool scale_pow2 = false;    // the compiled chains' scalar factor is +-2^e (normal): multiplying by it is exact
    if constexpr (CH != 0) {
        const unsigned hi = (unsigned)__double2hiint(P.steps[0].imm), ex = (hi >> 20) & 0x7ffu;
        scale_pow2 = __double2loint(P.steps[0].imm) == 0 && (hi & 0xfffffu) == 0 && ex != 0 && ex != 0x7ffu;
    }
    const unsigned At_s = (unsigned)__cvta_generic_to_shared(At);
    const unsigned afrag_s = At_s + (unsigned)((g * PA + 4 * t) * 8);
    const unsigned bfrag_s = (unsigned)__cvta_generic_to_shared(Bs) + (unsigned)((g * PB + 4 * t) * 8);
    for (int64_t tile = (int64_t)blockIdx.x * SK_WARPS + warp; tile < ntiles; tile += (int64_t)gridDim.x * SK_WARPS) {
        const int64_t r0 = tile * SK_WROWS;
        if (KPT != 0 && s.K == KPT && r0 + SK_WROWS <= s.n) {
            // full tile: lane -> packet p of rows r, r + 32 / packets, ...
            constexpr int PK = KPT ? KPT / 2 : 1, RSTEP = 32 / PK, NCP = SK_WROWS * PK / 32;
            const int r = lane / PK, p = lane % PK;
            const double *src = s.A + (r0 + r) * s.lda + 2 * p;
            const unsigned d = At_s + (unsigned)((r * PA + 2 * p) * 8);
#pragma unroll
            for (int i = 0; i < NCP; i++)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d + (unsigned)(i * RSTEP * PA * 8)),
                             "l"(src + (int64_t)(i * RSTEP) * s.lda)
                             : "memory");
        } else {
            const int dr = 32 / packets, dp = 32 % packets;
            int r = lane / packets, p = lane % packets;
            for (int e = lane; e < SK_WROWS * packets; e += 32) {
                const int64_t row = r0 + r;
                const int k = 2 * p;
                int bytes = 0;
                if (row < s.n && k < s.K)
                    bytes = (s.K - k >= 2) ? 16 : 8;
                const unsigned d = At_s + (unsigned)((r * PA + k) * 8);
                const double *src = bytes ? s.A + row * s.lda + k : s.A;
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
                r += dr;
                p += dp;
                if (p >= packets) {
                    p -= packets;
                    r++;
                }
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

        double acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                acc[nt][e] = 0.0;
        auto kblock = [&](int ks) { // 16 values of k: 8 DMMAs per 8-column block
            const unsigned ka = (unsigned)(ks * 8);
            const double2 a0l = sk_lds128(afrag_s + ka), a0h = sk_lds128(afrag_s + ka + 16);
            const double2 a1l = sk_lds128(afrag_s + ka + (unsigned)(8 * PA * 8));
            const double2 a1h = sk_lds128(afrag_s + ka + (unsigned)(8 * PA * 8) + 16);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                const double2 bl = sk_lds128(bfrag_s + ka + (unsigned)(nt * 8 * PB * 8));
                const double2 bh = sk_lds128(bfrag_s + ka + (unsigned)(nt * 8 * PB * 8) + 16);
                sk_dmma(acc[nt][0], acc[nt][1], a0l.x, bl.x);
                sk_dmma(acc[nt][2], acc[nt][3], a1l.x, bl.x);
                sk_dmma(acc[nt][0], acc[nt][1], a0l.y, bl.y);
                sk_dmma(acc[nt][2], acc[nt][3], a1l.y, bl.y);
                sk_dmma(acc[nt][0], acc[nt][1], a0h.x, bh.x);
                sk_dmma(acc[nt][2], acc[nt][3], a1h.x, bh.x);
                sk_dmma(acc[nt][0], acc[nt][1], a0h.y, bh.y);
                sk_dmma(acc[nt][2], acc[nt][3], a1h.y, bh.y);
            }
        };
        if constexpr (KPT != 0) {
#pragma unroll
            for (int ks = 0; ks < KPT; ks += 16)
                kblock(ks);
        } else {
            for (int ks = 0; ks < KP; ks += 16)
                kblock(ks);
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
            if constexpr (CH != 0) {
                double rvv[NV]; // the row-vector operand, as this lane's columns
                const double *src = rv + P.steps[CH == 1 ? 2 : 1].smem_off * SK_MAXN + 2 * t;
#pragma unroll
                for (int nt = 0; nt < NT; nt++) {
                    const double2 two = *reinterpret_cast<const double2 *>(src + nt * 8);
                    rvv[2 * nt] = two.x;
                    rvv[2 * nt + 1] = two.y;
                }
                const double m = P.steps[0].imm;
                double colv = 0.0;
                if constexpr (CH == 1)
                    colv = cv[P.steps[1].smem_off * SK_WROWS + g + 8 * h];
                if (scale_pow2) {
                    // v * m is exact, so the multiplication and the first addition are one FMA with the same bits
                    // (scalar FP64 instructions take the pipe the DMMAs of the other warps are waiting for)
#pragma unroll
                    for (int i = 0; i < NV; i++) {
                        if constexpr (CH == 1)
                            v[i] = __dadd_rn(__fma_rn(v[i], m, colv), rvv[i]);
                        else
                            v[i] = __fma_rn(v[i], m, rvv[i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < NV; i++) {
                        v[i] = __dmul_rn(v[i], m);
                        if constexpr (CH == 1)
                            v[i] = __dadd_rn(v[i], colv);
                        v[i] = __dadd_rn(v[i], rvv[i]);
                    }
                }
            } else {
#pragma unroll 1
                for (int st = 0; st < P.nsteps; st++) {
                    const FusedStep &fs = P.steps[st];
                    double o[NV];
                    if (fs.kind == FK_ROWVEC) {
#pragma unroll
                        for (int nt = 0; nt < NT; nt++) {
                            const double2 two =
                                *reinterpret_cast<const double2 *>(rv + fs.smem_off * SK_MAXN + nt * 8 + 2 * t);
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
                // column 0 anyway; a NaN in column 0 is put back at the end.  Block tournament (depth 4): slot i of a
                // round stands for the slots [i, i + w); every column of the left block is lower than every column
                // of the right block, so keeping the left candidate on ties keeps the first extremum.  Only the two
                // cross-lane rounds need a column tie-break.
                const bool want_max = P.taps[tp].kind == FT_MAX;
                double x[16];
                int c[16]; // slot numbers (immediates); turned into a column once, for the winner
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    x[i] = i < NV ? v[i < NV ? i : 0] : (double)INFINITY;
                    c[i] = i;
                }
                if (want_max) {
#pragma unroll
                    for (int i = 0; i < NV; i++)
                        x[i] = -x[i];
                }
                {
                    // NaNs are looked for with integer instructions (any exponent of all ones: NaN or infinity)
                    unsigned spare = 0x7ff00000u; // the smallest  ~exponent  seen: 0 = some exponent is all ones
#pragma unroll
                    for (int i = 0; i < NV; i++)
                        spare = min(spare, ~(unsigned)__double2hiint(x[i]) & 0x7ff00000u);
                    if (spare == 0) {
#pragma unroll
                        for (int i = 0; i < NV; i++)
                            x[i] = fmin(x[i], (double)INFINITY);
                    }
                }
#pragma unroll
                for (int i = NV - 2; i < NV; i++) // padding columns exist only in the last 8-column block
                    if ((i >> 1) * 8 + 2 * t + (i & 1) >= s.N)
                        x[i] = (double)INFINITY;
#pragma unroll
                for (int w = 1; w <= 8; w <<= 1)
#pragma unroll
                    for (int i = 0; i < 16; i += 2 * w) {
                        const bool right = x[i + w] < x[i];
                        x[i] = right ? x[i + w] : x[i];
                        c[i] = right ? c[i + w] : c[i];
                    }
                double best = x[0];
                int bi = (c[0] >> 1) * 8 + 2 * t + (c[0] & 1);
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
                    if (best == (double)INFINITY || v0 != v0) { // the scan never left column 0
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

static size_t skinny_smem(int K, int nt) {
    const int KP = (K + 15) / 16 * 16, PA = KP + 2, PB = KP + 2;
    return ((size_t)nt * 8 * PB + SK_VEC_SLOTS * SK_MAXN +
            (size_t)SK_WARPS * (SK_WROWS * PA + SK_VEC_SLOTS * SK_WROWS)) * sizeof(double);
}

bool skinny_shape_ok(int64_t n, int64_t K, int64_t N, const void *A, int64_t lda) {
    return n >= 4096 && K >= 1 && K <= SK_MAXK && N >= 1 && N <= SK_MAXN && aligned16(A) && lda % 2 == 0 &&
           skinny_smem((int)K, (int)((N + 7) / 8)) <= 220 * 1024;
}

template <int NT, int KPT, int CH> static int launch_skinny_k(const SkinnyArgs &a, cudaStream_t st) {
    const size_t smem = skinny_smem(a.K, NT);
    static PerDeviceOnce attr;
    if (attr.need()) {
        DB2_CUDA(cudaFuncSetAttribute(skinny_gemm_kernel<NT, KPT, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      220 * 1024));
        attr.mark();
    }
    const int64_t ctas = ((a.n + SK_WROWS - 1) / SK_WROWS + SK_WARPS - 1) / SK_WARPS;
    const int grid = (int)(ctas < sm_count() ? ctas : sm_count());
    skinny_gemm_kernel<NT, KPT, CH><<<grid, SK_THREADS, smem, st>>>(a);
    return after_launch("skinny_gemm_kernel");
}
template <int NT, int CH> static int launch_skinny(const SkinnyArgs &a, cudaStream_t st) {
    switch ((a.K + 15) / 16 * 16) { // the common contraction lengths get their own instantiation
    case 16: return launch_skinny_k<NT, 16, CH>(a, st);
    case 32: return launch_skinny_k<NT, 32, CH>(a, st);
    case 64: return launch_skinny_k<NT, 64, CH>(a, st);
    default: return launch_skinny_k<NT, 0, CH>(a, st);
    }
}

int skinny_vec_slots() { return SK_VEC_SLOTS; }

// the chains that are compiled in (the CH parameter of the kernel); anything else is interpreted
static int compiled_chain(const FusedProgram &P) {
    auto is = [&](int i, int op, int kind) { return P.steps[i].op == op && P.steps[i].kind == kind; };
    if (P.nsteps == 3 && is(0, FO_MUL, FK_SCALAR) && is(1, FO_ADD, FK_COLVEC) && is(2, FO_ADD, FK_ROWVEC))
        return 1;
    if (P.nsteps == 2 && is(0, FO_MUL, FK_SCALAR) && is(1, FO_ADD, FK_ROWVEC))
        return 2;
    return 0;
}

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
    const int nt = (a.N + 7) / 8, ch = compiled_chain(a.prog);
#define DB2_SK(NTV)                                                                                                    \
    case NTV:                                                                                                          \
        return ch == 1 ? launch_skinny<NTV, 1>(a, st) : (ch == 2 ? launch_skinny<NTV, 2>(a, st) : launch_skinny<NTV, 0>(a, st));
    switch (nt) {
        DB2_SK(1) DB2_SK(2) DB2_SK(3) DB2_SK(4) DB2_SK(5) DB2_SK(6) DB2_SK(7) DB2_SK(8)
    default: return set_error(DB2_EINVAL, "skinny product: more than 64 columns");
    }
#undef DB2_SK
}

} // namespace db2
