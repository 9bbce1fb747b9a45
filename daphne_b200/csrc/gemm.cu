// FP64 contractions on the tensor cores: MatMul (all four transpose combinations) and Syrk (t(X) X / X t(X)).
//
// Blackwell's tcgen05 tensor path has no FP64 kind, so the FP64 contraction is the warp-level DMMA
// (mma.sync.aligned.m16n8k16.f64), fed from shared memory tiles that are filled with 16-byte cp.async copies in a
// 3-stage ring.  Tile layouts are chosen so that every fragment load is a conflict-free 128-bit shared load: an
// operand whose contraction index is contiguous in memory is stored [row][KC + 2], the other kind is stored
// [k][tile + 4].  The FP64 pipe takes one DMMA per 16 cycles and scheduler, and every other instruction of the
// warps on that scheduler needs an issue slot in between, so the loop is kept short: two values per shared load,
// and a loader without bounds tests for the stages that lie inside the operands.
//
// The tall-skinny products of the workloads (t(X) X with 8.4 M x 512, t(P) X with 1 M x 50) contract over the ROWS:
// the row range is split over gridDim.z, each split accumulates a private tile and writes it to scratch, and a second
// kernel adds the splits in a fixed order (deterministic, no atomics).  Syrk computes only the tiles on and above the
// diagonal (36 of 64 tiles for d = 512) and mirrors them in the reduce step.
#include "common.cuh"

namespace db2 {

constexpr int KC = 32;     // contraction depth per stage (two m16n8k16 steps)
// pitch of a [row][k] tile (doubles).  When both operands are stored that way (A B^T) their fragments are read with
// 128-bit loads, which are conflict free at a pitch of 2 mod 4; next to a [k][row] operand the loads are 64 bits wide
// and want 4 mod 16.
__host__ __device__ constexpr int pitch_k(bool ta, bool tb) { return (!ta && tb) ? KC + 2 : KC + 4; }
// CTA tiles: BM x BN in {64,128}^2 with (BM / 32) x (BN / 32) warps of 32 x 32.  128 x 128 (16 warps) gives 16 flop
// per byte fetched from L2, which is what keeps the FP64 tensor pipe busy (a 64 x 64 tile needs twice the L2 traffic
// and stalls at about half of peak on this part).
template <int BM, int BN> struct TileCfg {
    static constexpr int WN = 32;
    static constexpr int THREADS = (BM / 32) * (BN / 32) * 32;
    static constexpr int STAGES = 3;
};

// D (16 x 8) += A (16 x 16, row) * B (16 x 8, col).  With g = lane / 4, t = lane % 4:
//   a[i]: row g + 8 * (i & 1), k = t + 4 * (i >> 1);   b[i]: k = t + 4 * i, column g;
//   c[i]: row g + 8 * (i >> 1), column 2 * t + (i & 1).
__device__ __forceinline__ void dmma16x8x16(double (&c)[4], const double (&a)[8], const double (&b)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f64.f64.f64.f64 {%0,%1,%2,%3}, {%4,%5,%6,%7,%8,%9,%10,%11}, "
                 "{%12,%13,%14,%15}, {%0,%1,%2,%3};\n"
                 : "+d"(c[0]), "+d"(c[1]), "+d"(c[2]), "+d"(c[3])
                 : "d"(a[0]), "d"(a[1]), "d"(a[2]), "d"(a[3]), "d"(a[4]), "d"(a[5]), "d"(a[6]), "d"(a[7]), "d"(b[0]),
                   "d"(b[1]), "d"(b[2]), "d"(b[3]));
}
// 16-byte async copy with zero fill: `bytes` (0, 8 or 16) are read from global, the rest of the slot is zeroed
__device__ __forceinline__ void cp_async16_zfill(void *smem_dst, const void *gsrc, int bytes) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

struct GemmArgs {
    const double *A, *B;
    double *C;      // result (splits == 1) ...
    double *part;   // ... or per-split partial tiles [split][tile_m][tile_n][BM][BN]
    int64_t lda, ldb, ldc;
    int64_t M, N, K;
    int splits;
    int64_t k_per_split; // multiple of KC
    // syrk: tiles on the diagonal run only the warps on or above it, so they get fewer, longer shares of the
    // contraction range than the full tiles (same time per CTA)
    int splits_diag;
    int64_t k_per_split_diag;
    int syrk;            // only tiles with tile_n*BN + BN > tile_m*BM are computed (upper triangle incl. diagonal)
    int aligned;         // operands allow 16-byte copies (bases 16-byte aligned, even leading dimensions)
    // t(X) y next to t(X) X (syrk with A = B = X stored K x M): the warps of a diagonal tile that have no sub-tile to
    // compute form the products of their tile's columns with y from the operand stages that pass through shared
    // memory anyway, so X is read once for both results.  yv: K contiguous doubles, 16-byte aligned;
    // ypart: [splits_diag][M] partial sums, added up in split order by gemv_fold_kernel.
    const double *yv;
    double *ypart;
};

// Loads one stage.  TA: A is stored K x M (contraction index = row);  !TA: A is M x K.  Same for TB with N.
// FULL: the stage lies inside the operands and 16-byte copies are allowed -- no bounds tests, no zero fill.
template <bool TA, bool TB, int BM, int BN, bool FULL>
__device__ __forceinline__ void load_stage(const GemmArgs &g, double *As, double *Bs, int64_t m0, int64_t n0,
                                           int64_t k0, int64_t k_end, int tid, int nthreads, bool load_b,
                                           const double *a_src, const double *b_src) {
    constexpr int PA = BM + 4, PB = BN + 4, PK = pitch_k(TA, TB);
    if constexpr (FULL) {
        // a_src / b_src: this thread's first 16 bytes of the stage (see full_src)
        constexpr int NT = (BM / 32) * (BN / 32) * 32;
        if constexpr (TA) {
            double *dst = As + (tid / (BM / 2)) * PA + 2 * (tid % (BM / 2));
#pragma unroll
            for (int i = 0; i < KC * (BM / 2) / NT; i++)
                cp_async16(dst + i * (NT / (BM / 2)) * PA, a_src + (int64_t)(i * (NT / (BM / 2))) * g.lda);
        } else {
            double *dst = As + (tid / (KC / 2)) * PK + 2 * (tid % (KC / 2));
#pragma unroll
            for (int i = 0; i < BM * (KC / 2) / NT; i++)
                cp_async16(dst + i * (NT / (KC / 2)) * PK, a_src + (int64_t)(i * (NT / (KC / 2))) * g.lda);
        }
        if (!load_b) {
        } else if constexpr (!TB) {
            double *dst = Bs + (tid / (BN / 2)) * PB + 2 * (tid % (BN / 2));
#pragma unroll
            for (int i = 0; i < KC * (BN / 2) / NT; i++)
                cp_async16(dst + i * (NT / (BN / 2)) * PB, b_src + (int64_t)(i * (NT / (BN / 2))) * g.ldb);
        } else {
            double *dst = Bs + (tid / (KC / 2)) * PK + 2 * (tid % (KC / 2));
#pragma unroll
            for (int i = 0; i < BN * (KC / 2) / NT; i++)
                cp_async16(dst + i * (NT / (KC / 2)) * PK, b_src + (int64_t)(i * (NT / (KC / 2))) * g.ldb);
        }
    } else if (g.aligned) {
        if constexpr (TA) { // [KC][BM]: KC rows of BM contiguous doubles
            for (int idx = tid; idx < KC * (BM / 2); idx += nthreads) {
                const int kk = idx / (BM / 2), p = idx % (BM / 2);
                const int64_t k = k0 + kk, m = m0 + 2 * p;
                int bytes = 0;
                if (k < k_end && m < g.M)
                    bytes = (g.M - m >= 2) ? 16 : 8;
                cp_async16_zfill(As + kk * PA + 2 * p, bytes ? (g.A + k * g.lda + m) : g.A, bytes);
            }
        } else { // [BM][KC]
            for (int idx = tid; idx < BM * (KC / 2); idx += nthreads) {
                const int r = idx / (KC / 2), p = idx % (KC / 2);
                const int64_t m = m0 + r, k = k0 + 2 * p;
                int bytes = 0;
                if (m < g.M && k < k_end)
                    bytes = (k_end - k >= 2) ? 16 : 8;
                cp_async16_zfill(As + r * PK + 2 * p, bytes ? (g.A + m * g.lda + k) : g.A, bytes);
            }
        }
        if (!load_b) {
        } else if constexpr (!TB) { // B is K x N: [KC][BN]
            for (int idx = tid; idx < KC * (BN / 2); idx += nthreads) {
                const int kk = idx / (BN / 2), p = idx % (BN / 2);
                const int64_t k = k0 + kk, n = n0 + 2 * p;
                int bytes = 0;
                if (k < k_end && n < g.N)
                    bytes = (g.N - n >= 2) ? 16 : 8;
                cp_async16_zfill(Bs + kk * PB + 2 * p, bytes ? (g.B + k * g.ldb + n) : g.B, bytes);
            }
        } else { // B is N x K: [BN][KC]
            for (int idx = tid; idx < BN * (KC / 2); idx += nthreads) {
                const int r = idx / (KC / 2), p = idx % (KC / 2);
                const int64_t n = n0 + r, k = k0 + 2 * p;
                int bytes = 0;
                if (n < g.N && k < k_end)
                    bytes = (k_end - k >= 2) ? 16 : 8;
                cp_async16_zfill(Bs + r * PK + 2 * p, bytes ? (g.B + n * g.ldb + k) : g.B, bytes);
            }
        }
    } else {
        // unaligned operands: element-wise loads (rare: odd leading dimensions or offset views)
        if constexpr (TA) {
            for (int idx = tid; idx < KC * BM; idx += nthreads) {
                const int kk = idx / BM, c = idx % BM;
                const int64_t k = k0 + kk, m = m0 + c;
                As[kk * PA + c] = (k < k_end && m < g.M) ? g.A[k * g.lda + m] : 0.0;
            }
        } else {
            for (int idx = tid; idx < BM * KC; idx += nthreads) {
                const int r = idx / KC, c = idx % KC;
                const int64_t m = m0 + r, k = k0 + c;
                As[r * PK + c] = (m < g.M && k < k_end) ? g.A[m * g.lda + k] : 0.0;
            }
        }
        if (!load_b) {
        } else if constexpr (!TB) {
            for (int idx = tid; idx < KC * BN; idx += nthreads) {
                const int kk = idx / BN, c = idx % BN;
                const int64_t k = k0 + kk, n = n0 + c;
                Bs[kk * PB + c] = (k < k_end && n < g.N) ? g.B[k * g.ldb + n] : 0.0;
            }
        } else {
            for (int idx = tid; idx < BN * KC; idx += nthreads) {
                const int r = idx / KC, c = idx % KC;
                const int64_t n = n0 + r, k = k0 + c;
                Bs[r * PK + c] = (n < g.N && k < k_end) ? g.B[n * g.ldb + k] : 0.0;
            }
        }
    }
}

// C (M x N) = op(A) op(B).  blockIdx.x = tile_n (fastest), blockIdx.y = tile_m, blockIdx.z = split of the
// contraction range.  With `syrk`, warps whose 32 x 32 sub-tile lies strictly below the diagonal do no arithmetic
// (the reduce step mirrors those entries), and a tile on the diagonal loads its operand once.
template <bool TA, bool TB, int BM, int BN>
__global__ void __launch_bounds__(TileCfg<BM, BN>::THREADS) gemm_f64_kernel(const __grid_constant__ GemmArgs ga) {
    using Cfg = TileCfg<BM, BN>;
    constexpr int NT = Cfg::THREADS, WN = Cfg::WN, STAGES = Cfg::STAGES, NTILES = WN / 8;
    constexpr int PA = BM + 4, PB = BN + 4, PK = pitch_k(TA, TB);
    constexpr bool K4 = !TA && TB; // both operands [row][k]: lane t takes k = 4 t + j, else k = t + 4 j
    constexpr int A_ELEMS = TA ? KC * PA : BM * PK;
    constexpr int B_ELEMS = TB ? BN * PK : KC * PB;
    extern __shared__ __align__(16) double gsm[];
    double *ysm = gsm + (size_t)STAGES * (A_ELEMS + B_ELEMS); // [STAGES][KC]: the stage's piece of y (fold only)
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    // warp -> sub-tile: rotating the column by the row spreads the warps that stay active in a diagonal syrk tile
    // (column block >= row block) evenly over the four scheduler partitions (warp id mod 4)
    constexpr int WCOLS = BN / 32;
    const int wm = warp / WCOLS, wn = (warp % WCOLS + WCOLS - wm % WCOLS) % WCOLS;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
    if (ga.syrk && n0 + BN <= m0)
        return; // strictly below the diagonal: mirrored by the reduce step
    const bool warp_active = !ga.syrk || (n0 + wn * WN + WN > m0 + wm * 32);
    const bool same_tile = ga.syrk && BM == BN && m0 == n0 && (TA != TB);
    const bool diag_tile = ga.syrk && BM == BN && m0 == n0;
    if ((int)blockIdx.z >= (diag_tile ? ga.splits_diag : ga.splits))
        return;
    // fold: this CTA also forms t(X) y for its 128 columns; four of the six idle warps take 32 columns each
    const bool fold = TA && !TB && BM == 128 && BN == 128 && diag_tile && ga.yv != nullptr;
    const int yrank = wm * (wm - 1) / 2 + wn; // 0..5 over the warps below the diagonal (wn < wm)
    double ysum = 0.0;
    const int64_t kps = diag_tile ? ga.k_per_split_diag : ga.k_per_split;
    const int64_t k_begin = (int64_t)blockIdx.z * kps;
    const int64_t k_end = (k_begin + kps < ga.K) ? k_begin + kps : ga.K;
    const int64_t nchunks = (k_end > k_begin) ? (k_end - k_begin + KC - 1) / KC : 0;

    double acc[2][NTILES][4];
#pragma unroll
    for (int i = 0; i < 2; i++)
#pragma unroll
        for (int j = 0; j < NTILES; j++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                acc[i][j][e] = 0.0;
    const int g = lane / 4, t = lane % 4;

    auto stage_a = [&](int s) { return gsm + (size_t)s * (A_ELEMS + B_ELEMS); };
    auto stage_b = [&](int s) { return same_tile ? stage_a(s) : gsm + (size_t)s * (A_ELEMS + B_ELEMS) + A_ELEMS; };

    // a tile inside the operands takes the loader without bounds tests (all but the last stage of a ragged range)
    const bool interior = ga.aligned && m0 + BM <= ga.M && n0 + BN <= ga.N;
    // the thread's first source of a full stage at k_begin, and what one stage adds to it
    const double *a_src0 = TA ? ga.A + (k_begin + tid / (BM / 2)) * ga.lda + m0 + 2 * (tid % (BM / 2))
                              : ga.A + (m0 + tid / (KC / 2)) * ga.lda + k_begin + 2 * (tid % (KC / 2));
    const double *b_src0 = !TB ? ga.B + (k_begin + tid / (BN / 2)) * ga.ldb + n0 + 2 * (tid % (BN / 2))
                               : ga.B + (n0 + tid / (KC / 2)) * ga.ldb + k_begin + 2 * (tid % (KC / 2));
    const int64_t a_step = TA ? KC * ga.lda : KC, b_step = !TB ? KC * ga.ldb : KC;
    auto load = [&](int slot, int64_t chunk) {
        const int64_t k0 = k_begin + chunk * KC;
        if (interior && k0 + KC <= k_end)
            load_stage<TA, TB, BM, BN, true>(ga, stage_a(slot), stage_b(slot), m0, n0, k0, k_end, tid, NT, !same_tile,
                                             a_src0 + chunk * a_step, b_src0 + chunk * b_step);
        else
            load_stage<TA, TB, BM, BN, false>(ga, stage_a(slot), stage_b(slot), m0, n0, k0, k_end, tid, NT, !same_tile,
                                              nullptr, nullptr);
        if (fold && tid < KC / 2) { // the rows' entries of y travel with the stage (zeros beyond the range)
            const int64_t k = k0 + 2 * tid;
            const int bytes = k + 2 <= k_end ? 16 : (k < k_end ? 8 : 0);
            cp_async16_zfill(ysm + slot * KC + 2 * tid, bytes ? ga.yv + k : ga.yv, bytes);
        }
    };
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < nchunks)
            load(s, s);
        cp_async_commit();
    }
    for (int64_t ch = 0; ch < nchunks; ch++) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int64_t nx = ch + STAGES - 1;
            if (nx < nchunks)
                load((int)(nx % STAGES), nx);
            cp_async_commit();
        }
        if (!warp_active) {
            if (fold && yrank < 4) { // column yrank * 32 + lane of the tile: its 32 entries of this stage, in row order
                const double *col = stage_a((int)(ch % STAGES)) + yrank * 32 + lane;
                const double *ys = ysm + (int)(ch % STAGES) * KC;
#pragma unroll
                for (int kk = 0; kk < KC; kk += 2) {
                    const double2 yy = *reinterpret_cast<const double2 *>(ys + kk);
                    ysum = __fma_rn(col[kk * PA], yy.x, ysum);
                    ysum = __fma_rn(col[(kk + 1) * PA], yy.y, ysum);
                }
            }
            continue;
        }
        const double *As = stage_a((int)(ch % STAGES));
        const double *Bs = stage_b((int)(ch % STAGES));
        static_assert(KC % 16 == 0, "whole m16n8k16 steps per stage");
#pragma unroll
        for (int kk = 0; kk < KC; kk += 16) {
        // Fragments come in with 128-bit shared loads where the layout allows it.  An operand stored [k][row] yields
        // the same k of two 8-row blocks per load because its rows are interleaved: block b of a 16-row group holds
        // the rows 2 g + b (not g + 8 b); the epilogue undoes the interleaving.  When both operands are stored
        // [row][k], lane t takes k = 4 t + j (j = 0..3) for slot j of both (the product is the same sum in a
        // different fixed order) and a load yields two slots; next to a [k][row] operand k stays t + 4 j (the order
        // that spreads the [k][row] rows over the banks) and the [row][k] operand is read 64 bits at a time.
        double af[2][8];
#pragma unroll
        for (int mt = 0; mt < 2; mt++) {
            if constexpr (TA) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const double2 v = *reinterpret_cast<const double2 *>(As + (kk + t + 4 * j) * PA + wm * 32 + mt * 16 + 2 * g);
                    af[mt][2 * j] = v.x;
                    af[mt][2 * j + 1] = v.y;
                }
            } else if constexpr (K4) {
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    const double *row = As + (wm * 32 + mt * 16 + g + 8 * b) * PK + kk + 4 * t;
                    const double2 lo = *reinterpret_cast<const double2 *>(row), hi = *reinterpret_cast<const double2 *>(row + 2);
                    af[mt][b] = lo.x;
                    af[mt][2 + b] = lo.y;
                    af[mt][4 + b] = hi.x;
                    af[mt][6 + b] = hi.y;
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++)
                    af[mt][i] = As[(wm * 32 + mt * 16 + g + 8 * (i & 1)) * PK + kk + t + 4 * (i >> 1)];
            }
        }
#pragma unroll
        for (int q = 0; q < NTILES / 2; q++) {
            double bf[2][4];
            if constexpr (!TB) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const double2 v = *reinterpret_cast<const double2 *>(Bs + (kk + t + 4 * j) * PB + wn * WN + q * 16 + 2 * g);
                    bf[0][j] = v.x;
                    bf[1][j] = v.y;
                }
            } else if constexpr (K4) {
#pragma unroll
                for (int b = 0; b < 2; b++) {
                    const double *row = Bs + (wn * WN + q * 16 + 8 * b + g) * PK + kk + 4 * t;
                    const double2 lo = *reinterpret_cast<const double2 *>(row), hi = *reinterpret_cast<const double2 *>(row + 2);
                    bf[b][0] = lo.x;
                    bf[b][1] = lo.y;
                    bf[b][2] = hi.x;
                    bf[b][3] = hi.y;
                }
            } else {
#pragma unroll
                for (int b = 0; b < 2; b++)
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        bf[b][i] = Bs[(wn * WN + q * 16 + 8 * b + g) * PK + kk + t + 4 * i];
            }
#pragma unroll
            for (int b = 0; b < 2; b++) {
                dmma16x8x16(acc[0][2 * q + b], af[0], bf[b]);
                dmma16x8x16(acc[1][2 * q + b], af[1], bf[b]);
            }
        }
        } // kk
    }
    cp_async_wait<0>();
    if (!warp_active) {
        if (fold && yrank < 4 && m0 + yrank * 32 + lane < ga.M)
            ga.ypart[(size_t)blockIdx.z * ga.M + m0 + yrank * 32 + lane] = ysum;
        return;
    }

    // acc[mt][nt][2 h + e]: row block h of the 16-row group mt, column 2 t + e of the 8-column block nt.  Rows: block h
    // holds the rows 2 g + h when A was stored [k][row], g + 8 h otherwise.  Columns: when B was stored [k][column]
    // the blocks 2 q and 2 q + 1 interleave, so a lane owns the four adjacent columns 16 q + 4 t .. + 3 =
    // (block 2q, e 0), (block 2q+1, e 0), (block 2q, e 1), (block 2q+1, e 1).
    auto row_of = [&](int mt, int h) { return wm * 32 + mt * 16 + (TA ? 2 * g + h : g + 8 * h); };
    if (ga.splits > 1) {
        double *tile =
            ga.part + (((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * (BM * BN);
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                double *out = tile + row_of(mt, h) * BN + wn * WN;
                if constexpr (!TB) {
#pragma unroll
                    for (int q = 0; q < NTILES / 2; q++) {
                        double2 *o = reinterpret_cast<double2 *>(out + q * 16 + 4 * t);
                        o[0] = make_double2(acc[mt][2 * q][2 * h], acc[mt][2 * q + 1][2 * h]);
                        o[1] = make_double2(acc[mt][2 * q][2 * h + 1], acc[mt][2 * q + 1][2 * h + 1]);
                    }
                } else {
#pragma unroll
                    for (int nt = 0; nt < NTILES; nt++)
                        *reinterpret_cast<double2 *>(out + nt * 8 + 2 * t) =
                            make_double2(acc[mt][nt][2 * h], acc[mt][nt][2 * h + 1]);
                }
            }
    } else {
#pragma unroll
        for (int mt = 0; mt < 2; mt++)
#pragma unroll
            for (int nt = 0; nt < NTILES; nt++)
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int64_t r = m0 + row_of(mt, h);
                        const int64_t c =
                            n0 + wn * WN + (TB ? nt * 8 + 2 * t + e : (nt / 2) * 16 + 4 * t + 2 * e + (nt & 1));
                        if (r < ga.M && c < ga.N)
                            ga.C[r * ga.ldc + c] = acc[mt][nt][2 * h + e];
                    }
    }
}

// Adds the per-split tiles in split order; with `syrk` the entries of the skipped 32 x 32 sub-tiles are the mirror
// of computed ones, and when splits == 1 only the mirroring is done (the tiles were written to C directly).
template <int BM, int BN>
__global__ void gemm_reduce_kernel(const double *__restrict__ part, double *__restrict__ C, int64_t ldc, int64_t M,
                                   int64_t N, int tiles_m, int tiles_n, int splits, int splits_diag, int syrk) {
    constexpr int WN = 32;
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * N)
        return;
    const int64_t i = idx / N, j = idx % N;
    int64_t si = i, sj = j;
    if (syrk && (j / WN) * WN + WN <= (i / 32) * 32) { // (i, j) was skipped: take (j, i)
        si = j;
        sj = i;
    }
    if (splits > 1) {
        const int64_t tm = si / BM, tn = sj / BN;
        const double *p = part + ((size_t)tm * tiles_n + tn) * (BM * BN) + (si % BM) * BN + (sj % BN);
        const size_t stride = (size_t)tiles_m * tiles_n * (BM * BN);
        const int mine = (syrk && BM == BN && tm == tn) ? splits_diag : splits;
        double a = p[0];
        for (int s = 1; s < mine; s++)
            a = __dadd_rn(a, p[(size_t)s * stride]);
        C[i * ldc + j] = a;
    } else if (si != i) {
        C[i * ldc + j] = C[si * ldc + sj];
    }
}

// t(X) y: the diagonal tiles' partial sums, added in split order
__global__ void gemv_fold_kernel(const double *__restrict__ ypart, int64_t n, int splits, double *__restrict__ out) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n)
        return;
    double a = ypart[c];
    for (int s = 1; s < splits; s++)
        a = __dadd_rn(a, ypart[(size_t)s * n + c]);
    out[c] = a;
}

struct GemmPlan {
    int bm, bn, tiles_m, tiles_n, splits, splits_diag;
    int64_t k_per_split, k_per_split_diag;
    size_t scratch;
};

static size_t tile_smem(int bm, int bn, bool ta, bool tb) {
    const size_t a = ta ? (size_t)KC * (bm + 4) : (size_t)bm * pitch_k(ta, tb);
    const size_t b = tb ? (size_t)bn * pitch_k(ta, tb) : (size_t)KC * (bn + 4);
    return 3 * (a + b + KC) * 8; // TileCfg::STAGES stages of both operands and of a piece of y
}

static GemmPlan plan_gemm(int64_t M, int64_t N, int64_t K, bool syrk, bool ta, bool tb) {
    GemmPlan p;
    p.bm = M > 64 ? 128 : 64;
    p.bn = N > 64 ? 128 : 64;
    p.tiles_m = (int)((M + p.bm - 1) / p.bm);
    p.tiles_n = (int)((N + p.bn - 1) / p.bn);
    int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    if (syrk) { // tiles on or above the diagonal
        tiles = 0;
        for (int tm = 0; tm < p.tiles_m; tm++)
            for (int tn = 0; tn < p.tiles_n; tn++)
                if ((int64_t)tn * p.bn + p.bn > (int64_t)tm * p.bm)
                    tiles++;
    }
    int per_sm = (int)((220 * 1024) / tile_smem(p.bm, p.bn, ta, tb));
    if (per_sm < 1)
        per_sm = 1;
    const int max_per_sm = 2048 / ((p.bm / 32) * (p.bn / 32) * 32);
    if (per_sm > max_per_sm)
        per_sm = max_per_sm;
    if (per_sm > 4)
        per_sm = 4;
    const int64_t slots = (int64_t)sm_count() * per_sm;
    const int64_t chunks = (K + KC - 1) / KC;
    int64_t splits = slots / (tiles > 0 ? tiles : 1);
    if (splits < 1)
        splits = 1;
    auto shares = [&](int64_t want, int *count, int64_t *k_per) { // `want` shares of whole chunks
        if (want > chunks / 4)
            want = chunks / 4; // at least 4 chunks (128 rows) per share
        if (want < 1)
            want = 1;
        if (want > 512)
            want = 512;
        const int64_t cps = (chunks + want - 1) / want;
        *k_per = cps * KC;
        *count = (int)((chunks + cps - 1) / cps);
    };
    shares(splits, &p.splits, &p.k_per_split);
    p.splits_diag = p.splits;
    p.k_per_split_diag = p.k_per_split;
    const int n_diag = p.tiles_m, n_off = (int)tiles - n_diag;
    if (syrk && p.bm == p.bn && n_off > 0) {
        // a diagonal tile keeps w (w + 1) / 2 of its w x w warps busy: give it that fraction of the shares of a full
        // tile, so that every CTA runs about equally long and all of them fit the SMs at once
        const int w = p.bm / 32;
        const double rho = (w + 1) / (2.0 * w);
        int64_t so = (int64_t)(slots / (n_off + rho * n_diag));
        int64_t sd = (int64_t)(rho * so + 0.5);
        while (so > 1 && n_off * so + n_diag * (sd < 1 ? 1 : sd) > slots) {
            so--;
            sd = (int64_t)(rho * so + 0.5);
        }
        shares(so, &p.splits, &p.k_per_split);
        shares(sd, &p.splits_diag, &p.k_per_split_diag);
        if (p.splits_diag > p.splits) // the partial buffer and the grid are sized by p.splits
            p.splits = p.splits_diag, p.k_per_split = p.k_per_split_diag;
    }
    p.scratch = p.splits > 1 ? (size_t)p.splits * p.tiles_m * p.tiles_n * p.bm * p.bn * 8 : 0;
    return p;
}

template <bool TA, bool TB, int BM, int BN>
static int launch_gemm(const GemmArgs &g, const GemmPlan &p, cudaStream_t st) {
    const size_t smem = tile_smem(BM, BN, TA, TB);
    static PerDeviceOnce attr;
    if (attr.need()) {
        DB2_CUDA(cudaFuncSetAttribute(gemm_f64_kernel<TA, TB, BM, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
        attr.mark();
    }
    dim3 grid(p.tiles_n, p.tiles_m, p.splits);
    gemm_f64_kernel<TA, TB, BM, BN><<<grid, TileCfg<BM, BN>::THREADS, smem, st>>>(g);
    DB2_TRY(after_launch("gemm_f64_kernel"));
    if (p.splits > 1 || g.syrk) {
        const int64_t total = g.M * g.N;
        gemm_reduce_kernel<BM, BN><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            g.part, g.C, g.ldc, g.M, g.N, p.tiles_m, p.tiles_n, p.splits, p.splits_diag, g.syrk);
        DB2_TRY(after_launch("gemm_reduce_kernel"));
    }
    return DB2_OK;
}

template <bool TA, bool TB> static int dispatch_tiles(const GemmArgs &g, const GemmPlan &p, cudaStream_t st) {
    if (p.bm == 128 && p.bn == 128)
        return launch_gemm<TA, TB, 128, 128>(g, p, st);
    if (p.bm == 128)
        return launch_gemm<TA, TB, 128, 64>(g, p, st);
    if (p.bn == 128)
        return launch_gemm<TA, TB, 64, 128>(g, p, st);
    return launch_gemm<TA, TB, 64, 64>(g, p, st);
}

static int run_gemm(bool ta, bool tb, GemmArgs g, cudaStream_t st, void *scratch, size_t scratch_bytes) {
    if (g.M == 0 || g.N == 0)
        return DB2_OK;
    const GemmPlan p = plan_gemm(g.M, g.N, g.K, g.syrk != 0, ta, tb);
    double *yout = nullptr;
    if (g.yv) { // t(X) y folded into the syrk: partial sums behind the partial tiles; g.ypart carries the result pointer in
        DB2_CHECK(g.syrk && ta && !tb && p.bm == 128 && p.bn == 128 && aligned16(g.yv), DB2_EINVAL,
                  "t(X) y can only ride along with t(X) X on 128 x 128 tiles");
        DB2_CHECK(scratch && scratch_bytes >= p.scratch + (size_t)p.splits_diag * g.M * 8, DB2_EINVAL,
                  "syrk + gemv scratch too small");
        yout = g.ypart;
        g.ypart = reinterpret_cast<double *>(static_cast<char *>(scratch) + p.scratch);
    }
    DB2_CHECK(p.scratch == 0 || (scratch && scratch_bytes >= p.scratch), DB2_EINVAL,
              "matMul/syrk scratch too small: %zu < %zu", scratch_bytes, p.scratch);
    g.part = static_cast<double *>(scratch);
    g.splits = p.splits;
    g.k_per_split = p.k_per_split;
    g.splits_diag = p.splits_diag;
    g.k_per_split_diag = p.k_per_split_diag;
    g.aligned = aligned16(g.A) && aligned16(g.B) && (g.lda % 2 == 0) && (g.ldb % 2 == 0);
    if (!ta && !tb)
        return dispatch_tiles<false, false>(g, p, st);
    if (!ta && tb)
        return dispatch_tiles<false, true>(g, p, st);
    if (ta && !tb) {
        DB2_TRY((dispatch_tiles<true, false>(g, p, st)));
        if (yout) {
            gemv_fold_kernel<<<(unsigned)((g.M + 255) / 256), 256, 0, st>>>(g.ypart, g.M, p.splits_diag, yout);
            DB2_TRY(after_launch("gemv_fold_kernel"));
        }
        return DB2_OK;
    }
    return dispatch_tiles<true, true>(g, p, st);
}

// f32 path (gemm_tf32.cu): tcgen05 kind::tf32 with split operands
namespace tc {
size_t tf32_scratch_bytes(int64_t M, int64_t N, int64_t K, bool syrk);
int tf32_gemm(const float *A, int64_t lda, bool ta, const float *B, int64_t ldb, bool tb, float *C, int64_t ldc,
              int64_t M, int64_t N, int64_t K, bool syrk, void *scratch, size_t scratch_bytes, cudaStream_t st);
} // namespace tc

} // namespace db2

using namespace db2;

namespace db2 {
int gemm_int(int dtype, const void *lhs, int64_t lhs_ld, bool ta, const void *rhs, int64_t rhs_ld, bool tb, void *res,
             int64_t ldc, int64_t m, int64_t n, int64_t k, cudaStream_t st); // gemm_int.cu
}

static bool int_matmul_type(int dtype) {
    return dtype == DB2_I64 || dtype == DB2_I32 || dtype == DB2_U64 || dtype == DB2_U32;
}

extern "C" size_t db2k_matmul_scratch_bytes(int dtype, int64_t m, int64_t n, int64_t k) {
    if (int_matmul_type(dtype))
        return 256;
    if (dtype == DB2_F32)
        return tc::tf32_scratch_bytes(m, n, k, false);
    size_t worst = 0;
    for (int c = 0; c < 4; c++) {
        const size_t b = plan_gemm(m, n, k, false, c & 1, c & 2).scratch;
        worst = b > worst ? b : worst;
    }
    return worst + 256;
}

extern "C" int db2k_matmul(int dtype, const void *lhs, int64_t lhs_rows, int64_t lhs_cols, int64_t lhs_ld,
                           const void *rhs, int64_t rhs_rows, int64_t rhs_cols, int64_t rhs_ld, int transa, int transb,
                           void *res, int64_t res_ld, void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(dtype == DB2_F64 || dtype == DB2_F32 || int_matmul_type(dtype), DB2_EUNSUPPORTED,
              "matMul: value type %d is not implemented on the device", dtype);
    const int64_t m = transa ? lhs_cols : lhs_rows, k = transa ? lhs_rows : lhs_cols;
    const int64_t k2 = transb ? rhs_cols : rhs_rows, n = transb ? rhs_rows : rhs_cols;
    DB2_CHECK(k == k2, DB2_EINVAL, "MatMul - #cols of lhs and #rows of rhs must be the same, but got%lldand%lld",
              (long long)k, (long long)k2);
    DB2_CHECK((lhs && rhs && res) || m * n == 0, DB2_EINVAL, "null operand");
    if (int_matmul_type(dtype))
        return gemm_int(dtype, lhs, lhs_ld, transa != 0, rhs, rhs_ld, transb != 0, res, res_ld, m, n, k,
                        as_stream(stream));
    if (dtype == DB2_F32)
        return tc::tf32_gemm(static_cast<const float *>(lhs), lhs_ld, transa != 0, static_cast<const float *>(rhs),
                             rhs_ld, transb != 0, static_cast<float *>(res), res_ld, m, n, k, false, scratch,
                             scratch_bytes, as_stream(stream));
    GemmArgs g{};
    g.A = static_cast<const double *>(lhs);
    g.B = static_cast<const double *>(rhs);
    g.C = static_cast<double *>(res);
    g.lda = lhs_ld;
    g.ldb = rhs_ld;
    g.ldc = res_ld;
    g.M = m;
    g.N = n;
    g.K = k;
    g.syrk = 0;
    return run_gemm(transa != 0, transb != 0, g, as_stream(stream), scratch, scratch_bytes);
}

extern "C" size_t db2k_syrk_scratch_bytes(int dtype, int64_t rows, int64_t cols, int trans_left) {
    const int64_t n = trans_left ? cols : rows, k = trans_left ? rows : cols;
    if (dtype == DB2_F32)
        return tc::tf32_scratch_bytes(n, n, k, true);
    return plan_gemm(n, n, k, true, trans_left != 0, trans_left == 0).scratch + 256;
}

// t(X) X and t(X) y in one pass over X (f64; the reference issues syrk and gemv, Syrk.h:40-43 and Gemv.h:51-63, and
// reads X for each).  res: cols x cols, yres: cols contiguous doubles; yvec: rows contiguous doubles.
extern "C" size_t db2k_syrk_gemv_scratch_bytes(int64_t rows, int64_t cols) {
    const GemmPlan p = plan_gemm(cols, cols, rows, true, true, false);
    return p.scratch + (size_t)p.splits_diag * cols * 8 + 256;
}
extern "C" int db2k_syrk_gemv_supported(int64_t rows, int64_t cols) {
    const GemmPlan p = plan_gemm(cols, cols, rows, true, true, false);
    return rows > 0 && p.bm == 128 && p.bn == 128;
}
extern "C" int db2k_syrk_gemv(const void *arg, int64_t rows, int64_t cols, int64_t ld, const void *yvec, void *res,
                              int64_t res_ld, void *yres, void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(arg && yvec && res && yres, DB2_EINVAL, "null operand");
    DB2_CHECK(db2k_syrk_gemv_supported(rows, cols), DB2_EUNSUPPORTED, "syrk + gemv: needs more than 64 columns");
    GemmArgs g{};
    g.A = g.B = static_cast<const double *>(arg);
    g.C = static_cast<double *>(res);
    g.lda = g.ldb = ld;
    g.ldc = res_ld;
    g.M = g.N = cols;
    g.K = rows;
    g.syrk = 1;
    g.yv = static_cast<const double *>(yvec);
    g.ypart = static_cast<double *>(yres); // run_gemm moves it to the scratch area and folds into yres
    return run_gemm(true, false, g, as_stream(stream), scratch, scratch_bytes);
}

extern "C" int db2k_syrk(int dtype, const void *arg, int64_t rows, int64_t cols, int64_t ld, int trans_left, void *res,
                         int64_t res_ld, void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(dtype == DB2_F64 || dtype == DB2_F32, DB2_EUNSUPPORTED,
              "syrk: only double and float are implemented on the device");
    DB2_CHECK((arg && res) || rows * cols == 0, DB2_EINVAL, "null operand");
    if (dtype == DB2_F32) {
        const int64_t n = trans_left ? cols : rows, k = trans_left ? rows : cols;
        const float *x = static_cast<const float *>(arg);
        return tc::tf32_gemm(x, ld, trans_left != 0, x, ld, trans_left == 0, static_cast<float *>(res), res_ld, n, n, k,
                             true, scratch, scratch_bytes, as_stream(stream));
    }
    GemmArgs g{};
    g.A = g.B = static_cast<const double *>(arg);
    g.C = static_cast<double *>(res);
    g.lda = g.ldb = ld;
    g.ldc = res_ld;
    g.M = g.N = trans_left ? cols : rows;
    g.K = trans_left ? rows : cols;
    g.syrk = 1;
    // t(X) X: A is stored K x M and B is K x N;  X t(X): A is M x K and B is N x K
    return run_gemm(trans_left != 0, trans_left == 0, g, as_stream(stream), scratch, scratch_bytes);
}
