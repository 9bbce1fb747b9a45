// FP64 contractions on the tensor cores: MatMul (all four transpose combinations) and Syrk (t(X) X / X t(X)).
//
// Blackwell's tcgen05 tensor path has no FP64 kind, so the FP64 contraction is the warp-level DMMA
// (mma.sync.aligned.m8n8k4.f64), fed from shared memory tiles that are filled with 16-byte cp.async copies in a
// 4-stage ring.  Tile layouts are chosen so that every fragment load is one conflict-free 64-bit shared load per
// thread: an operand whose contraction index is contiguous in memory is stored [row][KC + 4], the other kind is stored
// [k][tile + 4]; both pitches are 4 mod 16 doubles, which spreads the 8 x 4 fragment of a half warp over all banks.
//
// The tall-skinny products of the workloads (t(X) X with 8.4 M x 512, t(P) X with 1 M x 50) contract over the ROWS:
// the row range is split over gridDim.z, each split accumulates a private tile and writes it to scratch, and a second
// kernel adds the splits in a fixed order (deterministic, no atomics).  Syrk computes only the tiles on and above the
// diagonal (36 of 64 tiles for d = 512) and mirrors them in the reduce step.
#include "common.cuh"

namespace db2 {

constexpr int KC = 16;     // contraction depth per stage
constexpr int BN = 64;     // tile columns
constexpr int STAGES = 4;
constexpr int PK = KC + 4; // pitch of a [row][k] tile (doubles)

__device__ __forceinline__ void dmma8x8x4(double &c0, double &c1, double a, double b) {
    asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};\n"
                 : "+d"(c0), "+d"(c1)
                 : "d"(a), "d"(b));
}
// 16-byte async copy with zero fill: `bytes` (0, 8 or 16) are read from global, the rest of the slot is zeroed
__device__ __forceinline__ void cp_async16_zfill(void *smem_dst, const void *gsrc, int bytes) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gsrc), "r"(bytes) : "memory");
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
    int syrk;            // only tiles with tile_n*BN + BN > tile_m*BM are computed (upper triangle incl. diagonal)
    int aligned;         // operands allow 16-byte copies (bases 16-byte aligned, even leading dimensions)
};

// Loads one stage.  TA: A is stored K x M (contraction index = row);  !TA: A is M x K.  Same for TB with N.
template <bool TA, bool TB, int BM>
__device__ __forceinline__ void load_stage(const GemmArgs &g, double *As, double *Bs, int64_t m0, int64_t n0,
                                           int64_t k0, int64_t k_end, int tid, int nthreads) {
    constexpr int PA = BM + 4, PB = BN + 4;
    if (g.aligned) {
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
        if constexpr (!TB) { // B is K x N: [KC][BN]
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
        if constexpr (!TB) {
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
// contraction range.  BM x BN tile, (BM / 32) x 2 warps of 32 x 32.
template <bool TA, bool TB, int BM>
__global__ void __launch_bounds__(BM * 2) gemm_f64_kernel(const __grid_constant__ GemmArgs g) {
    constexpr int NT = BM * 2;
    constexpr int PA = BM + 4, PB = BN + 4;
    constexpr int A_ELEMS = TA ? KC * PA : BM * PK;
    constexpr int B_ELEMS = TB ? BN * PK : KC * PB;
    extern __shared__ __align__(16) double gsm[];
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const int wm = warp / 2, wn = warp % 2;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
    if (g.syrk && n0 + BN <= m0)
        return; // strictly below the diagonal: mirrored by the reduce step
    const int64_t k_begin = (int64_t)blockIdx.z * g.k_per_split;
    const int64_t k_end = (k_begin + g.k_per_split < g.K) ? k_begin + g.k_per_split : g.K;
    const int64_t nchunks = (k_end > k_begin) ? (k_end - k_begin + KC - 1) / KC : 0;

    double acc[4][4][2];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
            acc[i][j][0] = acc[i][j][1] = 0.0;

    auto stage_a = [&](int s) { return gsm + (size_t)s * (A_ELEMS + B_ELEMS); };
    auto stage_b = [&](int s) { return gsm + (size_t)s * (A_ELEMS + B_ELEMS) + A_ELEMS; };

#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < nchunks)
            load_stage<TA, TB, BM>(g, stage_a(s), stage_b(s), m0, n0, k_begin + (int64_t)s * KC, k_end, tid, NT);
        cp_async_commit();
    }
    for (int64_t ch = 0; ch < nchunks; ch++) {
        cp_async_wait<STAGES - 2>();
        __syncthreads();
        {
            const int64_t nx = ch + STAGES - 1;
            if (nx < nchunks)
                load_stage<TA, TB, BM>(g, stage_a((int)(nx % STAGES)), stage_b((int)(nx % STAGES)), m0, n0,
                                       k_begin + nx * KC, k_end, tid, NT);
            cp_async_commit();
        }
        const double *As = stage_a((int)(ch % STAGES));
        const double *Bs = stage_b((int)(ch % STAGES));
#pragma unroll
        for (int kk = 0; kk < KC; kk += 4) {
            double a[4], b[4];
#pragma unroll
            for (int mt = 0; mt < 4; mt++) {
                const int m = wm * 32 + mt * 8 + lane / 4;
                a[mt] = TA ? As[(kk + lane % 4) * PA + m] : As[m * PK + kk + lane % 4];
            }
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int n = wn * 32 + nt * 8 + lane / 4;
                b[nt] = TB ? Bs[n * PK + kk + lane % 4] : Bs[(kk + lane % 4) * PB + n];
            }
#pragma unroll
            for (int mt = 0; mt < 4; mt++)
#pragma unroll
                for (int nt = 0; nt < 4; nt++)
                    dmma8x8x4(acc[mt][nt][0], acc[mt][nt][1], a[mt], b[nt]);
        }
    }
    cp_async_wait<0>();

    if (g.splits > 1) {
        double *tile = g.part + (((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * (BM * BN);
#pragma unroll
        for (int mt = 0; mt < 4; mt++)
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int r = wm * 32 + mt * 8 + lane / 4, c = wn * 32 + nt * 8 + (lane % 4) * 2;
                *reinterpret_cast<double2 *>(tile + r * BN + c) = make_double2(acc[mt][nt][0], acc[mt][nt][1]);
            }
    } else {
#pragma unroll
        for (int mt = 0; mt < 4; mt++)
#pragma unroll
            for (int nt = 0; nt < 4; nt++) {
                const int64_t r = m0 + wm * 32 + mt * 8 + lane / 4, c = n0 + wn * 32 + nt * 8 + (lane % 4) * 2;
                if (r < g.M) {
                    if (c < g.N)
                        g.C[r * g.ldc + c] = acc[mt][nt][0];
                    if (c + 1 < g.N)
                        g.C[r * g.ldc + c + 1] = acc[mt][nt][1];
                }
            }
    }
}

// Adds the per-split tiles in split order; with `syrk` the strictly lower part is the mirror of the upper one, and
// when splits == 1 only the mirroring is done (the tiles were written to C directly).
template <int BM>
__global__ void gemm_reduce_kernel(const double *__restrict__ part, double *__restrict__ C, int64_t ldc, int64_t M,
                                   int64_t N, int tiles_m, int tiles_n, int splits, int syrk) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= M * N)
        return;
    const int64_t i = idx / N, j = idx % N;
    int64_t si = i, sj = j;
    if (syrk && (j / BN) * BN + BN <= (i / BM) * BM) { // (i, j) lies in a tile that was skipped: take (j, i)
        si = j;
        sj = i;
    }
    if (splits > 1) {
        const int64_t tm = si / BM, tn = sj / BN;
        const double *p = part + ((size_t)tm * tiles_n + tn) * (BM * BN) + (si % BM) * BN + (sj % BN);
        const size_t stride = (size_t)tiles_m * tiles_n * (BM * BN);
        double a = p[0];
        for (int s = 1; s < splits; s++)
            a = __dadd_rn(a, p[(size_t)s * stride]);
        C[i * ldc + j] = a;
    } else if (si != i) {
        C[i * ldc + j] = C[si * ldc + sj];
    }
}

struct GemmPlan {
    int bm, tiles_m, tiles_n, splits;
    int64_t k_per_split;
    size_t scratch;
};

static GemmPlan plan_gemm(int64_t M, int64_t N, int64_t K, bool syrk) {
    GemmPlan p;
    // tall-skinny contractions (K much larger than the output) use the smaller tile and split the contraction range
    const bool tall = K >= 64 * (M > N ? M : N) || M * N <= (int64_t)BN * 64 * 148;
    p.bm = (M <= 64 || (tall && K > 8 * M)) ? 64 : 128;
    p.tiles_m = (int)((M + p.bm - 1) / p.bm);
    p.tiles_n = (int)((N + BN - 1) / BN);
    int64_t tiles = (int64_t)p.tiles_m * p.tiles_n;
    if (syrk) { // tiles on or above the diagonal
        tiles = 0;
        for (int tm = 0; tm < p.tiles_m; tm++)
            for (int tn = 0; tn < p.tiles_n; tn++)
                if ((int64_t)tn * BN + BN > (int64_t)tm * p.bm)
                    tiles++;
    }
    const size_t smem = (size_t)STAGES * ((size_t)KC * (p.bm + 4) + (size_t)KC * (BN + 4)) * 8; // upper bound
    int per_sm = (int)((200 * 1024) / smem);
    if (per_sm < 1)
        per_sm = 1;
    if (per_sm > (p.bm == 64 ? 4 : 2))
        per_sm = (p.bm == 64 ? 4 : 2);
    const int64_t slots = (int64_t)sm_count() * per_sm;
    const int64_t chunks = (K + KC - 1) / KC;
    int64_t splits = slots / (tiles > 0 ? tiles : 1);
    if (splits < 1)
        splits = 1;
    if (splits > chunks / 8)
        splits = chunks / 8 > 0 ? chunks / 8 : 1; // at least 8 chunks (128 rows) per split
    if (splits > 512)
        splits = 512;
    const int64_t cps = (chunks + splits - 1) / splits;
    p.k_per_split = cps * KC;
    p.splits = (int)((chunks + cps - 1) / cps);
    p.scratch = p.splits > 1 ? (size_t)p.splits * p.tiles_m * p.tiles_n * p.bm * BN * 8 : 0;
    return p;
}

template <bool TA, bool TB, int BM> static int launch_gemm(const GemmArgs &g, const GemmPlan &p, cudaStream_t st) {
    constexpr int A_ELEMS = TA ? KC * (BM + 4) : BM * PK;
    constexpr int B_ELEMS = TB ? BN * PK : KC * (BN + 4);
    const size_t smem = (size_t)STAGES * (A_ELEMS + B_ELEMS) * sizeof(double);
    static bool attr = false;
    if (!attr) {
        DB2_CUDA(cudaFuncSetAttribute(gemm_f64_kernel<TA, TB, BM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)smem));
        attr = true;
    }
    dim3 grid(p.tiles_n, p.tiles_m, p.splits);
    gemm_f64_kernel<TA, TB, BM><<<grid, BM * 2, smem, st>>>(g);
    DB2_TRY(after_launch("gemm_f64_kernel"));
    if (p.splits > 1 || g.syrk) {
        const int64_t total = g.M * g.N;
        gemm_reduce_kernel<BM><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(g.part, g.C, g.ldc, g.M, g.N,
                                                                                p.tiles_m, p.tiles_n, p.splits, g.syrk);
        DB2_TRY(after_launch("gemm_reduce_kernel"));
    }
    return DB2_OK;
}

static int run_gemm(bool ta, bool tb, GemmArgs g, cudaStream_t st, void *scratch, size_t scratch_bytes) {
    if (g.M == 0 || g.N == 0)
        return DB2_OK;
    const GemmPlan p = plan_gemm(g.M, g.N, g.K, g.syrk != 0);
    DB2_CHECK(p.scratch == 0 || (scratch && scratch_bytes >= p.scratch), DB2_EINVAL,
              "matMul/syrk scratch too small: %zu < %zu", scratch_bytes, p.scratch);
    g.part = static_cast<double *>(scratch);
    g.splits = p.splits;
    g.k_per_split = p.k_per_split;
    g.aligned = aligned16(g.A) && aligned16(g.B) && (g.lda % 2 == 0) && (g.ldb % 2 == 0);
#define DB2_GEMM_CASE(TA_, TB_)                                                                                        \
    if (ta == TA_ && tb == TB_)                                                                                        \
        return p.bm == 64 ? launch_gemm<TA_, TB_, 64>(g, p, st) : launch_gemm<TA_, TB_, 128>(g, p, st);
    DB2_GEMM_CASE(false, false)
    DB2_GEMM_CASE(false, true)
    DB2_GEMM_CASE(true, false)
    DB2_GEMM_CASE(true, true)
#undef DB2_GEMM_CASE
    return DB2_OK;
}

} // namespace db2

using namespace db2;

extern "C" size_t db2k_matmul_scratch_bytes(int dtype, int64_t m, int64_t n, int64_t k) {
    (void)dtype;
    return plan_gemm(m, n, k, false).scratch + 256;
}

extern "C" int db2k_matmul(int dtype, const void *lhs, int64_t lhs_rows, int64_t lhs_cols, int64_t lhs_ld,
                           const void *rhs, int64_t rhs_rows, int64_t rhs_cols, int64_t rhs_ld, int transa, int transb,
                           void *res, int64_t res_ld, void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(dtype == DB2_F64, DB2_EUNSUPPORTED, "matMul: only double is implemented on the device");
    const int64_t m = transa ? lhs_cols : lhs_rows, k = transa ? lhs_rows : lhs_cols;
    const int64_t k2 = transb ? rhs_cols : rhs_rows, n = transb ? rhs_rows : rhs_cols;
    DB2_CHECK(k == k2, DB2_EINVAL, "MatMul - #cols of lhs and #rows of rhs must be the same, but got%lldand%lld",
              (long long)k, (long long)k2);
    DB2_CHECK((lhs && rhs && res) || m * n == 0, DB2_EINVAL, "null operand");
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
    (void)dtype;
    const int64_t n = trans_left ? cols : rows, k = trans_left ? rows : cols;
    return plan_gemm(n, n, k, true).scratch + 256;
}

extern "C" int db2k_syrk(int dtype, const void *arg, int64_t rows, int64_t cols, int64_t ld, int trans_left, void *res,
                         int64_t res_ld, void *scratch, size_t scratch_bytes, void *stream) {
    DB2_CHECK(dtype == DB2_F64, DB2_EUNSUPPORTED, "syrk: only double is implemented on the device");
    DB2_CHECK((arg && res) || rows * cols == 0, DB2_EINVAL, "null operand");
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
