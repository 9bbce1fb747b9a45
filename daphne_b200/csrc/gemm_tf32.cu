// FP32 matMul / syrk on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// The reference multiplies f32 matrices with cblas_sgemm (src/runtime/local/kernels/MatMul.cpp:31-36,284-288) and
// cblas_ssyrk (Syrk.h:80-92), i.e. with full single-precision products.  The tensor cores take f32 operands as TF32
// (10 explicit mantissa bits), so every operand is split on the way into shared memory,
//      x = hi + lo,   hi = tf32(x) (round to nearest),   lo = tf32(x - hi)   (x - hi is exact in f32),
// and three MMAs per k-step accumulate  hi*hi + hi*lo + lo*hi  in f32; the dropped lo*lo term and the rounding of lo
// are below 2^-21 relative per product, the same order as sgemm's own rounding.
//
// One CTA computes a 128 x 128 tile of C (or one split-K share of it):
//   warps 0-7  producers: 16-byte global loads -> hi/lo split -> 16-byte stores into a 3-stage ring of shared-memory
//              tiles laid out in the tensor core's canonical 128-byte-swizzled form.  Both operand majors are
//              supported by the MMA, so no transposition is needed: a tile whose contraction index is contiguous in
//              memory is stored K-major (rows of 32 k = 128 bytes), the other kind MN-major (rows of 32 m = 128 bytes,
//              4 k per swizzle atom).  Writers fence the async proxy and arrive on the stage's "full" mbarrier.
//   warp 8     one thread issues tcgen05.mma.kind::tf32 (M 128, N 128, K 8) from shared-memory descriptors; a
//              tcgen05.commit on the stage's "empty" mbarrier hands the buffer back when the MMAs have read it.
//   warps 0-3  epilogue: tcgen05.ld of the accumulator (lane = row, 32 columns at a time) and stores to C or to the
//              split-K partial buffer (summed afterwards in a fixed order: results do not depend on scheduling).
// Every mbarrier wait is bounded (about a second): on expiry the kernel raises a flag in *status, all roles fall
// through to the common exit and tensor memory is released.
#include "common.cuh"

namespace db2 {
namespace tc {

constexpr int BM = 128, BN = 128, BK = 32; // f32 elements; BK * 4 bytes = one 128-byte swizzle row
constexpr int TILE_BYTES = BM * BK * 4;    // 16 KB (A and B tiles have the same size)
constexpr int STAGE_BYTES = 4 * TILE_BYTES; // A hi, A lo, B hi, B lo
constexpr int STAGES = 3;
constexpr int PRODUCER_THREADS = 256, THREADS = PRODUCER_THREADS + 32;
constexpr int TMEM_COLS = 128;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr long long WAIT_LIMIT_CLOCKS = 2000000000LL;

struct TcArgs {
    const float *A, *B;
    float *C, *part;
    int64_t lda, ldb, ldc, M, N, K;
    int64_t k_per_split; // multiple of BK
    int splits;
    int to_part; // tiles go to the partial buffer [splits][M][N] (split-K and/or syrk mirroring)
    int vec_a, vec_b, vec_c; // 16-byte accesses allowed (base alignment and leading dimension)
    int32_t *status;
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    return ok != 0;
}
// bounded wait: false when another role gave up or the limit expired (then *abort is raised)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort) {
    if (mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort)
            return false;
        if (clock64() - t0 > WAIT_LIMIT_CLOCKS) {
            *abort = 1;
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; accumulate = 0 overwrites D
__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
                 "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
                   "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
                   "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor: start address, leading and stride byte offsets in 16-byte units, descriptor
// version 1, layout type (2 = 128-byte swizzle of 16-byte units; 1 = 128-byte swizzle of 32-byte units, the only
// swizzled form the tensor core accepts for MN-major 32-bit operands).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout_type) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout_type << 61;
    return d;
}
// Instruction descriptor of kind::tf32: f32 accumulator, tf32 operands, operand majors, N / 8, M / 16.
__host__ __device__ constexpr uint32_t instr_desc(bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ---------------------------------------------------------------------------
// operand staging
// ---------------------------------------------------------------------------
// A tile is 128 (m or n) x 32 (k) elements = 1024 packets of 16 bytes; thread t handles packets t, t+256, t+512, t+768.
//
// KMAJ (k contiguous in global memory; element (r, k) at src[(r0 + r) * ld + k]):
//   packet p: r = p / 8, kc = p % 8 (k = 4 kc);   shared offset (r/8)*1024 + (r%8)*128 + ((kc ^ r%8) * 16)
// MN-major (m contiguous; element (m, k) at src[k * ld + m0 + m]): atoms of 4 k-rows x 128 bytes (32 m), whose
// 32-byte units are swizzled with the k-row;  4 atoms along m (512 bytes apart), groups of 4 k 2048 bytes apart
//   packet p: kk = p / 32, mc = p % 32 (m = 4 mc);
//   offset (kk/4)*2048 + (mc/8)*512 + (kk%4)*128 + (((mc%8)/2 ^ kk%4) * 32) + (mc%2)*16
template <bool KMAJ>
__device__ __forceinline__ void load_tile(const float *__restrict__ src, int64_t ld, int64_t r0, int64_t R, int64_t k0,
                                          int64_t kend, bool vec, int tid, float4 (&v)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int p = tid + i * PRODUCER_THREADS;
        int64_t row, col, col_end; // global row, first column of the packet, end of the valid columns
        bool row_ok;
        if (KMAJ) {
            row = r0 + (p >> 3);
            col = k0 + (p & 7) * 4;
            row_ok = row < R;
            col_end = kend;
        } else {
            row = k0 + (p >> 5);
            col = r0 + (p & 31) * 4;
            row_ok = row < kend;
            col_end = R;
        }
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row_ok && col < col_end) {
            const float *g = src + row * ld + col;
            if (vec && col + 4 <= col_end) {
                x = __ldg(reinterpret_cast<const float4 *>(g));
            } else {
                x.x = g[0];
                if (col + 1 < col_end)
                    x.y = g[1];
                if (col + 2 < col_end)
                    x.z = g[2];
                if (col + 3 < col_end)
                    x.w = g[3];
            }
        }
        v[i] = x;
    }
}

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    // a non-finite hi (infinite or NaN operand) keeps a zero low part so that the product stays inf / NaN
    const float d = (fabsf(hi) <= 3.4028234e38f) ? (x - hi) : 0.f;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(d));
    lo = __uint_as_float(l);
}

template <bool KMAJ>
__device__ __forceinline__ void store_tile(unsigned char *hi_tile, unsigned char *lo_tile, int tid,
                                           const float4 (&v)[4]) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int p = tid + i * PRODUCER_THREADS;
        uint32_t off;
        if (KMAJ) {
            const int r = p >> 3, kc = p & 7;
            off = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((kc ^ (r & 7)) << 4));
        } else {
            const int kk = p >> 5, mc = p & 31;
            off = (uint32_t)((kk >> 2) * 2048 + (mc >> 3) * 512 + (kk & 3) * 128 + ((((mc & 7) >> 1) ^ (kk & 3)) << 5) +
                             ((mc & 1) << 4));
        }
        float4 h, l;
        split_tf32(v[i].x, h.x, l.x);
        split_tf32(v[i].y, h.y, l.y);
        split_tf32(v[i].z, h.z, l.z);
        split_tf32(v[i].w, h.w, l.w);
        *reinterpret_cast<float4 *>(hi_tile + off) = h;
        *reinterpret_cast<float4 *>(lo_tile + off) = l;
    }
}

// ---------------------------------------------------------------------------
// the kernel: grid (tiles_n, tiles_m, splits)
// ---------------------------------------------------------------------------
template <bool TA, bool TB> __global__ void __launch_bounds__(THREADS, 1) gemm_tf32_kernel(const TcArgs g) {
    constexpr bool A_KMAJ = !TA; // A stored M x K: k contiguous
    constexpr bool B_KMAJ = TB;  // B stored N x K: k contiguous
    extern __shared__ unsigned char smem_raw[];
    // the swizzle pattern is a function of the absolute shared address: tiles start on 1024-byte boundaries
    unsigned char *tiles = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles + STAGES * STAGE_BYTES);
    // bars[0..S) full, bars[S..2S) empty, bars[2S] accumulator ready; then the tensor-memory base and the abort flag
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * STAGES + 1);
    volatile int *abort = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;
    const int64_t kbeg = (int64_t)blockIdx.z * g.k_per_split;
    const int64_t kend = (kbeg + g.k_per_split < g.K) ? kbeg + g.k_per_split : g.K;
    const int nkb = (int)((kend - kbeg + BK - 1) / BK);

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(smem_u32(bars + s), PRODUCER_THREADS);
            mbar_init(smem_u32(bars + STAGES + s), 1);
        }
        mbar_init(smem_u32(bars + 2 * STAGES), 1);
        *abort = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == 8)
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // ---------------- producers ----------------
        float4 a_cur[4], b_cur[4], a_nxt[4], b_nxt[4];
        if (nkb > 0) {
            load_tile<A_KMAJ>(g.A, g.lda, m0, g.M, kbeg, kend, g.vec_a != 0, tid, a_cur);
            load_tile<B_KMAJ>(g.B, g.ldb, n0, g.N, kbeg, kend, g.vec_b != 0, tid, b_cur);
        }
        for (int kb = 0; kb < nkb; kb++) {
            const int s = kb % STAGES;
            if (kb + 1 < nkb) {
                const int64_t k1 = kbeg + (int64_t)(kb + 1) * BK;
                load_tile<A_KMAJ>(g.A, g.lda, m0, g.M, k1, kend, g.vec_a != 0, tid, a_nxt);
                load_tile<B_KMAJ>(g.B, g.ldb, n0, g.N, k1, kend, g.vec_b != 0, tid, b_nxt);
            }
            // the slot is free once the MMAs of its previous use have completed (first round: passes at once)
            if (!mbar_wait(smem_u32(bars + STAGES + s), ((kb / STAGES) & 1) ^ 1, abort))
                break;
            unsigned char *st = tiles + s * STAGE_BYTES;
            store_tile<A_KMAJ>(st, st + TILE_BYTES, tid, a_cur);
            store_tile<B_KMAJ>(st + 2 * TILE_BYTES, st + 3 * TILE_BYTES, tid, b_cur);
            fence_proxy_async_smem(); // generic-proxy stores -> visible to the tensor core's async proxy
            mbar_arrive(smem_u32(bars + s));
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a_cur[i] = a_nxt[i];
                b_cur[i] = b_nxt[i];
            }
        }
    } else {
      if (lane == 0) {
        // ---------------- MMA issuer ----------------
        constexpr uint32_t idesc = instr_desc(!A_KMAJ, !B_KMAJ);
        // per k-step of 8: K-major tiles advance 32 bytes inside the swizzle row (8-row groups 1024 bytes apart);
        // MN-major tiles advance two groups of 4 k (2048 bytes each; the 4 atoms of 32 m in a group 512 bytes apart)
        constexpr uint32_t A_STEP = A_KMAJ ? 32 : 4096, B_STEP = B_KMAJ ? 32 : 4096;
        constexpr uint32_t A_LBO = A_KMAJ ? 16 : 512, A_SBO = A_KMAJ ? 1024 : 2048, A_LT = A_KMAJ ? 2 : 1;
        constexpr uint32_t B_LBO = B_KMAJ ? 16 : 512, B_SBO = B_KMAJ ? 1024 : 2048, B_LT = B_KMAJ ? 2 : 1;
        bool ok = true;
        for (int kb = 0; kb < nkb && ok; kb++) {
            const int s = kb % STAGES;
            ok = mbar_wait(smem_u32(bars + s), (kb / STAGES) & 1, abort);
            if (!ok)
                break;
            tc_fence_after();
            const uint32_t st = smem_u32(tiles + s * STAGE_BYTES);
#pragma unroll
            for (int j = 0; j < BK / 8; j++) {
                const uint64_t a_hi = smem_desc(st + j * A_STEP, A_LBO, A_SBO, A_LT);
                const uint64_t a_lo = smem_desc(st + TILE_BYTES + j * A_STEP, A_LBO, A_SBO, A_LT);
                const uint64_t b_hi = smem_desc(st + 2 * TILE_BYTES + j * B_STEP, B_LBO, B_SBO, B_LT);
                const uint64_t b_lo = smem_desc(st + 3 * TILE_BYTES + j * B_STEP, B_LBO, B_SBO, B_LT);
                mma_tf32(tmem_base, a_lo, b_hi, idesc, (kb | j) != 0);
                mma_tf32(tmem_base, a_hi, b_lo, idesc, 1);
                mma_tf32(tmem_base, a_hi, b_hi, idesc, 1);
            }
            mma_commit(smem_u32(bars + STAGES + s));
        }
        mma_commit(smem_u32(bars + 2 * STAGES));
      }
      __syncwarp();
    }

    if (warp < 4) {
        // ---------------- epilogue: lane of tensor memory = row of the tile ----------------
        __syncwarp();
        const bool ready =
            __all_sync(0xffffffffu, nkb > 0 && mbar_wait(smem_u32(bars + 2 * STAGES), 0, abort)) != 0;
        tc_fence_after();
        const int64_t row = m0 + warp * 32 + lane;
        float *out = g.to_part ? g.part + ((int64_t)blockIdx.z * g.M + row) * g.N : g.C + row * g.ldc;
        const bool vec = g.to_part ? (g.N % 4 == 0) : (g.vec_c != 0);
        for (int c4 = 0; c4 < BN / 32; c4++) {
            uint32_t r[32];
            if (ready) {
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(c4 * 32), r);
            } else {
#pragma unroll
                for (int i = 0; i < 32; i++)
                    r[i] = 0u;
            }
            const int64_t c0 = n0 + c4 * 32;
            if (row < g.M && c0 < g.N && (ready || nkb == 0)) {
                if (vec && c0 + 32 <= g.N) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<uint4 *>(out + c0 + i) = make_uint4(r[i], r[i + 1], r[i + 2], r[i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (c0 + i < g.N)
                            out[c0 + i] = __uint_as_float(r[i]);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort)
        atomicExch(g.status, 1);
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// fixed-order sum of the split-K partial products; mirror: element (r, c) below the diagonal takes the sum of
// (c, r), which makes a syrk result exactly symmetric like the reference's (Syrk.h:65-69 copies the upper triangle)
__global__ void tf32_reduce_kernel(const float *__restrict__ part, float *__restrict__ C, int64_t ldc, int64_t M,
                                   int64_t N, int splits, int mirror) {
    const int64_t total = M * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / N, c = i % N;
        const int64_t src = (mirror && r > c) ? c * N + r : i;
        float acc = part[src];
        for (int s = 1; s < splits; s++)
            acc += part[(int64_t)s * total + src];
        C[r * ldc + c] = acc;
    }
}

struct TcPlan {
    int tiles_m, tiles_n, splits;
    int64_t k_per_split;
    size_t part_bytes;
};

static TcPlan plan_tc(int64_t M, int64_t N, int64_t K, bool syrk) {
    TcPlan p{};
    p.tiles_m = (int)((M + BM - 1) / BM);
    p.tiles_n = (int)((N + BN - 1) / BN);
    const int64_t tiles = (int64_t)p.tiles_m * p.tiles_n, nkb = (K + BK - 1) / BK;
    int64_t splits = 1;
    if (tiles < sm_count()) { // few tiles, long contraction: share the k range so that every SM has a CTA
        splits = sm_count() / tiles;
        if (splits > nkb / 8)
            splits = nkb / 8; // at least 8 k-blocks (256 k) per share
        if (splits < 1)
            splits = 1;
    }
    const int64_t kb_per = (nkb + splits - 1) / splits;
    p.splits = (int)((nkb + kb_per - 1) / (kb_per > 0 ? kb_per : 1));
    if (p.splits < 1)
        p.splits = 1;
    p.k_per_split = (kb_per > 0 ? kb_per : 1) * BK;
    p.part_bytes = (p.splits > 1 || syrk) ? (size_t)p.splits * M * N * sizeof(float) : 0;
    return p;
}

// the first 256 bytes of the scratch area hold the status word, the partial buffer follows
constexpr size_t STATUS_BYTES = 256;

size_t tf32_scratch_bytes(int64_t M, int64_t N, int64_t K, bool syrk) {
    return STATUS_BYTES + plan_tc(M, N, K, syrk).part_bytes;
}

template <bool TA, bool TB> static int launch_tc(const TcArgs &g, const TcPlan &p, cudaStream_t st) {
    static bool attr = false;
    if (!attr) {
        DB2_CUDA(cudaFuncSetAttribute(gemm_tf32_kernel<TA, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)SMEM_BYTES));
        attr = true;
    }
    dim3 grid(p.tiles_n, p.tiles_m, p.splits);
    gemm_tf32_kernel<TA, TB><<<grid, THREADS, SMEM_BYTES, st>>>(g);
    return after_launch("gemm_tf32_kernel");
}

// C (M x N, row-major, ldc) = op(A) op(B) in f32;  ta: A is stored K x M;  tb: B is stored N x K
int tf32_gemm(const float *A, int64_t lda, bool ta, const float *B, int64_t ldb, bool tb, float *C, int64_t ldc,
              int64_t M, int64_t N, int64_t K, bool syrk, void *scratch, size_t scratch_bytes, cudaStream_t st) {
    if (M == 0 || N == 0)
        return DB2_OK;
    if (K == 0) {
        DB2_CUDA(cudaMemset2DAsync(C, (size_t)ldc * 4, 0, (size_t)N * 4, (size_t)M, st));
        return DB2_OK;
    }
    const TcPlan p = plan_tc(M, N, K, syrk);
    DB2_CHECK(scratch && scratch_bytes >= STATUS_BYTES + p.part_bytes, DB2_EINVAL,
              "matMul/syrk scratch too small: %zu < %zu", scratch_bytes, STATUS_BYTES + p.part_bytes);
    TcArgs g{};
    g.A = A;
    g.B = B;
    g.C = C;
    g.lda = lda;
    g.ldb = ldb;
    g.ldc = ldc;
    g.M = M;
    g.N = N;
    g.K = K;
    g.k_per_split = p.k_per_split;
    g.splits = p.splits;
    g.to_part = p.part_bytes != 0;
    g.part = reinterpret_cast<float *>(static_cast<char *>(scratch) + STATUS_BYTES);
    g.status = static_cast<int32_t *>(scratch);
    g.vec_a = aligned16(A) && lda % 4 == 0;
    g.vec_b = aligned16(B) && ldb % 4 == 0;
    g.vec_c = aligned16(C) && ldc % 4 == 0;
    DB2_CUDA(cudaMemsetAsync(scratch, 0, sizeof(int32_t), st));
    int rc;
    if (!ta && !tb)
        rc = launch_tc<false, false>(g, p, st);
    else if (!ta && tb)
        rc = launch_tc<false, true>(g, p, st);
    else if (ta && !tb)
        rc = launch_tc<true, false>(g, p, st);
    else
        rc = launch_tc<true, true>(g, p, st);
    DB2_TRY(rc);
    if (g.to_part) {
        const int64_t total = M * N;
        int64_t blocks = (total + 255) / 256;
        if (blocks > (int64_t)sm_count() * 8)
            blocks = (int64_t)sm_count() * 8;
        tf32_reduce_kernel<<<(unsigned)blocks, 256, 0, st>>>(g.part, C, ldc, M, N, p.splits, syrk ? 1 : 0);
        DB2_TRY(after_launch("tf32_reduce_kernel"));
    }
    return DB2_OK;
}

} // namespace tc
} // namespace db2
