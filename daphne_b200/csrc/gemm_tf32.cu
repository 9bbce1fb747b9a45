// FP32 matMul / syrk on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory).
//
// The reference multiplies f32 matrices with cblas_sgemm (src/runtime/local/kernels/MatMul.cpp:31-36,284-288) and
// cblas_ssyrk (Syrk.h:80-92), i.e. with full single-precision products.  The tensor cores take f32 operands as TF32
// (10 explicit mantissa bits, the low 13 bits of the f32 pattern are ignored), so every operand is used twice,
//      x = hi + lo,   hi = x with the low 13 mantissa bits cleared (the raw tile as the tensor core reads it),
//                     lo = x - hi   (exact in f32; the tensor core keeps its leading 11 bits),
// and three MMAs per k-step accumulate  hi*hi  and  hi*lo + lo*hi  in two f32 accumulators; the dropped lo*lo term
// and the truncation of lo are about 2^-20 relative per product, the same order as sgemm's own rounding.
//
// One CTA computes a 128 x 128 tile of C (or one split-K share of it):
//   warps 0-7   producers: cp.async (16 bytes, zero-filling) of the raw f32 tiles into a 5-slot ring of shared memory,
//               directly in the tensor core's canonical 128-byte-swizzled layouts, four k-blocks ahead of their use; then
//               each thread derives the low tile (2-slot ring) from its own packets, fences the async proxy and arrives
//               on the "full" mbarrier.  Both operand majors are supported by the MMA, so nothing is transposed: a
//               tile whose contraction index is contiguous in memory is stored K-major (rows of 32 k = 128 bytes),
//               the other kind MN-major (rows of 32 m = 128 bytes, 4 k per swizzle atom of 32-byte units).
//   warp 16     one thread issues tcgen05.mma.kind::tf32 (M 128, N 128, K 8) from shared-memory descriptors; a
//               tcgen05.commit on the k-block's "done" mbarrier hands the buffers back when the MMAs have read them.
//   warps 8-15  drain: the tensor core adds into its accumulator with truncation, so after every 64 k the main
//               accumulator (double-buffered in tensor memory) is read with tcgen05.ld (lane = row) and added to a
//               register accumulator with round-to-nearest; at the end the cross terms are added and the rows are
//               stored to C or to the split-K partial buffer (summed afterwards in a fixed order).
// Every mbarrier wait is bounded (about a second): on expiry the kernel raises a flag in *status, all roles fall
// through to the common exit and tensor memory is released.
#include "common.cuh"

namespace db2 {
namespace tc {

constexpr int BM = 128, BN = 128, BK = 32; // f32 elements; BK * 4 bytes = one 128-byte swizzle row
constexpr int TILE_BYTES = BM * BK * 4;    // 16 KB (A and B tiles have the same size)
constexpr int SLOT_BYTES = 2 * TILE_BYTES;  // an A tile and a B tile
constexpr int RAW_SLOTS = 5, LOOKAHEAD = 4; // ring of raw (= high part) tiles; k-blocks copied ahead of their use
constexpr int LOW_SLOTS = 2;                // ring of low-part tiles
constexpr int CHUNK_KB = 2;              // k-blocks (64 k) accumulated in tensor memory between two promotions
constexpr int PRODUCER_THREADS = 256, DRAIN_THREADS = 256, MMA_WARP = (PRODUCER_THREADS + DRAIN_THREADS) / 32;
constexpr int THREADS = PRODUCER_THREADS + DRAIN_THREADS + 32;
constexpr int TMEM_COLS = 512; // two main accumulators and the cross-term accumulator of 128 columns each
constexpr size_t SMEM_BYTES = (size_t)(RAW_SLOTS + LOW_SLOTS) * SLOT_BYTES + 1024 /* alignment slack */ + 256;
constexpr long long WAIT_LIMIT_CLOCKS = 2000000000LL;
// The limit of every bounded wait, and a switch that keeps the MMA issuer from issuing anything.  Both exist so that a
// test can make the waits of the other roles run out on purpose (db2k_test_tf32_starve): the barriers they wait on are
// then never completed, the waits expire after the (shortened) limit, and the kernel must leave through its common
// exit with the status bit set and its tensor memory released.
__device__ long long d_wait_limit = WAIT_LIMIT_CLOCKS;
__device__ int d_starve = 0;

// bits of the status word
constexpr int STATUS_WAIT_EXPIRED = 1; // a bounded wait ran out: the result is not valid
constexpr int STATUS_NONFINITE = 2;    // a result was inf / NaN (inf / NaN operands, overflow): recomputed by the plain kernel

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
    const long long t0 = clock64(), limit = d_wait_limit;
    while (!mbar_try_wait(bar, parity)) {
        if (*abort)
            return false;
        if (clock64() - t0 > limit) {
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
                   "=r"(r[15])
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
// KMAJ (k contiguous in global memory; element (r, k) at src[(r0 + r) * ld + k]): rows of 32 k = 128 bytes whose
// 16-byte units are swizzled with the row;  groups of 8 rows 1024 bytes apart
//   packet p: r = p / 8, kc = p % 8 (k = 4 kc);   shared offset (r/8)*1024 + (r%8)*128 + ((kc ^ r%8) * 16)
// MN-major (m contiguous; element (m, k) at src[k * ld + m0 + m]): atoms of 4 k-rows x 128 bytes (32 m), whose
// 32-byte units are swizzled with the k-row;  4 atoms along m (512 bytes apart), groups of 4 k 2048 bytes apart
//   packet p: kk = p / 32, mc = p % 32 (m = 4 mc);
//   offset (kk/4)*2048 + (mc/8)*512 + (kk%4)*128 + (((mc%8)/2 ^ kk%4) * 32) + (mc%2)*16
template <bool KMAJ> __device__ __forceinline__ uint32_t packet_offset(int p) {
    if (KMAJ) {
        const int r = p >> 3, kc = p & 7;
        return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((kc ^ (r & 7)) << 4));
    }
    const int kk = p >> 5, mc = p & 31;
    return (uint32_t)((kk >> 2) * 2048 + (mc >> 3) * 512 + (kk & 3) * 128 + ((((mc & 7) >> 1) ^ (kk & 3)) << 5) +
                      ((mc & 1) << 4));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src, uint32_t src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Asynchronous copy of this thread's 4 packets of one operand tile (raw f32; missing elements are zero-filled).
template <bool KMAJ>
__device__ __forceinline__ void issue_tile(const float *__restrict__ src, int64_t ld, int64_t r0, int64_t R, int64_t k0,
                                           int64_t kend, bool vec, int tid, uint32_t tile) {
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
        int64_t valid = row_ok ? col_end - col : 0; // elements of the packet that exist
        valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
        const float *g = valid > 0 ? src + row * ld + col : src;
        const uint32_t dst = tile + packet_offset<KMAJ>(p);
        if (vec) {
            cp_async16(dst, g, (uint32_t)valid * 4u);
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++)
                cp_async4(dst + 4 * e, e < valid ? g + e : src, e < valid ? 4u : 0u);
        }
    }
}

// Per-thread plan of the 4 packets of an operand tile for k-blocks that lie completely inside the k range and
// 16-byte-aligned operands: source pointer of the first k-block (advanced by `step` elements per k-block), bytes that
// exist (0, 4, .. 16; the rest of the packet is zero-filled) and shared-memory offset.
struct PacketPlan {
    const float *src[4];
    uint32_t bytes[4], off[4];
    int64_t step;
};
template <bool KMAJ>
__device__ __forceinline__ void plan_tile(const float *__restrict__ src, int64_t ld, int64_t r0, int64_t R, int64_t k0,
                                          int tid, PacketPlan &pl) {
    pl.step = KMAJ ? BK : (int64_t)BK * ld;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int p = tid + i * PRODUCER_THREADS;
        pl.off[i] = packet_offset<KMAJ>(p);
        int64_t valid;
        const float *g;
        if (KMAJ) {
            const int64_t row = r0 + (p >> 3);
            valid = row < R ? 4 : 0;
            g = src + row * ld + k0 + (p & 7) * 4;
        } else {
            const int64_t col = r0 + (p & 31) * 4;
            valid = R - col;
            valid = valid < 0 ? 0 : (valid > 4 ? 4 : valid);
            g = src + (k0 + (p >> 5)) * ld + col;
        }
        pl.bytes[i] = (uint32_t)valid * 4u;
        pl.src[i] = valid > 0 ? g : src; // a zero-byte copy still needs a valid address
    }
}
__device__ __forceinline__ void issue_planned(PacketPlan &pl, uint32_t tile) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        cp_async16(tile + pl.off[i], pl.src[i], pl.bytes[i]);
        if (pl.bytes[i])
            pl.src[i] += pl.step;
    }
}

// The tensor core reads an f32 bit pattern as TF32 by ignoring the low 13 mantissa bits, so the raw tile already is
// the high part  hi = x with those bits cleared;  lo = x - hi  (exact in f32, 13 significant bits of which the tensor
// core again keeps the leading 11) goes to a second tile.  Two instructions per element: the producers are the
// kernel's bottleneck.  inf / NaN operands give lo = NaN and therefore non-finite results, which the drain warps detect.
__device__ __forceinline__ float low_part(float x) { return x - __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }
template <bool KMAJ> __device__ __forceinline__ void make_low_tile(unsigned char *raw, unsigned char *lo, int tid) {
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t off = packet_offset<KMAJ>(tid + i * PRODUCER_THREADS);
        const float4 x = *reinterpret_cast<const float4 *>(raw + off);
        *reinterpret_cast<float4 *>(lo + off) = make_float4(low_part(x.x), low_part(x.y), low_part(x.z), low_part(x.w));
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
    unsigned char *low_tiles = tiles + RAW_SLOTS * SLOT_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(low_tiles + LOW_SLOTS * SLOT_BYTES);
    // full[kb % 2]: low tiles of k-block kb written (and its raw tiles landed);  done[kb % RAW_SLOTS]: MMAs of kb finished
    uint64_t *full = bars, *done = bars + LOW_SLOTS, *acc_full = done + RAW_SLOTS, *acc_empty = acc_full + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
    volatile int *abort = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // tile order: bands of 8 tile rows are walked column by column, so that the CTAs resident at one time share
    // their A and B panels in L2
    int tile_m, tile_n;
    {
        const int tiles_n = gridDim.x, tiles_m = gridDim.y, lin = blockIdx.y * gridDim.x + blockIdx.x;
        const int band = lin / (8 * tiles_n), first_m = band * 8;
        const int band_rows = tiles_m - first_m < 8 ? tiles_m - first_m : 8;
        tile_m = first_m + (lin - band * 8 * tiles_n) % band_rows;
        tile_n = (lin - band * 8 * tiles_n) / band_rows;
    }
    const int64_t m0 = (int64_t)tile_m * BM, n0 = (int64_t)tile_n * BN;
    const int64_t kbeg = (int64_t)blockIdx.z * g.k_per_split;
    const int64_t kend = (kbeg + g.k_per_split < g.K) ? kbeg + g.k_per_split : g.K;
    const int nkb = (int)((kend - kbeg + BK - 1) / BK);
    const int nch = (nkb + CHUNK_KB - 1) / CHUNK_KB;

    if (tid == 0) {
        for (int s = 0; s < LOW_SLOTS; s++)
            mbar_init(smem_u32(full + s), PRODUCER_THREADS);
        for (int s = 0; s < RAW_SLOTS; s++)
            mbar_init(smem_u32(done + s), 1);
        for (int b = 0; b < 2; b++) {
            mbar_init(smem_u32(acc_full + b), 1);
            mbar_init(smem_u32(acc_empty + b), DRAIN_THREADS);
        }
        *abort = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == MMA_WARP)
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // tensor-memory columns: [0,128) and [128,256) the two main accumulators, [256,384) the cross terms
    const uint32_t tmem_cross = tmem_base + 2 * BN;

    if (warp < PRODUCER_THREADS / 32) {
        // ---------------- producers: cp.async LOOKAHEAD k-blocks ahead, then the low tiles ----------------
        auto mma_done = [&](int kb) { // the MMAs of k-block kb have completed (their slots may be rewritten)
            return mbar_wait(smem_u32(done + kb % RAW_SLOTS), (kb / RAW_SLOTS) & 1, abort);
        };
        // k-blocks are issued in order, so the planned pointers simply advance; the last, partial k-block and
        // operands without 16-byte alignment take the general path
        PacketPlan pa, pb;
        plan_tile<A_KMAJ>(g.A, g.lda, m0, g.M, kbeg, tid, pa);
        plan_tile<B_KMAJ>(g.B, g.ldb, n0, g.N, kbeg, tid, pb);
        const bool fast_a = g.vec_a != 0, fast_b = g.vec_b != 0;
        auto issue = [&](int kb) {
            const uint32_t st = smem_u32(tiles + (kb % RAW_SLOTS) * SLOT_BYTES);
            const int64_t k0 = kbeg + (int64_t)kb * BK;
            const bool whole = k0 + BK <= kend;
            if (fast_a && whole)
                issue_planned(pa, st);
            else
                issue_tile<A_KMAJ>(g.A, g.lda, m0, g.M, k0, kend, fast_a, tid, st);
            if (fast_b && whole)
                issue_planned(pb, st + TILE_BYTES);
            else
                issue_tile<B_KMAJ>(g.B, g.ldb, n0, g.N, k0, kend, fast_b, tid, st + TILE_BYTES);
        };
        for (int kb = 0; kb < LOOKAHEAD; kb++) {
            if (kb < nkb)
                issue(kb);
            cp_async_commit();
        }
        for (int kb = 0; kb < nkb; kb++) {
            cp_async_wait<LOOKAHEAD - 1>(); // this thread's packets of k-block kb have landed
            if (kb >= LOW_SLOTS && !mma_done(kb - LOW_SLOTS))
                break;
            unsigned char *raw = tiles + (kb % RAW_SLOTS) * SLOT_BYTES, *low = low_tiles + (kb % LOW_SLOTS) * SLOT_BYTES;
            make_low_tile<A_KMAJ>(raw, low, tid);
            make_low_tile<B_KMAJ>(raw + TILE_BYTES, low + TILE_BYTES, tid);
            fence_proxy_async_smem(); // own cp.async data and stores -> visible to the tensor core's async proxy
            mbar_arrive(smem_u32(full + kb % LOW_SLOTS));
            // refill the raw slot that k-block kb - 1 is leaving (its MMAs ran while this block was prepared)
            const int kn = kb + LOOKAHEAD;
            if (kn < nkb) {
                if (kn >= RAW_SLOTS && !mma_done(kn - RAW_SLOTS))
                    break;
                issue(kn);
            }
            cp_async_commit();
        }
        cp_async_wait<0>();
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            constexpr uint32_t idesc = instr_desc(!A_KMAJ, !B_KMAJ);
            // per k-step of 8: K-major tiles advance 32 bytes inside the swizzle row (8-row groups 1024 bytes apart);
            // MN-major tiles advance two groups of 4 k (2048 bytes each; the 4 atoms of 32 m of a group 512 apart)
            constexpr uint32_t A_STEP = A_KMAJ ? 32 : 4096, B_STEP = B_KMAJ ? 32 : 4096;
            constexpr uint32_t A_LBO = A_KMAJ ? 16 : 512, A_SBO = A_KMAJ ? 1024 : 2048, A_LT = A_KMAJ ? 2 : 1;
            constexpr uint32_t B_LBO = B_KMAJ ? 16 : 512, B_SBO = B_KMAJ ? 1024 : 2048, B_LT = B_KMAJ ? 2 : 1;
            bool ok = d_starve == 0; // (test switch: the issuer stays silent and everybody else's wait runs out)
            for (int kb = 0; kb < nkb && ok; kb++) {
                const int c = kb / CHUNK_KB, b = c & 1;
                const bool chunk_start = kb % CHUNK_KB == 0;
                if (chunk_start && c >= 2) // the drain warps have taken chunk c - 2 out of this accumulator
                    ok = mbar_wait(smem_u32(acc_empty + b), ((c >> 1) - 1) & 1, abort);
                ok = ok && mbar_wait(smem_u32(full + kb % LOW_SLOTS), (kb / LOW_SLOTS) & 1, abort);
                if (!ok)
                    break;
                tc_fence_after();
                const uint32_t raw = smem_u32(tiles + (kb % RAW_SLOTS) * SLOT_BYTES);
                const uint32_t low = smem_u32(low_tiles + (kb % LOW_SLOTS) * SLOT_BYTES);
                const uint32_t tmem_main = tmem_base + (uint32_t)b * BN;
#pragma unroll
                for (int j = 0; j < BK / 8; j++) {
                    const uint64_t a_hi = smem_desc(raw + j * A_STEP, A_LBO, A_SBO, A_LT);
                    const uint64_t a_lo = smem_desc(low + j * A_STEP, A_LBO, A_SBO, A_LT);
                    const uint64_t b_hi = smem_desc(raw + TILE_BYTES + j * B_STEP, B_LBO, B_SBO, B_LT);
                    const uint64_t b_lo = smem_desc(low + TILE_BYTES + j * B_STEP, B_LBO, B_SBO, B_LT);
                    mma_tf32(tmem_cross, a_lo, b_hi, idesc, (kb | j) != 0);
                    mma_tf32(tmem_cross, a_hi, b_lo, idesc, 1);
                    mma_tf32(tmem_main, a_hi, b_hi, idesc, !(chunk_start && j == 0));
                }
                mma_commit(smem_u32(done + kb % RAW_SLOTS));
                if (kb % CHUNK_KB == CHUNK_KB - 1 || kb == nkb - 1)
                    mma_commit(smem_u32(acc_full + b));
            }
        }
        __syncwarp();
    } else {
        // ---------------- drain warps: lane of tensor memory = row of the tile ----------------
        // The tensor core adds into its f32 accumulator with truncation, which drifts with the number of additions;
        // every CHUNK_KB k-blocks the main accumulator is therefore taken out and added (round to nearest) to a
        // register accumulator.  The cross terms are 2^-10 of the main ones and stay in tensor memory to the end.
        // a warp reaches the tensor-memory lanes 32 (warp % 4) .. +31; two warps share a lane quarter and take 64
        // columns each
        const int q = warp & 3, half = (warp - PRODUCER_THREADS / 32) >> 2;
        constexpr int HN = BN / 2;
        float acc[HN];
#pragma unroll
        for (int i = 0; i < HN; i++)
            acc[i] = 0.f;
        bool ok = true;
        for (int c = 0; c <= nch && nch > 0; c++) {
            const bool cross = c == nch; // last round: the cross-term accumulator (complete with the last chunk)
            const int b = c & 1;
            if (!cross)
                ok = __all_sync(0xffffffffu, ok && mbar_wait(smem_u32(acc_full + b), (c >> 1) & 1, abort)) != 0;
            if (!ok)
                break;
            tc_fence_after();
            const uint32_t src =
                (cross ? tmem_cross : tmem_base + (uint32_t)b * BN) + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * HN);
#pragma unroll
            for (int c4 = 0; c4 < HN / 16; c4++) {
                uint32_t r[16];
                tmem_ld16(src + (uint32_t)(c4 * 16), r);
#pragma unroll
                for (int i = 0; i < 16; i++)
                    acc[c4 * 16 + i] += __uint_as_float(r[i]);
            }
            if (!cross) {
                tc_fence_before();
                mbar_arrive(smem_u32(acc_empty + b));
            }
        }
        // inf / NaN anywhere in this row of the tile (an inf or NaN operand, whose low part is NaN, or an overflow):
        // the split product does not keep IEEE semantics there, the plain kernel recomputes the product
        bool non_finite = false;
#pragma unroll
        for (int i = 0; i < HN; i++)
            non_finite |= (__float_as_uint(acc[i]) & 0x7F800000u) == 0x7F800000u;
        if (non_finite)
            atomicOr(g.status, STATUS_NONFINITE);
        const int64_t row = m0 + q * 32 + lane;
        if (ok && row < g.M) {
            float *out = g.to_part ? g.part + ((int64_t)blockIdx.z * g.M + row) * g.N : g.C + row * g.ldc;
            const bool vec = g.to_part ? (g.N % 4 == 0) : (g.vec_c != 0);
#pragma unroll
            for (int c4 = 0; c4 < HN / 32; c4++) {
                const int64_t c0 = n0 + half * HN + c4 * 32;
                if (c0 >= g.N)
                    break;
                if (vec && c0 + 32 <= g.N) {
#pragma unroll
                    for (int i = 0; i < 32; i += 4)
                        *reinterpret_cast<float4 *>(out + c0 + i) = make_float4(
                            acc[c4 * 32 + i], acc[c4 * 32 + i + 1], acc[c4 * 32 + i + 2], acc[c4 * 32 + i + 3]);
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (c0 + i < g.N)
                            out[c0 + i] = acc[c4 * 32 + i];
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (tid == 0 && *abort)
        atomicOr(g.status, STATUS_WAIT_EXPIRED);
    if (warp == MMA_WARP) {
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

// inf / NaN: the split products cannot keep IEEE semantics (inf * 1 becomes inf * 1 + NaN * 1), so the whole product
// is recomputed with plain f32 FMAs.  Launched after every tensor-core product; returns at once unless the drain
// warps saw a non-finite result and raised STATUS_NONFINITE.
__global__ void __launch_bounds__(256)
    gemm_f32_plain_kernel(const TcArgs g, int ta, int tb) {
    if (!(*g.status & STATUS_NONFINITE))
        return;
    const int64_t total = g.M * g.N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / g.N, c = i % g.N;
        float acc = 0.f;
        for (int64_t k = 0; k < g.K; k++) {
            const float a = ta ? g.A[k * g.lda + r] : g.A[r * g.lda + k];
            const float b = tb ? g.B[c * g.ldb + k] : g.B[k * g.ldb + c];
            acc = fmaf(a, b, acc);
        }
        g.C[r * g.ldc + c] = acc;
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
    static PerDeviceOnce attr;
    if (attr.need()) {
        DB2_CUDA(cudaFuncSetAttribute(gemm_tf32_kernel<TA, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)SMEM_BYTES));
        attr.mark();
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
    gemm_f32_plain_kernel<<<sm_count() * 4, 256, 0, st>>>(g, ta ? 1 : 0, tb ? 1 : 0);
    return after_launch("gemm_f32_plain_kernel");
}

} // namespace tc
} // namespace db2

// Test hook, not part of the public interface: sets the limit of the kernel's bounded waits (in clock cycles; <= 0
// restores the default of about a second) and switches the MMA issuer off (starve != 0) or back on, on the current device.
extern "C" int db2k_test_tf32_starve(long long limit_clocks, int starve) {
    const long long limit = limit_clocks > 0 ? limit_clocks : db2::tc::WAIT_LIMIT_CLOCKS;
    DB2_CUDA(cudaMemcpyToSymbol(db2::tc::d_wait_limit, &limit, sizeof(limit)));
    DB2_CUDA(cudaMemcpyToSymbol(db2::tc::d_starve, &starve, sizeof(starve)));
    return DB2_OK;
}
