// rand(rows, cols, min, max, sparsity, seed) with a device-resident result.
//
// The reference's generator (src/runtime/local/kernels/RandMatrix.h:82-161) is a sequential walk: one std::mt19937
// for the values (seed), one for the positions (seed * 3), values drawn in row-major order with zeros redrawn, and --
// for sparsity < 1 -- a selection-sampling pass over all positions that decides where values (sparsity < 0.5) or
// zeros (sparsity >= 0.5) go.  Every draw depends on how many draws came before it, and a 32-bit Mersenne twister has
// no cheap skip-ahead, so the walk is done where it is sequential anyway -- on the host, with the same standard-library
// engine and distributions, which makes the stream the reference's by construction -- in blocks of rows that go
// through two pinned staging buffers straight into the device placement: block i + 1 is generated while block i is on
// its way.  No pageable host copy of the matrix ever exists.
#include "runtime.h"

#include <cmath>
#include <random>
#include <type_traits>

namespace db2 {

namespace {

struct Stage {
    void *buf[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
    ~Stage() {
        for (int i = 0; i < 2; i++) {
            if (buf[i])
                cudaFreeHost(buf[i]);
            if (ev[i])
                cudaEventDestroy(ev[i]);
        }
    }
    int init(size_t bytes) {
        for (int i = 0; i < 2; i++) {
            DB2_CUDA(cudaMallocHost(&buf[i], bytes));
            DB2_CUDA(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming));
        }
        return DB2_OK;
    }
};

template <typename VT> int rand_impl(db2_context *ctx, db2_matrix *m, VT lo, VT hi, double sparsity, int64_t seed) {
    const int64_t rows = m->rows, cols = m->cols, total = rows * cols;
    std::mt19937 gen_val((std::mt19937::result_type)seed), gen_idx((std::mt19937::result_type)(seed * 3));
    typename std::conditional<std::is_floating_point<VT>::value, std::uniform_real_distribution<VT>,
                              std::uniform_int_distribution<VT>>::type value(lo, hi);
    std::uniform_int_distribution<int> position(0, (int)(total - 1));
    auto nonzero = [&]() {
        VT v = value(gen_val);
        while (v == 0)
            v = value(gen_val);
        return v;
    };
    const bool mostly_values = sparsity >= 0.5; // start from values and place zeros, or the other way round
    const size_t limit = (size_t)std::round((mostly_values ? 1.0 - sparsity : sparsity) * (double)total);

    int64_t block = (int64_t)((8u << 20) / (sizeof(VT) * (size_t)cols));
    block = block < 1 ? 1 : (block > rows ? rows : block);
    Stage st;
    DB2_TRY(st.init((size_t)block * cols * sizeof(VT)));
    VT *dev = static_cast<VT *>(m->dev_ptr());

    if (mostly_values && limit == 0) {
        // dense result (sparsity 1): the only pass is the value walk, streamed block by block
        int b = 0;
        for (int64_t r0 = 0; r0 < rows; r0 += block, b ^= 1) {
            const int64_t nr = rows - r0 < block ? rows - r0 : block;
            DB2_CUDA(cudaEventSynchronize(st.ev[b]));
            VT *h = static_cast<VT *>(st.buf[b]);
            for (int64_t i = 0; i < nr * cols; i++)
                h[i] = nonzero();
            DB2_CUDA(cudaMemcpyAsync(dev + r0 * m->dev_ld, h, (size_t)nr * cols * sizeof(VT), cudaMemcpyHostToDevice,
                                     ctx->stream));
            DB2_CUDA(cudaEventRecord(st.ev[b], ctx->stream));
        }
    } else {
        // the selection pass draws values (sparsity < 0.5) from the SAME value engine after the fill pass has used
        // it, so the two passes cannot be streamed independently: the matrix is assembled in one pinned buffer
        void *whole = nullptr;
        DB2_CUDA(cudaMallocHost(&whole, (size_t)total * sizeof(VT)));
        std::unique_ptr<void, void (*)(void *)> guard(whole, [](void *p) { cudaFreeHost(p); });
        VT *h = static_cast<VT *>(whole);
        for (int64_t i = 0; i < total; i++)
            h[i] = mostly_values ? nonzero() : VT(0);
        size_t placed = 0;
        for (int64_t i = 0; i < total && placed < limit; i++) {
            // selection sampling: position i is taken with probability (still to place) / (positions left)
            const double left = (double)(total - i), want = (double)(limit - placed);
            if (std::fmod((double)position(gen_idx), left) < want) {
                h[i] = mostly_values ? VT(0) : nonzero();
                placed++;
            }
        }
        DB2_CUDA(cudaMemcpyAsync(dev, h, (size_t)total * sizeof(VT), cudaMemcpyHostToDevice, ctx->stream));
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    }
    DB2_CUDA(cudaStreamSynchronize(ctx->stream)); // the staging buffers are released on return
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.h2d_bytes += (uint64_t)total * sizeof(VT);
    return DB2_OK;
}

} // namespace
} // namespace db2

using namespace db2;

extern "C" int db2_randMatrix(db2_context *ctx, db2_matrix **res, int dtype, int64_t rows, int64_t cols,
                              const void *min_p, const void *max_p, double sparsity, int64_t seed) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && min_p && max_p, DB2_EINVAL, "null argument");
    // checks and messages of RandMatrix.h:60-72
    DB2_CHECK(rows > 0, DB2_EINVAL, "RandMatrix - numRows must be > 0");
    DB2_CHECK(cols > 0, DB2_EINVAL, "RandMatrix - numCols must be > 0");
    DB2_CHECK(dtype == DB2_F64 || dtype == DB2_F32 || dtype == DB2_I64, DB2_EUNSUPPORTED,
              "randMatrix: double, float and int64 results");
    DB2_CHECK(rows * cols <= (int64_t)INT32_MAX || sparsity == 1.0, DB2_EUNSUPPORTED,
              "randMatrix: a sparse result with more than 2^31 - 1 cells (the reference draws positions as int)");
    double lo, hi;
    if (dtype == DB2_F64) {
        lo = *static_cast<const double *>(min_p);
        hi = *static_cast<const double *>(max_p);
    } else if (dtype == DB2_F32) {
        lo = *static_cast<const float *>(min_p);
        hi = *static_cast<const float *>(max_p);
    } else {
        lo = (double)*static_cast<const int64_t *>(min_p);
        hi = (double)*static_cast<const int64_t *>(max_p);
    }
    DB2_CHECK(!(lo > hi), DB2_EINVAL, "RandMatrix - min must be <= max");
    DB2_CHECK(!(lo == 0 && hi == 0), DB2_EINVAL,
              "RandMatrix - min and max must not both be zero, consider setting sparsity to zero instead");
    DB2_CHECK(sparsity >= 0.0 && sparsity <= 1.0, DB2_EINVAL, "sparsity has to be in the interval [0.0, 1.0]");
    if (seed == -1) {
        std::random_device rd;
        std::uniform_int_distribution<int64_t> pick;
        seed = pick(rd);
    }
    bind_device(ctx);
    DB2_TRY(prepare_result(ctx, res, dtype, rows, cols));
    db2_matrix *m = *res;
    DB2_CHECK(m->dev_ld == cols, DB2_EUNSUPPORTED, "randMatrix into a strided result view");
    if (dtype == DB2_F64)
        return rand_impl<double>(ctx, m, *static_cast<const double *>(min_p), *static_cast<const double *>(max_p),
                                 sparsity, seed);
    if (dtype == DB2_F32)
        return rand_impl<float>(ctx, m, *static_cast<const float *>(min_p), *static_cast<const float *>(max_p),
                                sparsity, seed);
    return rand_impl<int64_t>(ctx, m, *static_cast<const int64_t *>(min_p), *static_cast<const int64_t *>(max_p),
                              sparsity, seed);
    DB2_API_END
}
