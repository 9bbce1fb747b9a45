// TEST INFRASTRUCTURE / CPU BASELINE -- not part of the product.
//
// The column-standardisation workload run by the reference's OWN multithreaded vectorized engine: the engine sources
// (vectorized/MTWrapper_dense.cpp, MTWrapper_sparse.cpp, Tasks.cpp, the header-only workers, queues and
// LoadPartitioning) and the CPU kernels are compiled from a DAPHNE source tree where they lie, with the shim headers of
// ref_shim_engine/ standing in for the compiler-side headers; nothing of the tree is copied here.
//
// The script
//     mu = mean(X, 1); sd = sqrt(var(X, 1)); Z = (X - mu) / sd; r = sum(Z ^ 2, 0); s = sum(r);
//     m = aggMax(Z, 0); i = idxMax(Z, 0);
// lowers, under --vec, to the kernel calls made below: meanCol, varCol and idxmaxRow are not vectorizable
// (src/ir/daphneir/DaphneVectorizableOpInterface.cpp has no entry for them) and run as stand-alone single-threaded
// kernels; the elementwise ops, sumRow, maxRow and sumAll form ONE pipeline whose compiled body is `body` -- inputs
// X (ROWS), mu and sd (1-row ROWS inputs are broadcast, vectorized/Tasks.h:85-87), outputs Z, r, m (ROWS) and the
// 1 x 1 sum (ADD) -- executed by VectorizedPipeline<DenseMatrix<double>>::apply -> MTWrapper::executeCpuQueues
// (kernels/VectorizedPipeline.h:35-69, vectorized/MTWrapper_dense.cpp:88-200) with DAPHNE's defaults: STATIC
// partitioning, 96 KiB batches, one centralized queue.  Z leaves the pipeline because idxmaxRow consumes it.
#include <runtime/local/datastructures/DataObjectFactory.h>
#include <runtime/local/datastructures/DenseMatrix.h>
#include <runtime/local/kernels/AggAll.h>
#include <runtime/local/kernels/AggCol.h>
#include <runtime/local/kernels/AggRow.h>
#include <runtime/local/kernels/EwBinaryMat.h>
#include <runtime/local/kernels/EwBinaryObjSca.h>
#include <runtime/local/kernels/EwUnaryMat.h>
#include <runtime/local/kernels/VectorizedPipeline.h>

#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>

namespace {

using DM = DenseMatrix<double>;

double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// the compiled pipeline body (what LowerToLLVMPass outlines as _vectN): outs = {Z, r, m, s}, ins = {X, mu, sd};
// like the generated code it releases its inputs and its intermediates
void body(DM ***outs, Structure **ins, DaphneContext *ctx) {
    auto *X = static_cast<DM *>(ins[0]);
    auto *mu = static_cast<DM *>(ins[1]);
    auto *sd = static_cast<DM *>(ins[2]);
    DM *xc = nullptr, *Z = nullptr, *z2 = nullptr, *r = nullptr, *m = nullptr;
    ewBinaryMat<DM, DM, DM>(BinaryOpCode::SUB, xc, X, mu, ctx);
    ewBinaryMat<DM, DM, DM>(BinaryOpCode::DIV, Z, xc, sd, ctx);
    DataObjectFactory::destroy(xc);
    ewBinaryObjSca<DM, DM, double>(BinaryOpCode::POW, z2, Z, 2.0, ctx);
    aggRow<DM, DM>(AggOpCode::SUM, r, z2, ctx);
    DataObjectFactory::destroy(z2);
    aggRow<DM, DM>(AggOpCode::MAX, m, Z, ctx);
    DM *s = DataObjectFactory::create<DM>(1, 1, false);
    s->getValues()[0] = aggAll<double, DM>(AggOpCode::SUM, r, ctx);
    *outs[0] = Z;
    *outs[1] = r;
    *outs[2] = m;
    *outs[3] = s;
    DataObjectFactory::destroy(X);
    DataObjectFactory::destroy(mu);
    DataObjectFactory::destroy(sd);
}

DM *wrap(const double *p, int64_t rows, int64_t cols) {
    std::shared_ptr<double[]> sp(const_cast<double *>(p), [](double *) {});
    return DataObjectFactory::create<DM>((size_t)rows, (size_t)cols, sp);
}

} // namespace

// Runs the workload once.  X: rows x cols row-major.  Results are copied into mu, sd (cols), r, m (rows), idx (rows)
// and s (1) where the pointer is not NULL.  vectorized != 0: the engine as described above with `threads` workers
// (<= 0: one per CPU of the fake topology); vectorized == 0: the same kernels called once on the whole matrices
// (daphne without --vec).  ms[0..3] receive the wall time of the column statistics, of the pipeline (or the
// elementwise / row-aggregation calls), of idxmaxRow, and of the whole run.  Returns 0, or 1 on an exception.
extern "C" int ref_engine_standardise(const double *X, int64_t rows, int64_t cols, int threads, int vectorized,
                                      double *mu_out, double *sd_out, double *r_out, double *m_out, uint64_t *idx_out,
                                      double *s_out, double *ms) {
    try {
        DaphneContext ctx;
        ctx.config.numberOfThreads = threads;
        ctx.logger->set_level(spdlog::level::off);
        DM *Xm = wrap(X, rows, cols);
        const double t0 = now_ms();
        DM *mu = nullptr, *var = nullptr, *sd = nullptr;
        aggCol<DM, DM>(AggOpCode::MEAN, mu, Xm, &ctx);
        aggCol<DM, DM>(AggOpCode::VAR, var, Xm, &ctx);
        ewUnaryMat<DM, DM>(UnaryOpCode::SQRT, sd, var, &ctx);
        const double t1 = now_ms();
        DM *Z = nullptr, *r = nullptr, *m = nullptr, *s = nullptr;
        if (vectorized) {
            DM *outputs[4] = {nullptr, nullptr, nullptr, nullptr};
            bool isScalar[3] = {false, false, false};
            Structure *inputs[3] = {Xm, mu, sd};
            int64_t outRows[4] = {rows, rows, rows, 1}, outCols[4] = {cols, 1, 1, 1};
            int64_t splits[3] = {1, 1, 1};       // VectorSplit::ROWS; the 1-row inputs are broadcast
            int64_t combines[4] = {1, 1, 1, 3};  // ROWS, ROWS, ROWS, ADD
            void *fun[1] = {reinterpret_cast<void *>(&body)};
            vectorizedPipeline<DM>(outputs, 4, isScalar, inputs, 3, outRows, outCols, splits, combines, 1, fun, &ctx);
            Z = outputs[0];
            r = outputs[1];
            m = outputs[2];
            s = outputs[3];
        } else {
            DM *xc = nullptr, *z2 = nullptr;
            ewBinaryMat<DM, DM, DM>(BinaryOpCode::SUB, xc, Xm, mu, &ctx);
            ewBinaryMat<DM, DM, DM>(BinaryOpCode::DIV, Z, xc, sd, &ctx);
            DataObjectFactory::destroy(xc);
            ewBinaryObjSca<DM, DM, double>(BinaryOpCode::POW, z2, Z, 2.0, &ctx);
            aggRow<DM, DM>(AggOpCode::SUM, r, z2, &ctx);
            DataObjectFactory::destroy(z2);
            aggRow<DM, DM>(AggOpCode::MAX, m, Z, &ctx);
            s = DataObjectFactory::create<DM>(1, 1, false);
            s->getValues()[0] = aggAll<double, DM>(AggOpCode::SUM, r, &ctx);
        }
        const double t2 = now_ms();
        DenseMatrix<size_t> *idx = nullptr;
        aggRow<DenseMatrix<size_t>, DM>(AggOpCode::IDXMAX, idx, Z, &ctx);
        const double t3 = now_ms();
        if (ms) {
            ms[0] = t1 - t0;
            ms[1] = t2 - t1;
            ms[2] = t3 - t2;
            ms[3] = t3 - t0;
        }
        if (mu_out)
            memcpy(mu_out, mu->getValues(), cols * sizeof(double));
        if (sd_out)
            memcpy(sd_out, sd->getValues(), cols * sizeof(double));
        if (r_out)
            memcpy(r_out, r->getValues(), rows * sizeof(double));
        if (m_out)
            memcpy(m_out, m->getValues(), rows * sizeof(double));
        if (idx_out)
            for (int64_t i = 0; i < rows; i++)
                idx_out[i] = idx->getValues()[i];
        if (s_out)
            *s_out = s->getValues()[0];
        for (Structure *o : {(Structure *)Xm, (Structure *)mu, (Structure *)var, (Structure *)sd, (Structure *)Z,
                             (Structure *)r, (Structure *)m, (Structure *)s, (Structure *)idx})
            DataObjectFactory::destroy(o);
        return 0;
    } catch (const std::exception &e) {
        fprintf(stderr, "ref_engine_standardise: %s\n", e.what());
        return 1;
    }
}

// number of worker threads the engine starts for threads <= 0 (the CPUs of the fake topology)
extern "C" int ref_engine_default_threads() {
    PipelineHWlocInfo topo(QueueTypeOption::CENTRALIZED);
    return (int)topo.physicalIds.size();
}
