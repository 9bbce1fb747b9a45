// Row-partition scheduler for compiled pipelines on one GPU (one process per GPU; row shards across GPUs are
// combined through the context's communicator).
//
// Replaces VectorizedPipeline::apply -> MTWrapper::executeQueuePerDeviceType + CompiledPipelineTaskCUDA
// (src/runtime/local/kernels/VectorizedPipeline.h:35-69, vectorized/MTWrapper_dense.cpp:203-336,
// vectorized/TasksCUDA.cpp:21-123).  Differences by design:
//   * all rows go to the GPU (the reference gives one device a fixed 25 % and the rest to CPU workers);
//   * the batch is as large as the memory budget allows -- normally the whole row range: the operator calls inside
//     the body are deferred and fused (lazy.cu), so no intermediate of the body is ever materialised and a single
//     batch costs only inputs + results.  The reference batches by 8 MiB of row memory and allocates every
//     intermediate per batch;
//   * with one batch a ROWS/COLS result IS the body's result object (no copy); with several batches the slices are
//     copied device-to-device into the full result like TasksCUDA.cpp:77-102;
//   * ADD, MIN and MAX partials are combined on the device (the reference throws for MIN/MAX on the GPU,
//     TasksCUDA.cpp:113-116), then across the row shards of all ranks with one all-reduce per result.
// Contract with the body (the same as the reference's, vectorized/Tasks.h:85-110, TasksCUDA.cpp:33-46): it receives
// freshly created row views of the ROWS inputs and the broadcast inputs with one extra reference each, releases all
// of them itself, and returns results it allocated (each *outputs[i] is NULL on entry).
#include "runtime.h"

#include <vector>

using namespace db2;

typedef void (*db2_pipeline_fn)(db2_matrix ***outputs, db2_matrix **inputs, db2_context *ctx);

static bool is_broadcast(int64_t split, const db2_matrix *m) {
    return split == DB2_SPLIT_NONE || (split == DB2_SPLIT_ROWS && m->rows == 1);
}

static int combine_op(int64_t combine) {
    return combine == DB2_COMBINE_ADD ? DB2_ADD : (combine == DB2_COMBINE_MIN ? DB2_MIN : DB2_MAX);
}

extern "C" int db2_vectorizedPipeline(db2_context *ctx, db2_matrix **outputs, size_t numOutputs, const int *isScalar,
                                      db2_matrix **inputs, size_t numInputs, const int64_t *outRows,
                                      const int64_t *outCols, const int64_t *splits, const int64_t *combines,
                                      db2_pipeline_fn fun, int64_t batch_rows) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && outputs && fun && (inputs || numInputs == 0) && splits && combines, DB2_EINVAL, "null argument");
    bind_device(ctx);
    // length of the row range = the tallest ROWS input (MTWrapper.h:116-140)
    int64_t len = 0;
    size_t row_mem = 0;
    for (size_t i = 0; i < numInputs; i++) {
        if (isScalar && isScalar[i])
            continue;
        DB2_CHECK(inputs[i], DB2_EINVAL, "null pipeline input %zu", i);
        DB2_CHECK(splits[i] == DB2_SPLIT_NONE || splits[i] == DB2_SPLIT_ROWS, DB2_EINVAL, "unknown VectorSplit %lld",
                  (long long)splits[i]);
        if (!is_broadcast(splits[i], inputs[i])) {
            len = inputs[i]->rows > len ? inputs[i]->rows : len;
            row_mem += (size_t)inputs[i]->cols * inputs[i]->esize();
        }
    }
    for (size_t o = 0; o < numOutputs; o++) {
        DB2_CHECK(combines[o] >= DB2_COMBINE_ROWS && combines[o] <= DB2_COMBINE_MAX, DB2_EINVAL,
                  "unknown VectorCombine %lld", (long long)combines[o]);
        outputs[o] = nullptr;
        if (combines[o] == DB2_COMBINE_ROWS && outCols && outCols[o] > 0)
            row_mem += (size_t)outCols[o] * 8;
    }
    if (batch_rows <= 0) {
        // the free-memory query is a slow driver call: its answer is remembered per context and only refreshed when a
        // pipeline's footprint comes near the remembered budget
        const size_t need = row_mem * (size_t)(len > 0 ? len : 1);
        if (ctx->mem_free_seen == 0 || need > ctx->mem_free_seen / 8) {
            size_t free_b = 0, total_b = 0;
            DB2_CUDA(cudaMemGetInfo(&free_b, &total_b));
            ctx->mem_free_seen = free_b + ctx->cached_bytes;
        }
        const size_t budget = ctx->mem_free_seen / 4;
        batch_rows = row_mem ? (int64_t)(budget / row_mem) : len;
        if (batch_rows < 1024)
            batch_rows = 1024;
    }
    if (batch_rows > len)
        batch_rows = len > 0 ? len : 1;
    const bool single = batch_rows >= len;

    std::vector<db2_matrix *> ins(numInputs), res(numOutputs);
    std::vector<db2_matrix **> res_slots(numOutputs);
    for (int64_t r0 = 0; r0 < len || (len == 0 && r0 == 0); r0 += batch_rows) {
        const int64_t r1 = (r0 + batch_rows < len) ? r0 + batch_rows : len;
        for (size_t i = 0; i < numInputs; i++) {
            if (isScalar && isScalar[i]) {
                ins[i] = inputs[i];
            } else if (is_broadcast(splits[i], inputs[i])) {
                ins[i] = inputs[i];
                db2_matrix_incref(inputs[i]); // the body releases its inputs
            } else {
                ins[i] = nullptr;
                DB2_TRY(db2_matrix_slice_rows(inputs[i], r0, r1, &ins[i]));
            }
        }
        for (size_t o = 0; o < numOutputs; o++) {
            res[o] = nullptr;
            res_slots[o] = &res[o];
        }
        fun(res_slots.data(), ins.data(), ctx);
        for (size_t o = 0; o < numOutputs; o++) {
            db2_matrix *b = res[o];
            DB2_CHECK(b, DB2_EINVAL, "the pipeline body returned no result %zu", o);
            const int64_t cmb = combines[o];
            if (cmb == DB2_COMBINE_ROWS || cmb == DB2_COMBINE_COLS) {
                if (single) {
                    outputs[o] = b; // ownership moves to the caller; still deferred if the body left it so
                    continue;
                }
                if (!outputs[o]) {
                    const int64_t R = cmb == DB2_COMBINE_ROWS ? len : b->rows;
                    const int64_t Cn = cmb == DB2_COMBINE_ROWS ? b->cols : len;
                    DB2_TRY(db2_matrix_create(ctx, b->dtype, R, Cn, 0, &outputs[o]));
                }
                db2_matrix *f = outputs[o];
                DB2_TRY(ensure_device(b));
                const size_t es = b->esize();
                char *dst = static_cast<char *>(f->dev_ptr()) +
                            (cmb == DB2_COMBINE_ROWS ? (size_t)r0 * f->dev_ld : (size_t)r0) * es;
                DB2_CUDA(cudaMemcpy2DAsync(dst, (size_t)f->dev_ld * es, b->dev_ptr(), (size_t)b->dev_ld * es,
                                           (size_t)b->cols * es, (size_t)b->rows, cudaMemcpyDeviceToDevice,
                                           ctx->stream));
                {
                    std::lock_guard<std::mutex> lock(ctx->mu);
                    ctx->stats.d2d_bytes += (uint64_t)b->rows * b->cols * es;
                }
                db2_matrix_decref(b);
            } else {
                if (!outputs[o]) {
                    DB2_TRY(ensure_device(b));
                    outputs[o] = b;
                } else {
                    DB2_TRY(db2_ewBinaryMat(ctx, combine_op(cmb), &outputs[o], outputs[o], b));
                    db2_matrix_decref(b);
                }
            }
        }
        if (len == 0)
            break;
    }
    // row shards of other GPUs: one all-reduce per ADD/MIN/MAX result
    if (ctx->world > 1)
        for (size_t o = 0; o < numOutputs; o++)
            if (combines[o] >= DB2_COMBINE_ADD && outputs[o])
                DB2_TRY(db2_allreduce(ctx, outputs[o], (int)combines[o]));
    (void)outRows;
    return DB2_OK;
    DB2_API_END
}
