// The scheduler entry points under DAPHNE's own names.
//
// The lowering of a vectorized pipeline builds the callee name as a string
// (src/compiler/lowering/LowerToLLVMPass.cpp:727-850) and the JIT resolves it in the kernel libraries it has loaded:
//   _vectorizedPipeline__DenseMatrix_double_variadic__size_t__bool__Structure_variadic__size_t__int64_t__int64_t__
//   int64_t__int64_t__size_t__void_variadic(outputs, numOutputs, isScalar, inputs, numInputs, outRows, outCols,
//                                           splits, combines, numFuncs, fun, kId, ctx)
// and its siblings for DenseMatrix<float>, DenseMatrix<int64_t>, CSRMatrix<double> and CSRMatrix<float> results
// (src/runtime/local/kernels/kernels.json:5159ff, kernels/VectorizedPipeline.h:35-69).  fun[] holds the compiled
// bodies,  void(DT ***outs, Structure **ins, DaphneContext *):  the CPU body first and, under --cuda, the CUDA body
// after it (LowerToLLVMPass.cpp:588-590,665-667).
//
// These definitions run the LAST body (the CUDA one when there is one) on the GPUs of the DaphneContext's device group
// (adapter.cpp).  The row range is cut into one contiguous block per device -- the reference's WorkerGPU per CUDA
// context (vectorized/MTWrapper.h:93-98) with the device actually honoured -- and every block is processed by its own
// host thread, bound to its device's context, in one batch unless DAPHNE_B200_BATCH_ROWS asks for less: the kernel
// calls inside the body are deferred and fused, so no intermediate is materialised.  Inputs are handed to the body
// the way the reference's tasks do (vectorized/Tasks.h:85-110): row views of ROWS inputs, broadcast inputs with one
// more reference, scalars in the pointer slot; the body releases them.  Results: ROWS / COLS blocks are copied into
// place on the first device (peer copies over NVLink); ADD / MIN / MAX partials are folded per device and combined
// over the devices by db2_group_allreduce (NCCL, or peer copies and a fold in device order), then over the row shards
// of other processes when the context has a communicator.
// To use them, libAllKernels.so must not export the symbols as well (one definition per process).
#include <B200Adapter.h>
#include <B200Csr.h>
#include <runtime/local/kernels/BinaryOpCode.h>
#include <util/ErrorHandler.h>

#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

namespace {

enum : int64_t { SPLIT_NONE = 0, SPLIT_ROWS = 1, CMB_ROWS = 1, CMB_COLS = 2, CMB_ADD = 3, CMB_MIN = 4, CMB_MAX = 5 };

bool broadcast(int64_t split, const Structure *s) { return split == SPLIT_NONE || s->getNumRows() == 1; }

size_t env_batch_rows() {
    if (const char *e = std::getenv("DAPHNE_B200_BATCH_ROWS"))
        if (std::atoll(e) > 0)
            return (size_t)std::atoll(e);
    return 0;
}

// Runs the body over the rows [begin, end) of the ROWS inputs on the context the calling thread is bound to and leaves
// one result object per output in outs[] (ROWS: the block's rows; COLS: the block's columns; ADD/MIN/MAX: the
// block's partial).
template <typename VT>
void run_block(DenseMatrix<VT> **outs, size_t numOutputs, bool *isScalar, Structure **inputs, size_t numInputs,
               int64_t *splits, int64_t *combines, void (*body)(DenseMatrix<VT> ***, Structure **, DaphneContext *),
               size_t begin, size_t end, DaphneContext *ctx) {
    using DT = DenseMatrix<VT>;
    b200::Call call(ctx);
    const size_t len = end - begin;
    size_t batch = len ? len : 1;
    if (size_t b = env_batch_rows())
        batch = std::min(batch, b);
    const bool single = batch >= len;
    for (size_t o = 0; o < numOutputs; o++)
        outs[o] = nullptr;
    std::vector<Structure *> ins(numInputs);
    std::vector<DT *> res(numOutputs);
    std::vector<DT **> slots(numOutputs);
    for (size_t r0 = begin; r0 < end || (len == 0 && r0 == begin); r0 += batch) {
        const size_t r1 = std::min(r0 + batch, end);
        for (size_t i = 0; i < numInputs; i++) {
            if (isScalar[i]) {
                ins[i] = inputs[i];
            } else if (broadcast(splits[i], inputs[i])) {
                ins[i] = inputs[i];
                inputs[i]->increaseRefCounter();
            } else {
                ins[i] = inputs[i]->sliceRow(r0, r1);
            }
        }
        for (size_t o = 0; o < numOutputs; o++) {
            res[o] = nullptr;
            slots[o] = &res[o];
        }
        body(slots.data(), ins.data(), ctx);
        for (size_t o = 0; o < numOutputs; o++) {
            DT *b = res[o];
            if (!b)
                throw std::runtime_error("vectorizedPipeline: the body returned no result");
            const int64_t cmb = combines[o];
            if (cmb == CMB_ROWS || cmb == CMB_COLS) {
                if (single) {
                    outs[o] = b;
                    continue;
                }
                if (!outs[o]) {
                    const int64_t R = cmb == CMB_ROWS ? (int64_t)len : (int64_t)b->getNumRows();
                    const int64_t Cn = cmb == CMB_ROWS ? (int64_t)b->getNumCols() : (int64_t)len;
                    db2_matrix *full = nullptr;
                    b200::check(db2_matrix_create(call.c, b200::dtype_of<VT>(), R, Cn, 0, &full));
                    outs[o] = call.template wrap<VT>(full);
                }
                // the batch's rows (columns) go into place on the device
                const int64_t at = (int64_t)(r0 - begin);
                b200::check(db2_matrix_copy_block(call.in(outs[o]), cmb == CMB_ROWS ? at : 0, cmb == CMB_ROWS ? 0 : at,
                                                  call.in(b)));
                DataObjectFactory::destroy(b);
            } else if (cmb == CMB_ADD || cmb == CMB_MIN || cmb == CMB_MAX) {
                if (!outs[o]) {
                    outs[o] = b;
                } else {
                    const int op = cmb == CMB_ADD ? (int)BinaryOpCode::ADD
                                                  : (cmb == CMB_MIN ? (int)BinaryOpCode::MIN : (int)BinaryOpCode::MAX);
                    db2_matrix *acc = call.in(outs[o]);
                    b200::check(db2_ewBinaryMat(call.c, op, &acc, acc, call.in(b)));
                    DataObjectFactory::destroy(b);
                }
            } else {
                throw std::runtime_error("vectorizedPipeline: unknown VectorCombine");
            }
        }
        if (len == 0)
            break;
    }
}

template <typename VT>
void run(DenseMatrix<VT> **outputs, size_t numOutputs, bool *isScalar, Structure **inputs, size_t numInputs,
         int64_t *splits, int64_t *combines, size_t numFuncs, void **fun, DaphneContext *ctx) {
    using DT = DenseMatrix<VT>;
    if (!fun || numFuncs == 0)
        throw std::runtime_error("vectorizedPipeline: no compiled body");
    auto body = reinterpret_cast<void (*)(DT ***, Structure **, DaphneContext *)>(fun[numFuncs - 1]);
    size_t len = 0;
    for (size_t i = 0; i < numInputs; i++) {
        if (isScalar[i])
            continue;
        if (splits[i] != SPLIT_NONE && splits[i] != SPLIT_ROWS)
            throw std::runtime_error("vectorizedPipeline: unknown VectorSplit");
        if (!broadcast(splits[i], inputs[i]))
            len = std::max(len, inputs[i]->getNumRows());
    }
    for (size_t o = 0; o < numOutputs; o++) {
        if (combines[o] < CMB_ROWS || combines[o] > CMB_MAX)
            throw std::runtime_error("vectorizedPipeline: unknown VectorCombine");
        outputs[o] = nullptr;
    }
    db2_group *grp = b200::group(ctx);
    int ndev = 1;
    b200::check(db2_group_size(grp, &ndev));
    if (len < (size_t)ndev) // fewer rows than devices: the first device takes them all
        ndev = 1;
    db2_context *first = nullptr;
    b200::check(db2_group_context(grp, 0, &first));

    if (ndev == 1) {
        b200::ThreadContext bind(first);
        run_block<VT>(outputs, numOutputs, isScalar, inputs, numInputs, splits, combines, body, 0, len, ctx);
    } else {
        // Values that a stand-alone kernel left deferred on some device are produced now, by this thread, so that the
        // workers only read finished buffers of other contexts.
        for (size_t i = 0; i < numInputs; i++)
            if (!isScalar[i])
                if (auto *dm = dynamic_cast<DT *>(inputs[i]))
                    b200::settle(dm);
        std::vector<std::vector<DT *>> part(ndev, std::vector<DT *>(numOutputs, nullptr));
        std::vector<std::string> err(ndev);
        std::vector<size_t> lo(ndev), hi(ndev);
        std::vector<std::thread> workers;
        for (int d = 0; d < ndev; d++) {
            const size_t base = len / ndev, extra = len % ndev;
            lo[d] = d * base + std::min<size_t>(d, extra);
            hi[d] = lo[d] + base + ((size_t)d < extra ? 1 : 0);
            workers.emplace_back([&, d] {
                try {
                    db2_context *c = nullptr;
                    b200::check(db2_group_context(grp, d, &c));
                    b200::ThreadContext bind(c);
                    run_block<VT>(part[d].data(), numOutputs, isScalar, inputs, numInputs, splits, combines, body,
                                  lo[d], hi[d], ctx);
                } catch (std::exception &e) {
                    err[d] = e.what()[0] ? e.what() : "unknown error";
                }
            });
        }
        for (auto &w : workers)
            w.join();
        auto destroy_parts = [&] {
            for (auto &p : part)
                for (DT *&m : p)
                    if (m) {
                        DataObjectFactory::destroy(m);
                        m = nullptr;
                    }
        };
        for (int d = 0; d < ndev; d++)
            if (!err[d].empty()) {
                destroy_parts();
                throw std::runtime_error("vectorizedPipeline (device index " + std::to_string(d) + "): " + err[d]);
            }
        try {
            for (size_t o = 0; o < numOutputs; o++) {
                const int64_t cmb = combines[o];
                // the handle of every device's result, looked up on that device's context
                std::vector<db2_matrix *> hs(ndev, nullptr);
                std::vector<std::unique_ptr<b200::Call>> calls;
                for (int d = 0; d < ndev; d++) {
                    db2_context *c = nullptr;
                    b200::check(db2_group_context(grp, d, &c));
                    b200::ThreadContext bind(c);
                    calls.emplace_back(new b200::Call(ctx));
                    hs[d] = calls.back()->in(part[d][o]);
                }
                b200::ThreadContext bind(first);
                b200::Call call(ctx);
                if (cmb == CMB_ROWS || cmb == CMB_COLS) {
                    int64_t R = 0, Cn = 0;
                    for (int d = 0; d < ndev; d++) {
                        int64_t r = 0, c = 0;
                        b200::check(db2_matrix_info(hs[d], nullptr, &r, &c));
                        R = cmb == CMB_ROWS ? R + r : r;
                        Cn = cmb == CMB_ROWS ? c : Cn + c;
                    }
                    db2_matrix *full = nullptr;
                    b200::check(db2_matrix_create(first, b200::dtype_of<VT>(), R, Cn, 0, &full));
                    outputs[o] = call.template wrap<VT>(full);
                    int64_t at = 0;
                    for (int d = 0; d < ndev; d++) {
                        int64_t r = 0, c = 0;
                        b200::check(db2_matrix_info(hs[d], nullptr, &r, &c));
                        b200::check(db2_matrix_copy_block(full, cmb == CMB_ROWS ? at : 0, cmb == CMB_ROWS ? 0 : at, hs[d]));
                        at += cmb == CMB_ROWS ? r : c;
                    }
                } else {
                    // the combine may replace a handle by a new matrix and releases the old one: it works on
                    // references of its own, the result objects keep theirs
                    for (int d = 0; d < ndev; d++)
                        b200::check(db2_matrix_incref(hs[d]));
                    const int rc = db2_group_allreduce(grp, hs.data(), (int)cmb);
                    if (rc != DB2_OK) {
                        const std::string msg = db2_last_error();
                        for (int d = 0; d < ndev; d++)
                            db2_matrix_decref(hs[d]);
                        throw std::runtime_error(msg);
                    }
                    outputs[o] = call.template wrap<VT>(hs[0]); // takes over the reference
                    for (int d = 1; d < ndev; d++)
                        db2_matrix_decref(hs[d]);
                }
            }
        } catch (...) {
            destroy_parts();
            for (size_t o = 0; o < numOutputs; o++)
                if (outputs[o]) {
                    DataObjectFactory::destroy(outputs[o]);
                    outputs[o] = nullptr;
                }
            throw;
        }
        // (copies that read a block made the owning stream wait for them, so the blocks can be released now)
        destroy_parts();
    }
    // row shards of other processes (one process per GPU with a communicator): one all-reduce per result
    b200::ThreadContext bind(first);
    b200::Call call(ctx);
    int rank = 0, world = 1;
    b200::check(db2_comm_info(first, &rank, &world));
    if (world > 1)
        for (size_t o = 0; o < numOutputs; o++)
            if (combines[o] >= CMB_ADD && outputs[o])
                b200::check(db2_allreduce(first, call.in(outputs[o]), (int)combines[o]));
}

// CSRMatrix results (vectorized/MTWrapper_sparse.cpp:20-151 supports only the ROWS combine for them and collects the
// tasks' row blocks in a VectorizedDataSink): the body runs once over the whole row range on the first device, so its
// result objects are the outputs and nothing has to be concatenated.
template <typename VT>
void run_csr(CSRMatrix<VT> **outputs, size_t numOutputs, bool *isScalar, Structure **inputs, size_t numInputs,
             int64_t *splits, int64_t *combines, size_t numFuncs, void **fun, DaphneContext *ctx) {
    using DT = CSRMatrix<VT>;
    if (!fun || numFuncs == 0)
        throw std::runtime_error("vectorizedPipeline: no compiled body");
    auto body = reinterpret_cast<void (*)(DT ***, Structure **, DaphneContext *)>(fun[numFuncs - 1]);
    for (size_t o = 0; o < numOutputs; o++) {
        if (combines[o] != CMB_ROWS)
            throw std::runtime_error("vectorizedPipeline: sparse results support only the ROWS combine");
        outputs[o] = nullptr;
    }
    db2_context *first = nullptr;
    b200::check(db2_group_context(b200::group(ctx), 0, &first));
    b200::ThreadContext bind(first);
    std::vector<Structure *> ins(numInputs);
    for (size_t i = 0; i < numInputs; i++) {
        if (isScalar[i]) {
            ins[i] = inputs[i];
        } else if (broadcast(splits[i], inputs[i])) {
            ins[i] = inputs[i];
            inputs[i]->increaseRefCounter();
        } else {
            ins[i] = inputs[i]->sliceRow(0, inputs[i]->getNumRows());
        }
    }
    std::vector<DT **> slots(numOutputs);
    for (size_t o = 0; o < numOutputs; o++)
        slots[o] = &outputs[o];
    body(slots.data(), ins.data(), ctx);
    for (size_t o = 0; o < numOutputs; o++)
        if (!outputs[o])
            throw std::runtime_error("vectorizedPipeline: the body returned no result");
}

} // namespace

#define B200_VECT(DTNAME, DT, RUN)                                                                                     \
    extern "C" void                                                                                                    \
        _vectorizedPipeline__##DTNAME##_variadic__size_t__bool__Structure_variadic__size_t__int64_t__int64_t__int64_t__int64_t__size_t__void_variadic( \
            DT **outputs, size_t numOutputs, bool *isScalar, Structure **inputs, size_t numInputs, int64_t *outRows,   \
            int64_t *outCols, int64_t *splits, int64_t *combines, size_t numFuncs, void **fun, int kId,                \
            DaphneContext *ctx) {                                                                                      \
        (void)outRows;                                                                                                 \
        (void)outCols;                                                                                                 \
        try {                                                                                                          \
            RUN(outputs, numOutputs, isScalar, inputs, numInputs, splits, combines, numFuncs, fun, ctx);               \
        } catch (std::exception & e) {                                                                                 \
            throw ErrorHandler::runtimeError(kId, e.what(), &(ctx->dispatchMapping));                                  \
        }                                                                                                              \
    }
B200_VECT(DenseMatrix_double, DenseMatrix<double>, run<double>)
B200_VECT(DenseMatrix_float, DenseMatrix<float>, run<float>)
B200_VECT(DenseMatrix_int64_t, DenseMatrix<int64_t>, run<int64_t>)
B200_VECT(CSRMatrix_double, CSRMatrix<double>, run_csr<double>)
B200_VECT(CSRMatrix_float, CSRMatrix<float>, run_csr<float>)
