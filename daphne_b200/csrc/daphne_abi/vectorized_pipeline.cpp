// The scheduler entry point under DAPHNE's own name.
//
// The lowering of a vectorized pipeline builds the callee name as a string
// (src/compiler/lowering/LowerToLLVMPass.cpp:727-850) and the JIT resolves it in the kernel libraries it has loaded:
//   _vectorizedPipeline__DenseMatrix_double_variadic__size_t__bool__Structure_variadic__size_t__int64_t__int64_t__
//   int64_t__int64_t__size_t__void_variadic(outputs, numOutputs, isScalar, inputs, numInputs, outRows, outCols,
//                                           splits, combines, numFuncs, fun, kId, ctx)
// (src/runtime/local/kernels/kernels.json:5159ff, kernels/VectorizedPipeline.h:35-69).  fun[] holds the compiled
// bodies,  void(DenseMatrix<VT> ***outs, Structure **ins, DaphneContext *):  the CPU body first and, under --cuda, the
// CUDA body after it (LowerToLLVMPass.cpp:588-590,665-667).
//
// This definition runs the LAST body (the CUDA one when there is one) over the whole row range on the GPU of the
// DaphneContext -- the policy of db2_vectorizedPipeline (csrc/pipeline.cu): one batch unless DAPHNE_B200_BATCH_ROWS
// asks for less, because the kernel calls inside the body are deferred and fused and no intermediate is materialised.
// Inputs are handed to the body the way the reference's tasks do (vectorized/Tasks.h:85-110): row views of ROWS inputs,
// broadcast inputs with one more reference, scalars in the pointer slot; the body releases them.  Results: ROWS / COLS
// of a single batch ARE the body's result objects; several batches are copied into place on the device; ADD / MIN /
// MAX are folded on the device and then all-reduced over the row shards of the communicator's ranks.
// To use it, libAllKernels.so must not export the symbol as well (one definition per process).
#include <B200Adapter.h>
#include <runtime/local/kernels/BinaryOpCode.h>
#include <util/ErrorHandler.h>

#include <cstdlib>
#include <vector>

namespace {

enum : int64_t { SPLIT_NONE = 0, SPLIT_ROWS = 1, CMB_ROWS = 1, CMB_COLS = 2, CMB_ADD = 3, CMB_MIN = 4, CMB_MAX = 5 };

bool broadcast(int64_t split, const Structure *s) { return split == SPLIT_NONE || s->getNumRows() == 1; }

template <typename VT>
void run(DenseMatrix<VT> **outputs, size_t numOutputs, bool *isScalar, Structure **inputs, size_t numInputs,
         int64_t *splits, int64_t *combines, size_t numFuncs, void **fun, DaphneContext *ctx) {
    using DT = DenseMatrix<VT>;
    if (!fun || numFuncs == 0)
        throw std::runtime_error("vectorizedPipeline: no compiled body");
    auto body = reinterpret_cast<void (*)(DT ***, Structure **, DaphneContext *)>(fun[numFuncs - 1]);
    b200::Call call(ctx);
    size_t len = 0;
    for (size_t i = 0; i < numInputs; i++) {
        if (isScalar[i])
            continue;
        if (splits[i] != SPLIT_NONE && splits[i] != SPLIT_ROWS)
            throw std::runtime_error("vectorizedPipeline: unknown VectorSplit");
        if (!broadcast(splits[i], inputs[i]))
            len = std::max(len, inputs[i]->getNumRows());
    }
    size_t batch = len ? len : 1;
    if (const char *e = std::getenv("DAPHNE_B200_BATCH_ROWS"))
        if (std::atoll(e) > 0)
            batch = std::min<size_t>(batch, (size_t)std::atoll(e));
    const bool single = batch >= len;
    for (size_t o = 0; o < numOutputs; o++)
        outputs[o] = nullptr;
    std::vector<Structure *> ins(numInputs);
    std::vector<DT *> res(numOutputs);
    std::vector<DT **> slots(numOutputs);
    for (size_t r0 = 0; r0 < len || (len == 0 && r0 == 0); r0 += batch) {
        const size_t r1 = std::min(r0 + batch, len);
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
                    outputs[o] = b;
                    continue;
                }
                if (cmb == CMB_COLS)
                    throw std::runtime_error("vectorizedPipeline: COLS results in several batches are not implemented");
                if (!outputs[o]) {
                    db2_matrix *full = nullptr;
                    b200::check(db2_matrix_create(call.c, b200::dtype_of<VT>(), (int64_t)len, (int64_t)b->getNumCols(), 0,
                                                  &full));
                    outputs[o] = call.template wrap<VT>(full);
                }
                // the batch's rows are written through a row view of the full result (x * 1 keeps every bit)
                db2_matrix *view = nullptr;
                b200::check(db2_matrix_slice_rows(call.in(outputs[o]), (int64_t)r0, (int64_t)r1, &view));
                const VT one = (VT)1;
                const int rc = db2_ewBinaryObjSca(call.c, (int)BinaryOpCode::MUL, &view, call.in(b), &one);
                db2_matrix_decref(view);
                b200::check(rc);
                DataObjectFactory::destroy(b);
            } else if (cmb == CMB_ADD || cmb == CMB_MIN || cmb == CMB_MAX) {
                if (!outputs[o]) {
                    outputs[o] = b;
                } else {
                    const int op = cmb == CMB_ADD ? (int)BinaryOpCode::ADD
                                                  : (cmb == CMB_MIN ? (int)BinaryOpCode::MIN : (int)BinaryOpCode::MAX);
                    db2_matrix *acc = call.in(outputs[o]);
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
    int rank = 0, world = 1;
    b200::check(db2_comm_info(call.c, &rank, &world));
    if (world > 1)
        for (size_t o = 0; o < numOutputs; o++)
            if (combines[o] >= CMB_ADD && outputs[o])
                b200::check(db2_allreduce(call.c, call.in(outputs[o]), (int)combines[o]));
}

} // namespace

#define B200_VECT(VT)                                                                                                  \
    extern "C" void                                                                                                    \
        _vectorizedPipeline__DenseMatrix_##VT##_variadic__size_t__bool__Structure_variadic__size_t__int64_t__int64_t__int64_t__int64_t__size_t__void_variadic( \
            DenseMatrix<VT> **outputs, size_t numOutputs, bool *isScalar, Structure **inputs, size_t numInputs,        \
            int64_t *outRows, int64_t *outCols, int64_t *splits, int64_t *combines, size_t numFuncs, void **fun,       \
            int kId, DaphneContext *ctx) {                                                                             \
        (void)outRows;                                                                                                 \
        (void)outCols;                                                                                                 \
        try {                                                                                                          \
            run<VT>(outputs, numOutputs, isScalar, inputs, numInputs, splits, combines, numFuncs, fun, ctx);           \
        } catch (std::exception & e) {                                                                                 \
            throw ErrorHandler::runtimeError(kId, e.what(), &(ctx->dispatchMapping));                                  \
        }                                                                                                              \
    }
B200_VECT(double)
B200_VECT(float)
