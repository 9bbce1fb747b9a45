// CSRMatrix operands of the B200 kernels.
//
// The reference keeps a CSRMatrix in three host arrays (src/runtime/local/datastructures/CSRMatrix.h:70-72) and has no
// device residency for it, but every Structure owns a MetaDataObject (datastructures/Structure.h:43).  The device copy
// is hung there: a data placement whose descriptor carries a db2_csr handle.  It is created the first time a B200
// kernel sees the matrix (one upload; connected components reuses G in every iteration) and dies with the object,
// i.e. when DAPHNE's _decRef__Structure releases the last reference.
//
// Results of the elementwise product are CSRMatrix objects whose VALUES LIVE ON THE DEVICE ONLY (the product itself is
// deferred into the row aggregation that consumes it): their host arrays describe an empty matrix.  The B200 kernels
// registered for CSR operands (row aggregation, product with a dense matrix) find the device placement; a CPU kernel
// would not.  Set DAPHNE_B200_CSR_HOST_COPY=1 to have every such result written back to its host arrays as well.
#pragma once

#include <B200Adapter.h>
#include <runtime/local/datastructures/CSRMatrix.h>
#include <runtime/local/kernels/AggOpCode.h>
#include <runtime/local/kernels/BinaryOpCode.h>

#include <cstdlib>
#include <cstring>

namespace b200 {

struct CsrBox {
    db2_csr *m = nullptr;
    ~CsrBox() {
        if (m)
            db2_csr_decref(m);
    }
};

} // namespace b200

class AllocationDescriptorB200Csr : public IAllocationDescriptor {
    db2_context *dctx;
    std::shared_ptr<b200::CsrBox> box;

  public:
    AllocationDescriptorB200Csr(db2_context *c, db2_csr *handle) : dctx(c), box(std::make_shared<b200::CsrBox>()) {
        box->m = handle; // takes over the caller's reference
    }
    [[nodiscard]] ALLOCATION_TYPE getType() const override { return ALLOCATION_TYPE::GPU_CUDA; }
    [[nodiscard]] std::string getLocation() const override {
        int dev = 0, dup = 0;
        db2_context_device(dctx, &dev);
        db2_context_ordinal(dctx, &dup);
        return "csr:" + std::to_string(dev) + (dup ? "+" + std::to_string(dup) : std::string());
    }
    void createAllocation(size_t, bool) override {}
    std::shared_ptr<std::byte> getData() override {
        throw std::runtime_error("a CSR device placement has no single data pointer");
    }
    void transferTo(std::byte *, size_t) override {
        throw std::runtime_error("a CSR device placement is filled from the three host arrays, not from one buffer");
    }
    void transferFrom(std::byte *, size_t) override {
        throw std::runtime_error("a CSR device placement is read back into three host arrays, not into one buffer");
    }
    [[nodiscard]] std::unique_ptr<IAllocationDescriptor> clone() const override {
        return std::make_unique<AllocationDescriptorB200Csr>(*this);
    }
    bool operator==(const IAllocationDescriptor *other) const override {
        return getType() == other->getType() && getLocation() == other->getLocation();
    }
    [[nodiscard]] db2_csr *handle() const { return box->m; }
};

namespace b200 {

template <typename VT> void require_csr_supported() {
    if (!std::is_same_v<VT, double>)
        throw std::runtime_error("CSRMatrix operands: only double is implemented by the B200 kernel library");
}

// device handle of a CSR argument: its placement on this context, created from the host arrays on first use
template <typename VT> db2_csr *csr_in(Call &call, const CSRMatrix<VT> *m) {
    require_csr_supported<VT>();
    auto *mdo = m->getMetaDataObject();
    std::lock_guard<std::mutex> lock(mdo_mutex(mdo));
    AllocationDescriptorB200Csr probe(call.c, nullptr);
    const DataPlacement *dp = mdo->findDataPlacementByType(&probe, nullptr);
    if (!dp) {
        static_assert(sizeof(size_t) == sizeof(uint64_t), "CSRMatrix indices are 64-bit");
        db2_csr *h = nullptr;
        check(db2_csr_wrap_host(call.c, DB2_F64, (int64_t)m->getNumRows(), (int64_t)m->getNumCols(), m->getValues(),
                                reinterpret_cast<const uint64_t *>(m->getColIdxs()),
                                reinterpret_cast<const uint64_t *>(m->getRowOffsets()), &h));
        AllocationDescriptorB200Csr desc(call.c, h);
        auto *added = mdo->addDataPlacement(&desc);
        mdo->addLatest(added->dp_id);
        dp = added;
    }
    auto *desc = dynamic_cast<AllocationDescriptorB200Csr *>(dp->allocation.get());
    if (!desc || !desc->handle())
        throw std::runtime_error("no B200 device placement for a CSRMatrix argument");
    return desc->handle();
}

// new CSRMatrix around a device-resident result (takes over the reference)
template <typename VT> CSRMatrix<VT> *csr_wrap(Call &call, db2_csr *h) {
    int64_t rows = 0, cols = 0, nnz = 0;
    check(db2_csr_info(h, &rows, &cols, &nnz));
    const char *copy = std::getenv("DAPHNE_B200_CSR_HOST_COPY");
    CSRMatrix<VT> *res;
    if (copy && copy[0] == '1') {
        check(db2_csr_info(h, &rows, &cols, &nnz));
        res = DataObjectFactory::create<CSRMatrix<VT>>((size_t)rows, (size_t)cols, (size_t)nnz, false);
        check(db2_csr_to_host(h, res->getValues(), reinterpret_cast<uint64_t *>(res->getColIdxs()),
                              reinterpret_cast<uint64_t *>(res->getRowOffsets())));
    } else {
        res = DataObjectFactory::create<CSRMatrix<VT>>((size_t)rows, (size_t)cols, (size_t)0, true);
    }
    AllocationDescriptorB200Csr desc(call.c, h);
    auto *mdo = res->getMetaDataObject();
    auto *added = mdo->addDataPlacement(&desc);
    mdo->addLatest(added->dp_id);
    return res;
}

// EwBinaryMat<CSRMatrix, CSRMatrix, DenseMatrix> (src/runtime/local/kernels/EwBinaryMat.h:254-317): MUL only
template <typename VT>
void csr_ew_mul(BinaryOpCode opCode, CSRMatrix<VT> *&res, const CSRMatrix<VT> *lhs, const DenseMatrix<VT> *rhs,
                DaphneContext *ctx) {
    if (opCode != BinaryOpCode::MUL)
        throw std::runtime_error("EwBinaryMat(CSR) - unknown BinaryOpCode");
    if (res)
        throw std::runtime_error("EwBinaryMat(CSR): a pre-allocated sparse result is not supported");
    Call call(ctx);
    db2_csr *r = nullptr;
    check(db2_ewMulCsrDense(call.c, &r, csr_in(call, lhs), call.in(rhs)));
    res = csr_wrap<VT>(call, r);
}

// AggRow<DenseMatrix, CSRMatrix> (src/runtime/local/kernels/AggRow.h:178-238)
template <typename VT>
void csr_agg_row(AggOpCode opCode, DenseMatrix<VT> *&res, const CSRMatrix<VT> *arg, DaphneContext *ctx) {
    Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    check(db2_aggRowCsr(call.c, static_cast<int>(opCode), &r, csr_in(call, arg)));
    if (!res)
        res = call.template wrap<VT>(r);
}

// MatMul / Gemv <DenseMatrix, CSRMatrix, DenseMatrix> (src/runtime/local/kernels/MatMul.h:60-215, Gemv.h:79-117)
template <typename VT>
void csr_mat_mul(DenseMatrix<VT> *&res, const CSRMatrix<VT> *lhs, const DenseMatrix<VT> *rhs, bool transa, bool transb,
                 DaphneContext *ctx) {
    // like the reference, which takes the flags and does not look at them ("FIXME: transpose isn't supported atm",
    // MatMul.h:222)
    (void)transa;
    (void)transb;
    Call call(ctx);
    db2_matrix *r = res ? call.out(res) : nullptr;
    check(db2_matMulCsrDense(call.c, &r, csr_in(call, lhs), call.in(rhs)));
    if (!res)
        res = call.template wrap<VT>(r);
}

template <class T> struct is_csr : std::false_type {};
template <typename VT> struct is_csr<CSRMatrix<VT>> : std::true_type {};

} // namespace b200
