// Glue between DAPHNE's C++ data objects and the daphne_b200 C-ABI (include/daphne_b200.h).
//
// DAPHNE's kernels receive DenseMatrix<VT>* objects whose per-memory-space copies are tracked by a MetaDataObject
// (src/runtime/local/datastructures/MetaDataObject.h:39-57); the reference's CUDA kernels ask for a device pointer
// with getValues(&AllocationDescriptorCUDA) (datastructures/AllocationDescriptorCUDA.h:24-75).  This adapter plugs
// into the same mechanism with its own IAllocationDescriptor: the placement carries a db2_matrix handle, so a result
// of one kernel reaches the next kernel as a HANDLE (possibly still deferred) and the elementwise chains of a
// pipeline body are fused exactly as through the C-ABI; raw values are only produced when somebody calls getData()
// or the host asks for the values (transferFrom).
#pragma once

#include <runtime/local/context/DaphneContext.h>
#include <runtime/local/datastructures/DataObjectFactory.h>
#include <runtime/local/datastructures/DataPlacement.h>
#include <runtime/local/datastructures/DenseMatrix.h>
#include <runtime/local/datastructures/IAllocationDescriptor.h>

#include <daphne_b200.h>

#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

namespace b200 {

// Structure keeps the offsets of a view protected and DenseMatrix::offset() is private; a pointer to member formed in
// a derived class reads them without touching the reference's headers (a public accessor upstream would replace this).
struct ViewOffsets : Structure {
    static size_t row(const Structure *s) { return s->*(&ViewOffsets::row_offset); }
    static size_t col(const Structure *s) { return s->*(&ViewOffsets::col_offset); }
};

inline void check(int rc) {
    if (rc != DB2_OK)
        throw std::runtime_error(db2_last_error());
}

// value type -> db2 code (-1: not implemented on the device)
template <typename VT> constexpr int dtype_of() {
    if (std::is_same_v<VT, double>)
        return DB2_F64;
    if (std::is_same_v<VT, float>)
        return DB2_F32;
    if (std::is_same_v<VT, int64_t> || std::is_same_v<VT, long long>)
        return DB2_I64;
    if (std::is_same_v<VT, uint64_t> || std::is_same_v<VT, size_t>)
        return DB2_U64;
    if (std::is_same_v<VT, int32_t>)
        return DB2_I32;
    if (std::is_same_v<VT, uint32_t>)
        return DB2_U32;
    if (std::is_same_v<VT, uint8_t> || std::is_same_v<VT, bool>)
        return DB2_U8; // fill only
    return -1;
}
template <typename VT> void require_supported(const char *kernel) {
    if (dtype_of<VT>() < 0)
        throw std::runtime_error(std::string(kernel) + ": this value type is not implemented by the B200 kernel library");
}

// the device group of a DaphneContext (created by CUDA::createCUDAContext, or on first use) and the context kernels
// called on this thread run on: the one a scheduler worker bound with ThreadContext, else the group's first
db2_group *group(DaphneContext *ctx);
db2_context *context(DaphneContext *ctx);
void create_context(DaphneContext *ctx);
struct ThreadContext { // binds the calling thread to one context of the group until it goes out of scope
    db2_context *prev;
    explicit ThreadContext(db2_context *c);
    ~ThreadContext();
};
// Placement lists are not synchronised in the reference ("FIXME ... to avoid locking", datastructures/Structure.cpp:25);
// the workers of the scheduler share their broadcast inputs, so lookups and additions go through a striped lock keyed
// by the MetaDataObject (row views carry their own clone and do not contend).
std::mutex &mdo_mutex(const void *mdo);

struct HandleBox {
    db2_matrix *m = nullptr;
    ~HandleBox() {
        if (m)
            db2_matrix_decref(m);
    }
};

} // namespace b200

class AllocationDescriptorB200 : public IAllocationDescriptor {
    db2_context *dctx;
    int dtype;
    int64_t rows, cols;
    std::shared_ptr<b200::HandleBox> box;

  public:
    AllocationDescriptorB200(db2_context *c, int dtype, int64_t rows, int64_t cols, db2_matrix *preset = nullptr)
        : dctx(c), dtype(dtype), rows(rows), cols(cols), box(std::make_shared<b200::HandleBox>()) {
        box->m = preset; // takes over the caller's reference
    }
    [[nodiscard]] ALLOCATION_TYPE getType() const override { return ALLOCATION_TYPE::GPU_CUDA; }
    // the device id like the reference's descriptor; a further context that shares the device gets a suffix, so that
    // placements of different contexts (different streams and pools) are never mistaken for one another
    [[nodiscard]] std::string getLocation() const override {
        int dev = 0, dup = 0;
        db2_context_device(dctx, &dev);
        db2_context_ordinal(dctx, &dup);
        return dup ? std::to_string(dev) + "+" + std::to_string(dup) : std::to_string(dev);
    }
    [[nodiscard]] db2_context *context() const { return dctx; }
    void createAllocation(size_t size, bool zero) override {
        if (box->m)
            return; // the placement was created around an existing (possibly deferred) result
        const size_t es = dtype == DB2_U8 ? 1 : ((dtype == DB2_F32 || dtype == DB2_I32 || dtype == DB2_U32) ? 4 : 8);
        if ((size_t)rows * cols * es != size) { // a caller that only knows bytes
            rows = 1;
            cols = (int64_t)(size / es);
        }
        b200::check(db2_matrix_create(dctx, dtype, rows, cols, zero ? 1 : 0, &box->m));
    }
    std::shared_ptr<std::byte> getData() override {
        void *p = nullptr;
        b200::check(db2_matrix_device_ptr(box->m, &p, nullptr));
        return std::shared_ptr<std::byte>(box, static_cast<std::byte *>(p)); // keeps the handle alive
    }
    void transferTo(std::byte *src, size_t size) override {
        if (!src)
            throw std::runtime_error("src ptr requested for transfer to device is null");
        void *p = nullptr;
        b200::check(db2_matrix_device_ptr(box->m, &p, nullptr));
        b200::check(db2_memcpy_h2d(p, src, size, db2_context_stream(dctx)));
        b200::check(db2_context_sync(dctx)); // the source may be pageable memory that the caller reuses
    }
    void transferFrom(std::byte *dst, size_t size) override {
        (void)size;
        b200::check(db2_matrix_to_host(box->m, dst, cols));
    }
    [[nodiscard]] std::unique_ptr<IAllocationDescriptor> clone() const override {
        return std::make_unique<AllocationDescriptorB200>(*this);
    }
    bool operator==(const IAllocationDescriptor *other) const override {
        return getType() == other->getType() && getLocation() == other->getLocation();
    }
    [[nodiscard]] db2_matrix *handle() const { return box->m; }
};

namespace b200 {

// Collects the handles a kernel call borrows or creates and releases the temporary ones at scope exit.
class Call {
    std::vector<db2_matrix *> temps;

  public:
    DaphneContext *dctx;
    db2_context *c;
    explicit Call(DaphneContext *ctx) : dctx(ctx), c(context(ctx)) {}
    ~Call() {
        for (db2_matrix *t : temps)
            db2_matrix_decref(t);
    }
    Call(const Call &) = delete;

    // device handle of an argument: the handle of its (latest) device placement, else a new placement filled from
    // the host copy.  A row view of a device-resident parent becomes a row slice of the parent's handle.
    template <typename VT> db2_matrix *in(const DenseMatrix<VT> *m) {
        require_supported<VT>("kernel argument");
        auto *mdo = m->getMetaDataObject();
        std::lock_guard<std::mutex> lock(mdo_mutex(mdo));
        AllocationDescriptorB200 probe(c, dtype_of<VT>(), (int64_t)m->getNumRows(), (int64_t)m->getNumCols());
        const DataPlacement *dp = mdo->findDataPlacementByType(&probe, nullptr);
        if (!dp || !mdo->isLatestVersion(dp->dp_id)) {
            // the latest values may live on ANOTHER device of the group (a result of a stand-alone kernel consumed
            // by a scheduler worker): fetch them with a peer copy instead of a round trip through the host
            for (size_t id : mdo->getLatest()) {
                DataPlacement *p = mdo->getDataPlacementByID(id);
                auto *other = p ? dynamic_cast<AllocationDescriptorB200 *>(p->allocation.get()) : nullptr;
                if (!other || !other->handle() || other->context() == c)
                    continue;
                db2_matrix *mine = nullptr;
                check(db2_matrix_to_context(c, view_of(other->handle(), m), &mine));
                temps.push_back(mine);
                return mine;
            }
            m->getValues(&probe); // creates/refreshes the placement through AllocationDescriptorB200
            dp = mdo->findDataPlacementByType(&probe, nullptr);
        }
        auto *desc = dynamic_cast<AllocationDescriptorB200 *>(dp ? dp->allocation.get() : nullptr);
        if (!desc || !desc->handle())
            throw std::runtime_error("no B200 device placement for a kernel argument");
        return view_of(desc->handle(), m);
    }
    // the handle itself, or -- for a placement inherited from the parent of a view -- the same rows and columns of it
    template <typename VT> db2_matrix *view_of(db2_matrix *h, const DenseMatrix<VT> *m) {
        int64_t hr = 0, hc = 0;
        check(db2_matrix_info(h, nullptr, &hr, &hc));
        const int64_t mr = (int64_t)m->getNumRows(), mc = (int64_t)m->getNumCols();
        if (hr == mr && hc == mc)
            return h;
        const int64_t r0 = (int64_t)ViewOffsets::row(m), c0 = (int64_t)ViewOffsets::col(m);
        if (r0 + mr > hr || c0 + mc > hc)
            throw std::runtime_error("a view does not fit the device placement it inherited");
        db2_matrix *v = h;
        if (mr != hr) {
            check(db2_matrix_slice_rows(v, r0, r0 + mr, &v));
            temps.push_back(v);
        }
        if (mc != hc) {
            db2_matrix *w = nullptr;
            check(db2_matrix_slice_cols(v, c0, c0 + mc, &w));
            temps.push_back(w);
            v = w;
        }
        return v;
    }
    // handle of a pre-allocated result (the kernel overwrites it)
    template <typename VT> db2_matrix *out(DenseMatrix<VT> *m) {
        std::lock_guard<std::mutex> lock(mdo_mutex(m->getMetaDataObject()));
        AllocationDescriptorB200 probe(c, dtype_of<VT>(), (int64_t)m->getNumRows(), (int64_t)m->getNumCols());
        m->getValues(&probe); // non-const access: the device placement becomes the only latest version
        const DataPlacement *dp = m->getMetaDataObject()->findDataPlacementByType(&probe, nullptr);
        auto *desc = dynamic_cast<AllocationDescriptorB200 *>(dp ? dp->allocation.get() : nullptr);
        if (!desc || !desc->handle())
            throw std::runtime_error("no B200 device placement for a kernel result");
        return desc->handle();
    }
    // new device-only DenseMatrix around a result handle (takes over the reference)
    template <typename VT> DenseMatrix<VT> *wrap(db2_matrix *h) {
        int64_t r = 0, cc = 0;
        int dt = -1;
        check(db2_matrix_info(h, &dt, &r, &cc));
        if (dt != dtype_of<VT>()) { // an instantiation whose result type the device kernel does not produce
            db2_matrix_decref(h);
            throw std::runtime_error("the B200 kernel returned value type code " + std::to_string(dt) +
                                     " where the caller expects " + std::to_string(dtype_of<VT>()));
        }
        AllocationDescriptorB200 desc(c, dtype_of<VT>(), r, cc, h);
        return DataObjectFactory::create<DenseMatrix<VT>>((size_t)r, (size_t)cc, false, &desc);
    }
};

// Produces values that a kernel left deferred in a device placement of m (on the context that owns them), so that
// other threads can read the finished buffer.
template <typename VT> void settle(const DenseMatrix<VT> *m) {
    auto *mdo = m->getMetaDataObject();
    std::lock_guard<std::mutex> lock(mdo_mutex(mdo));
    for (size_t id : mdo->getLatest()) {
        DataPlacement *p = mdo->getDataPlacementByID(id);
        auto *d = p ? dynamic_cast<AllocationDescriptorB200 *>(p->allocation.get()) : nullptr;
        if (d && d->handle()) {
            void *ptr = nullptr;
            check(db2_matrix_device_ptr(d->handle(), &ptr, nullptr));
        }
    }
}

} // namespace b200
