// Cross-GPU combine of row-sharded results: one process per GPU, NCCL over NVLink/NVSwitch.
//
// The path shards by rows, so the only exchanges are the VectorCombine reductions of small partials (ADD/MIN/MAX of
// d x d, 1 x d and 1 x 1 results; src/runtime/local/vectorized/Tasks.cpp:51-82 does them under a mutex on the host)
// and, for connected components, the all-gather of the label vector.  Both run on the context's compute stream, so
// they are ordered after the kernels that produce their input without any host synchronisation.  The messages are a
// few KB to 2 MB: latency-bound, one collective per pipeline, never one per batch.
//
// NCCL is loaded with dlopen at first use (the library of the process if one is already loaded, e.g. PyTorch's), so
// single-GPU users need no NCCL at all.  No TMA/bulk loads with cluster multicast are used anywhere in this library.
#include "runtime.h"

#include <dlfcn.h>

namespace db2 {

// the few NCCL declarations needed (public API of nccl.h, stable across 2.x)
typedef struct ncclComm *ncclComm_t;
typedef struct {
    char internal[128];
} ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclInt64 = 4, ncclUint64 = 5, ncclFloat32 = 7, ncclFloat64 = 8 };
enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3 };

struct Nccl {
    void *handle = nullptr;
    int (*GetUniqueId)(ncclUniqueId *) = nullptr;
    int (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};

static Nccl *nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {"libnccl.so.2", "libnccl.so"};
        for (const char *nm : names) {
            n.handle = dlopen(nm, RTLD_NOW | RTLD_GLOBAL);
            if (n.handle)
                break;
        }
        if (!n.handle)
            return;
        n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(dlsym(n.handle, "ncclGetUniqueId"));
        n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(dlsym(n.handle, "ncclCommInitRank"));
        n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(dlsym(n.handle, "ncclCommDestroy"));
        n.AllReduce = reinterpret_cast<decltype(n.AllReduce)>(dlsym(n.handle, "ncclAllReduce"));
        n.AllGather = reinterpret_cast<decltype(n.AllGather)>(dlsym(n.handle, "ncclAllGather"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(dlsym(n.handle, "ncclGetErrorString"));
    });
    const bool ok = n.handle && n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.AllReduce && n.AllGather;
    return ok ? &n : nullptr;
}

#define DB2_NCCL(call)                                                                                                 \
    do {                                                                                                               \
        int r__ = (call);                                                                                              \
        if (r__ != ncclSuccess)                                                                                        \
            return set_error(DB2_ENCCL, "%s failed: %s", #call,                                                        \
                             nccl()->GetErrorString ? nccl()->GetErrorString(r__) : "NCCL error");                     \
    } while (0)

static int nccl_dtype(int dtype) {
    switch (dtype) {
    case DB2_F64: return ncclFloat64;
    case DB2_F32: return ncclFloat32;
    case DB2_I64: return ncclInt64;
    default: return ncclUint64;
    }
}

} // namespace db2

using namespace db2;

extern "C" {

int db2_comm_unique_id(void *id128) {
    DB2_CHECK(id128, DB2_EINVAL, "null id buffer");
    Nccl *n = nccl();
    DB2_CHECK(n, DB2_ENCCL, "NCCL library (libnccl.so.2) could not be loaded");
    ncclUniqueId id;
    DB2_NCCL(n->GetUniqueId(&id));
    memcpy(id128, &id, 128);
    return DB2_OK;
}

int db2_comm_init(db2_context *ctx, int rank, int world, const void *id128) {
    DB2_CHECK(ctx && id128, DB2_EINVAL, "null argument");
    DB2_CHECK(world >= 1 && rank >= 0 && rank < world, DB2_EINVAL, "bad rank %d of %d", rank, world);
    DB2_CHECK(ctx->comm == nullptr, DB2_EINVAL, "context already has a communicator");
    ctx->rank = rank;
    ctx->world = world;
    if (world == 1)
        return DB2_OK;
    Nccl *n = nccl();
    DB2_CHECK(n, DB2_ENCCL, "NCCL library (libnccl.so.2) could not be loaded");
    bind_device(ctx);
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    ncclComm_t c = nullptr;
    DB2_NCCL(n->CommInitRank(&c, world, id, rank));
    ctx->comm = c;
    return DB2_OK;
}

int db2_comm_destroy(db2_context *ctx) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    if (ctx->comm) {
        bind_device(ctx);
        cudaStreamSynchronize(ctx->stream);
        nccl()->CommDestroy(static_cast<ncclComm_t>(ctx->comm));
        ctx->comm = nullptr;
    }
    ctx->world = 1;
    ctx->rank = 0;
    return DB2_OK;
}

int db2_comm_info(const db2_context *ctx, int *rank, int *world) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    if (rank)
        *rank = ctx->rank;
    if (world)
        *world = ctx->world;
    return DB2_OK;
}

// In-place combine of a (small, contiguous) device-resident partial over all ranks; combine = VectorCombine code.
int db2_allreduce(db2_context *ctx, db2_matrix *m, int combine) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && m, DB2_EINVAL, "null argument");
    DB2_CHECK(combine == DB2_COMBINE_ADD || combine == DB2_COMBINE_MIN || combine == DB2_COMBINE_MAX, DB2_EINVAL,
              "only ADD, MIN and MAX results are combined across row shards");
    if (ctx->world == 1)
        return DB2_OK;
    DB2_CHECK(ctx->comm, DB2_ENCCL, "no communicator: call db2_comm_init first");
    bind_device(ctx);
    DB2_TRY(ensure_device(m));
    DB2_CHECK(m->dev_ld == m->cols || m->rows == 1, DB2_EUNSUPPORTED, "all-reduce of a strided view");
    const int op = combine == DB2_COMBINE_ADD ? ncclSum : (combine == DB2_COMBINE_MIN ? ncclMin : ncclMax);
    DB2_NCCL(nccl()->AllReduce(m->dev_ptr(), m->dev_ptr(), (size_t)m->rows * m->cols, nccl_dtype(m->dtype), op,
                               static_cast<ncclComm_t>(ctx->comm), ctx->stream));
    m->host_valid = false;
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.collectives++;
    ctx->stats.collective_bytes += (uint64_t)m->rows * m->cols * m->esize();
    return DB2_OK;
    DB2_API_END
}

// Concatenates the equally shaped row shards of all ranks in rank order (ROWS combine across GPUs).
int db2_allgather_rows(db2_context *ctx, db2_matrix *local, db2_matrix **full) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && local && full, DB2_EINVAL, "null argument");
    bind_device(ctx);
    DB2_TRY(ensure_device(local));
    DB2_CHECK(local->dev_ld == local->cols || local->rows <= 1, DB2_EUNSUPPORTED, "all-gather of a strided view");
    DB2_TRY(prepare_result(ctx, full, local->dtype, local->rows * ctx->world, local->cols));
    db2_matrix *f = *full;
    const size_t n = (size_t)local->rows * local->cols;
    if (ctx->world == 1) {
        DB2_CUDA(cudaMemcpyAsync(f->dev_ptr(), local->dev_ptr(), n * local->esize(), cudaMemcpyDeviceToDevice,
                                 ctx->stream));
        return DB2_OK;
    }
    DB2_CHECK(ctx->comm, DB2_ENCCL, "no communicator: call db2_comm_init first");
    DB2_NCCL(nccl()->AllGather(local->dev_ptr(), f->dev_ptr(), n, nccl_dtype(local->dtype),
                               static_cast<ncclComm_t>(ctx->comm), ctx->stream));
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.collectives++;
    ctx->stats.collective_bytes += (uint64_t)n * local->esize() * ctx->world;
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
