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
    int (*Broadcast)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
};

// Test hook (host-side failure injection): a table installed with db2_comm_test_override replaces the loaded library,
// so that the error paths of the collectives can be exercised without a second GPU and without faulting one.
static Nccl *g_override = nullptr;

static Nccl *nccl() {
    if (g_override)
        return g_override;
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
        n.Broadcast = reinterpret_cast<decltype(n.Broadcast)>(dlsym(n.handle, "ncclBroadcast"));
        n.CommInitAll = reinterpret_cast<decltype(n.CommInitAll)>(dlsym(n.handle, "ncclCommInitAll"));
        n.GroupStart = reinterpret_cast<decltype(n.GroupStart)>(dlsym(n.handle, "ncclGroupStart"));
        n.GroupEnd = reinterpret_cast<decltype(n.GroupEnd)>(dlsym(n.handle, "ncclGroupEnd"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(dlsym(n.handle, "ncclGetErrorString"));
    });
    const bool ok = n.handle && n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.AllReduce && n.AllGather &&
                    n.Broadcast && n.CommInitAll && n.GroupStart && n.GroupEnd;
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

// ---- one process, several devices (group.cu) ----

// One communicator per context of a device group (ncclCommInitAll); the devices must be distinct.
int nccl_init_group(const std::vector<db2_context *> &ctxs) {
    Nccl *n = nccl();
    DB2_CHECK(n, DB2_ENCCL, "NCCL library (libnccl.so.2) could not be loaded");
    std::vector<int> devs;
    for (db2_context *c : ctxs)
        devs.push_back(c->device);
    std::vector<ncclComm_t> comms(ctxs.size(), nullptr);
    DB2_NCCL(n->CommInitAll(comms.data(), (int)ctxs.size(), devs.data()));
    for (size_t i = 0; i < ctxs.size(); i++)
        ctxs[i]->group_comm = comms[i];
    return DB2_OK;
}

void nccl_destroy_group(const std::vector<db2_context *> &ctxs) {
    Nccl *n = nccl();
    for (db2_context *c : ctxs)
        if (c->group_comm) {
            bind_device(c);
            cudaStreamSynchronize(c->stream);
            if (n)
                n->CommDestroy(static_cast<ncclComm_t>(c->group_comm));
            c->group_comm = nullptr;
        }
}

// In-place all-reduce of ms[d] (one equally shaped, contiguous, device-resident partial per context) on every
// context's own stream, issued by the calling thread as one NCCL group.
int nccl_allreduce_group(const std::vector<db2_context *> &ctxs, const std::vector<db2_matrix *> &ms, int combine) {
    Nccl *n = nccl();
    DB2_CHECK(n, DB2_ENCCL, "NCCL library (libnccl.so.2) could not be loaded");
    const int op = combine == DB2_COMBINE_ADD ? ncclSum : (combine == DB2_COMBINE_MIN ? ncclMin : ncclMax);
    DB2_NCCL(n->GroupStart());
    int rc = ncclSuccess;
    for (size_t d = 0; d < ctxs.size() && rc == ncclSuccess; d++) {
        bind_device(ctxs[d]);
        rc = n->AllReduce(ms[d]->dev_ptr(), ms[d]->dev_ptr(), (size_t)ms[d]->rows * ms[d]->cols,
                          nccl_dtype(ms[d]->dtype), op, static_cast<ncclComm_t>(ctxs[d]->group_comm), ctxs[d]->stream);
    }
    const int rc_end = n->GroupEnd();
    if (rc == ncclSuccess)
        rc = rc_end;
    if (rc != ncclSuccess)
        return set_error(DB2_ENCCL, "ncclAllReduce over the device group failed: %s",
                         n->GetErrorString ? n->GetErrorString(rc) : "NCCL error");
    for (size_t d = 0; d < ctxs.size(); d++) {
        ms[d]->host_valid = false;
        std::lock_guard<std::mutex> lock(ctxs[d]->mu);
        ctxs[d]->stats.collectives++;
        ctxs[d]->stats.collective_bytes += (uint64_t)ms[d]->rows * ms[d]->cols * ms[d]->esize();
    }
    return DB2_OK;
}

int comm_allgather_f64(db2_context *ctx, const double *send, double *recv, size_t count) {
    Nccl *n = nccl();
    DB2_CHECK(n && ctx->comm, DB2_ENCCL, "no communicator: call db2_comm_init first");
    DB2_NCCL(n->AllGather(send, recv, count, ncclFloat64, static_cast<ncclComm_t>(ctx->comm), ctx->stream));
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.collectives++;
    ctx->stats.collective_bytes += (uint64_t)count * 8 * ctx->world;
    return DB2_OK;
}

// rows of rank r when n rows are cut into `world` contiguous blocks (the first n % world blocks hold one more row)
static void row_block(int64_t n, int r, int world, int64_t *lo, int64_t *hi) {
    const int64_t base = n / world, extra = n % world;
    *lo = r * base + (r < extra ? r : extra);
    *hi = *lo + base + (r < extra ? 1 : 0);
}

} // namespace db2

using namespace db2;

extern "C" {

// Test hook, not part of the public interface: installs (or with NULL removes) a table of stand-in NCCL entry points.
// Layout: {AllReduce, AllGather, Broadcast, GroupStart, GroupEnd} as function pointers with NCCL's signatures.
int db2_comm_test_override(void **fns) {
    static Nccl fake;
    if (!fns) {
        g_override = nullptr;
        return DB2_OK;
    }
    fake = Nccl();
    fake.handle = reinterpret_cast<void *>(1);
    fake.AllReduce = reinterpret_cast<decltype(fake.AllReduce)>(fns[0]);
    fake.AllGather = reinterpret_cast<decltype(fake.AllGather)>(fns[1]);
    fake.Broadcast = reinterpret_cast<decltype(fake.Broadcast)>(fns[2]);
    fake.GroupStart = reinterpret_cast<decltype(fake.GroupStart)>(fns[3]);
    fake.GroupEnd = reinterpret_cast<decltype(fake.GroupEnd)>(fns[4]);
    g_override = &fake;
    return DB2_OK;
}
// Test hook: marks a context as rank `rank` of `world` with a stand-in communicator (no NCCL call is made).
int db2_comm_test_attach(db2_context *ctx, int rank, int world) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    ctx->rank = rank;
    ctx->world = world;
    ctx->comm = world > 1 ? reinterpret_cast<void *>(1) : nullptr;
    ctx->comm_is_fake = world > 1;
    return DB2_OK;
}

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
        if (!ctx->comm_is_fake && nccl() && nccl()->CommDestroy)
            nccl()->CommDestroy(static_cast<ncclComm_t>(ctx->comm));
        ctx->comm = nullptr;
        ctx->comm_is_fake = false;
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

// Collectives issued between begin and end are handed to NCCL as one group: it launches them together, so a count
// all-reduce and the all-gather that follows it cost one launch on the stream instead of two.
int db2_comm_group_begin(db2_context *ctx) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    if (ctx->world == 1 || !ctx->comm)
        return DB2_OK;
    Nccl *n = nccl();
    DB2_CHECK(n, DB2_ENCCL, "NCCL library (libnccl.so.2) could not be loaded");
    DB2_NCCL(n->GroupStart());
    return DB2_OK;
}
int db2_comm_group_end(db2_context *ctx) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    if (ctx->world == 1 || !ctx->comm)
        return DB2_OK;
    Nccl *n = nccl();
    DB2_CHECK(n, DB2_ENCCL, "NCCL library (libnccl.so.2) could not be loaded");
    DB2_NCCL(n->GroupEnd());
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
    if (m->combined) { // answered from exchanged statistics: already the value over all shards
        m->combined = false;
        return DB2_OK;
    }
    DB2_CHECK(ctx->comm, DB2_ENCCL, "no communicator: call db2_comm_init first");
    bind_device(ctx);
    DB2_TRY(ensure_device(m));
    DB2_CHECK(m->dev_ld == m->cols || m->rows == 1, DB2_EUNSUPPORTED, "all-reduce of a strided view");
    if (combine == DB2_COMBINE_ADD) {
        bool handled = false;
        DB2_TRY(colstats_try_allreduce(ctx, m, &handled));
        if (handled)
            return DB2_OK;
    }
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

// The same combine, issued on a stream of its own behind what the context's stream has queued so far: the context's
// stream goes on at once, and whoever touches m next waits for the combine (DevBuf::ready).  For a partial that
// nothing on the device needs soon -- the final scalar of a pipeline -- the collective's latency is no longer part
// of the pipeline's step.
int db2_allreduce_async(db2_context *ctx, db2_matrix *m, int combine) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && m, DB2_EINVAL, "null argument");
    DB2_CHECK(combine == DB2_COMBINE_ADD || combine == DB2_COMBINE_MIN || combine == DB2_COMBINE_MAX, DB2_EINVAL,
              "only ADD, MIN and MAX results are combined across row shards");
    if (ctx->world == 1)
        return DB2_OK;
    if (m->combined || g_override) // nothing to do / the test table of stand-ins: the plain path
        return db2_allreduce(ctx, m, combine);
    DB2_CHECK(ctx->comm, DB2_ENCCL, "no communicator: call db2_comm_init first");
    bind_device(ctx);
    DB2_TRY(ensure_device(m));
    DB2_CHECK(m->dev_ld == m->cols || m->rows == 1, DB2_EUNSUPPORTED, "all-reduce of a strided view");
    if (!ctx->side_stream)
        DB2_CUDA(cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
    cudaEvent_t queued = nullptr, done = nullptr;
    DB2_CUDA(cudaEventCreateWithFlags(&queued, cudaEventDisableTiming));
    DB2_CUDA(cudaEventRecord(queued, ctx->stream));
    DB2_CUDA(cudaStreamWaitEvent(ctx->side_stream, queued, 0));
    DB2_CUDA(cudaEventDestroy(queued));
    const int op = combine == DB2_COMBINE_ADD ? ncclSum : (combine == DB2_COMBINE_MIN ? ncclMin : ncclMax);
    DB2_NCCL(nccl()->AllReduce(m->dev_ptr(), m->dev_ptr(), (size_t)m->rows * m->cols, nccl_dtype(m->dtype), op,
                               static_cast<ncclComm_t>(ctx->comm), ctx->side_stream));
    DB2_CUDA(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    DB2_CUDA(cudaEventRecord(done, ctx->side_stream));
    m->dev->ready = done;
    m->host_valid = false;
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.collectives++;
    ctx->stats.collective_bytes += (uint64_t)m->rows * m->cols * m->esize();
    return DB2_OK;
    DB2_API_END
}

// Concatenates the row shards of all ranks in rank order (ROWS combine across GPUs).  The shards follow the row
// partition of the scheduler: `total_rows` rows cut into `world` contiguous blocks, the first total_rows % world of
// them one row taller.  Every rank can compute every block from total_rows, so no sizes are exchanged; a shard whose
// height is not its block's is refused before any collective is issued (ranks that call with different counts would
// otherwise wait for one another or overrun the receive buffer).  Equal blocks take one ncclAllGather, ragged ones one
// ncclBroadcast per rank inside a group.
int db2_allgatherv_rows(db2_context *ctx, db2_matrix *local, int64_t total_rows, db2_matrix **full) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && local && full, DB2_EINVAL, "null argument");
    int64_t lo = 0, hi = 0;
    row_block(total_rows, ctx->rank, ctx->world, &lo, &hi);
    DB2_CHECK(total_rows >= 0 && local->rows == hi - lo, DB2_EINVAL,
              "all-gather of row shards: rank %d of %d holds %lld rows, its block of %lld rows has %lld", ctx->rank,
              ctx->world, (long long)local->rows, (long long)total_rows, (long long)(hi - lo));
    bind_device(ctx);
    DB2_TRY(ensure_device(local));
    DB2_CHECK(local->dev_ld == local->cols || local->rows <= 1, DB2_EUNSUPPORTED, "all-gather of a strided view");
    DB2_TRY(prepare_result(ctx, full, local->dtype, total_rows, local->cols));
    db2_matrix *f = *full;
    const size_t es = local->esize(), n = (size_t)local->rows * local->cols;
    if (ctx->world == 1) {
        DB2_CUDA(cudaMemcpyAsync(f->dev_ptr(), local->dev_ptr(), n * es, cudaMemcpyDeviceToDevice, ctx->stream));
        return DB2_OK;
    }
    DB2_CHECK(ctx->comm, DB2_ENCCL, "no communicator: call db2_comm_init first");
    Nccl *nc = nccl();
    DB2_CHECK(nc, DB2_ENCCL, "NCCL library (libnccl.so.2) could not be loaded");
    ncclComm_t comm = static_cast<ncclComm_t>(ctx->comm);
    if (total_rows % ctx->world == 0) {
        DB2_NCCL(nc->AllGather(local->dev_ptr(), f->dev_ptr(), n, nccl_dtype(local->dtype), comm, ctx->stream));
    } else {
        DB2_NCCL(nc->GroupStart());
        int rc = ncclSuccess;
        for (int r = 0; r < ctx->world && rc == ncclSuccess; r++) {
            int64_t a = 0, b = 0;
            row_block(total_rows, r, ctx->world, &a, &b);
            char *dst = static_cast<char *>(f->dev_ptr()) + (size_t)a * f->dev_ld * es;
            rc = nc->Broadcast(r == ctx->rank ? local->dev_ptr() : dst, dst, (size_t)(b - a) * local->cols,
                               nccl_dtype(local->dtype), r, comm, ctx->stream);
        }
        const int rc_end = nc->GroupEnd();
        if (rc == ncclSuccess)
            rc = rc_end;
        if (rc != ncclSuccess)
            return set_error(DB2_ENCCL, "ragged all-gather failed: %s",
                             nc->GetErrorString ? nc->GetErrorString(rc) : "NCCL error");
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.collectives++;
    ctx->stats.collective_bytes += (uint64_t)total_rows * local->cols * es;
    return DB2_OK;
    DB2_API_END
}

// Equally tall shards (every rank holds local->rows rows).
int db2_allgather_rows(db2_context *ctx, db2_matrix *local, db2_matrix **full) {
    DB2_CHECK(ctx && local && full, DB2_EINVAL, "null argument");
    return db2_allgatherv_rows(ctx, local, local->rows * ctx->world, full);
}

} // extern "C"
