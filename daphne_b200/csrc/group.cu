// Several GPUs in ONE process: device groups, row-distributed matrices and the scheduler that splits the row range of a
// compiled pipeline over the devices of a group.
//
// The reference's scheduler has the shape for this -- one WorkerGPU thread per entry of ctx->cuda_contexts
// (src/runtime/local/vectorized/MTWrapper.h:93-98,170-174), one task per device block
// (vectorized/MTWrapper_dense.cpp:204-336) -- but creates a single context and hard-codes device 0
// ("ToDo: multi-device support", MTWrapper_dense.cpp:220, vectorized/TasksCUDA.cpp:72).  Here:
//   * a db2_group owns one context (stream, pooled memory) per device and, when the devices are distinct, one NCCL
//     communicator per device (ncclCommInitAll);
//   * a db2_dist is a matrix whose rows (or columns) are cut into one contiguous block per device, or that is
//     replicated on every device.  A host matrix becomes a db2_dist without moving a byte: every shard wraps its rows
//     of the host buffer and the owning device fetches them on first use, so the uploads of all devices overlap;
//   * db2_vectorizedPipelineGroup runs the single-device scheduler (pipeline.cu) on every device's block from one
//     host thread per device, leaves ROWS / COLS results distributed (gathered only on request) and combines
//     ADD / MIN / MAX partials over the devices: one grouped ncclAllReduce per result over NVLink, or -- without
//     NCCL, or when several contexts of the group share a physical device (then NCCL's kernels would wait for one
//     another on one GPU) -- by copying every partial to every device and folding them there in device order with the
//     elementwise kernel, which gives bit-identical results on all devices.  No multicast loads of any kind.
#include "runtime.h"

#include <condition_variable>
#include <cstdlib>
#include <functional>
#include <string>
#include <thread>

using namespace db2;

typedef void (*db2_pipeline_fn)(db2_matrix ***outputs, db2_matrix **inputs, db2_context *ctx);

struct db2_group {
    std::vector<db2_context *> ctxs;
    bool distinct = true; // every context on its own physical device
    bool nccl = false;    // the contexts hold communicators made by ncclCommInitAll
    std::atomic<int> refs{1};
    // one host thread per device, like the reference's WorkerGPU per CUDA context (vectorized/MTWrapper.h:93-98), kept
    // for the lifetime of the group: a pipeline hands them its per-device task and waits (creating threads per
    // pipeline cost more than the kernels of a small one)
    std::vector<std::thread> workers;
    std::mutex mu;
    std::condition_variable cv_work, cv_done;
    std::function<void(int)> task;
    uint64_t generation = 0;
    int running = 0;
    bool stop = false;
    std::mutex call_mu; // one pipeline at a time per group
};

struct db2_dist {
    std::atomic<int> refs{1};
    db2_group *g = nullptr;
    int axis = 0; // 0: row blocks, 1: column blocks, -1: replicated
    int dtype = DB2_F64;
    int64_t rows = 0, cols = 0;
    std::vector<db2_matrix *> shard; // one per device; owned
    std::vector<int64_t> off;        // ndev + 1 offsets along `axis` (unused when replicated)
};

namespace {

void block_of(int64_t n, int r, int world, int64_t *lo, int64_t *hi) {
    const int64_t base = n / world, extra = n % world;
    *lo = r * base + (r < extra ? r : extra);
    *hi = *lo + base + (r < extra ? 1 : 0);
}

void worker_loop(db2_group *g, int d) {
    bind_device(g->ctxs[d]);
    uint64_t seen = 0;
    for (;;) {
        std::function<void(int)> f;
        {
            std::unique_lock<std::mutex> lock(g->mu);
            g->cv_work.wait(lock, [&] { return g->stop || g->generation != seen; });
            if (g->stop)
                return;
            seen = g->generation;
            f = g->task;
        }
        f(d);
        {
            std::lock_guard<std::mutex> lock(g->mu);
            if (--g->running == 0)
                g->cv_done.notify_all();
        }
    }
}

void group_release(db2_group *g) {
    if (g->refs.fetch_sub(1) != 1)
        return;
    {
        std::lock_guard<std::mutex> lock(g->mu);
        g->stop = true;
    }
    g->cv_work.notify_all();
    for (auto &w : g->workers)
        w.join();
    if (g->nccl)
        nccl_destroy_group(g->ctxs);
    for (db2_context *c : g->ctxs)
        db2_context_destroy(c);
    delete g;
}

db2_dist *new_dist(db2_group *g, int axis, int dtype, int64_t rows, int64_t cols) {
    db2_dist *d = new db2_dist();
    d->g = g;
    g->refs.fetch_add(1);
    d->axis = axis;
    d->dtype = dtype;
    d->rows = rows;
    d->cols = cols;
    d->shard.assign(g->ctxs.size(), nullptr);
    d->off.assign(g->ctxs.size() + 1, 0);
    return d;
}

// runs f(d) for every device index on its own host thread (device d bound); the first failure wins and its message is
// handed to the calling thread
template <typename F> int for_each_device(db2_group *g, F &&f) {
    const int n = (int)g->ctxs.size();
    std::vector<int> rc(n, DB2_OK);
    std::vector<std::string> msg(n);
    auto run = [&](int d) {
        bind_device(g->ctxs[d]);
        rc[d] = f(d);
        if (rc[d] != DB2_OK)
            msg[d] = err_buf();
    };
    if (n == 1) {
        run(0);
    } else {
        std::lock_guard<std::mutex> one(g->call_mu);
        std::unique_lock<std::mutex> lock(g->mu);
        if (g->workers.empty())
            for (int d = 0; d < n; d++)
                g->workers.emplace_back(worker_loop, g, d);
        g->task = run;
        g->running = n;
        g->generation++;
        g->cv_work.notify_all();
        g->cv_done.wait(lock, [&] { return g->running == 0; });
        g->task = nullptr;
    }
    for (int d = 0; d < n; d++)
        if (rc[d] != DB2_OK)
            return set_error(rc[d], "device %d of the group: %s", g->ctxs[d]->device, msg[d].c_str());
    return DB2_OK;
}

// copy of src (any context of this process) as a new matrix of ctx: plain device-to-device copy, peer copy over
// NVLink when the devices differ; ordered after everything already issued on src's stream
int copy_to_context(db2_context *ctx, db2_matrix *src, db2_matrix **out) {
    DB2_TRY(ensure_device(src));
    bind_device(src->ctx);
    cudaEvent_t ev;
    DB2_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    DB2_CUDA(cudaEventRecord(ev, src->ctx->stream));
    bind_device(ctx);
    DB2_TRY(db2_matrix_create(ctx, src->dtype, src->rows, src->cols, 0, out));
    db2_matrix *m = *out;
    DB2_CUDA(cudaStreamWaitEvent(ctx->stream, ev, 0));
    const size_t es = src->esize();
    if (src->rows * src->cols > 0) {
        if (src->dev_ld == src->cols || src->rows == 1) {
            DB2_CUDA(cudaMemcpyPeerAsync(m->dev_ptr(), ctx->device, src->dev_ptr(), src->ctx->device,
                                         (size_t)src->rows * src->cols * es, ctx->stream));
        } else {
            cudaMemcpy3DPeerParms p = {};
            p.srcDevice = src->ctx->device;
            p.dstDevice = ctx->device;
            p.srcPtr = make_cudaPitchedPtr(src->dev_ptr(), (size_t)src->dev_ld * es, (size_t)src->cols * es,
                                           (size_t)src->rows);
            p.dstPtr = make_cudaPitchedPtr(m->dev_ptr(), (size_t)m->dev_ld * es, (size_t)m->cols * es, (size_t)m->rows);
            p.extent = make_cudaExtent((size_t)src->cols * es, (size_t)src->rows, 1);
            DB2_CUDA(cudaMemcpy3DPeerAsync(&p, ctx->stream));
        }
        // the source buffer may be released (and reused) by its own context as soon as this call returns: make the
        // source stream wait for the copy
        cudaEvent_t done;
        DB2_CUDA(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
        DB2_CUDA(cudaEventRecord(done, ctx->stream));
        bind_device(src->ctx);
        DB2_CUDA(cudaStreamWaitEvent(src->ctx->stream, done, 0));
        DB2_CUDA(cudaEventDestroy(done));
        bind_device(ctx);
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.d2d_bytes += (uint64_t)src->rows * src->cols * es;
    }
    DB2_CUDA(cudaEventDestroy(ev));
    return DB2_OK;
}

// Combines the equally shaped partials parts[d] (one per device of the group, device-resident) with ADD / MIN / MAX.
// out[d] receives the combined matrix of device d (a new reference: either the partial itself, combined in place by
// NCCL, or a new matrix folded from copies of all partials in device order); consumed partials are set to NULL in
// `slots` (the caller releases what is left).
int combine_partials(db2_group *g, std::vector<std::vector<db2_matrix *>> &slots, size_t o, int cmb,
                     std::vector<db2_matrix *> &out) {
    const int n = (int)g->ctxs.size();
    std::vector<db2_matrix *> parts(n);
    db2_matrix *r0 = slots[0][o];
    for (int d = 0; d < n; d++) {
        parts[d] = slots[d][o];
        DB2_CHECK(parts[d], DB2_EINVAL, "missing partial result on device index %d", d);
        bind_device(g->ctxs[d]);
        DB2_TRY(ensure_device(parts[d]));
        DB2_CHECK(parts[d]->dev_ld == parts[d]->cols || parts[d]->rows == 1, DB2_EUNSUPPORTED,
                  "a partial result is a strided view");
        DB2_CHECK(parts[d]->rows == r0->rows && parts[d]->cols == r0->cols && parts[d]->dtype == r0->dtype, DB2_EINVAL,
                  "a partial result has different shapes on different devices");
    }
    if (n == 1 || g->nccl) {
        if (n > 1)
            DB2_TRY(nccl_allreduce_group(g->ctxs, parts, cmb));
        for (int d = 0; d < n; d++) {
            out[d] = parts[d];
            slots[d][o] = nullptr;
        }
        return DB2_OK;
    }
    // peer copies + fold, in device order on every device
    const int op = cmb == DB2_COMBINE_ADD ? DB2_ADD : (cmb == DB2_COMBINE_MIN ? DB2_MIN : DB2_MAX);
    for (int d = 0; d < n; d++) {
        db2_context *c = g->ctxs[d];
        db2_matrix *acc = nullptr;
        for (int e = 0; e < n; e++) {
            db2_matrix *pe = nullptr;
            int rc = copy_to_context(c, parts[e], &pe);
            bind_device(c);
            if (rc == DB2_OK && acc) {
                rc = db2_ewBinaryMat(c, op, &acc, acc, pe);
                db2_matrix_decref(pe);
            } else if (rc == DB2_OK) {
                acc = pe;
            }
            if (rc != DB2_OK) {
                if (acc)
                    db2_matrix_decref(acc);
                return rc;
            }
        }
        out[d] = acc;
        std::lock_guard<std::mutex> lock(c->mu);
        c->stats.collectives++;
        c->stats.collective_bytes += (uint64_t)r0->rows * r0->cols * dtype_size(r0->dtype) * (n - 1);
    }
    return DB2_OK;
}

} // namespace

extern "C" {

int db2_group_create(const int *devices, int ndev, db2_group **out) {
    DB2_API_BEGIN
    DB2_CHECK(out, DB2_EINVAL, "null group slot");
    *out = nullptr;
    std::vector<int> devs;
    if (devices && ndev > 0) {
        devs.assign(devices, devices + ndev);
    } else {
        const char *env = getenv("DAPHNE_B200_DEVICES");
        if (env && *env && std::string(env) != "all") {
            const char *p = env;
            while (*p) {
                char *end = nullptr;
                const long v = strtol(p, &end, 10);
                DB2_CHECK(end != p, DB2_EINVAL, "DAPHNE_B200_DEVICES=\"%s\" is not a comma-separated device list", env);
                devs.push_back((int)v);
                p = (*end == ',') ? end + 1 : end;
                DB2_CHECK(*end == ',' || *end == 0, DB2_EINVAL,
                          "DAPHNE_B200_DEVICES=\"%s\" is not a comma-separated device list", env);
            }
        } else {
            int n = 0;
            DB2_TRY(db2_device_count(&n));
            for (int d = 0; d < n; d++)
                devs.push_back(d);
        }
    }
    DB2_CHECK(!devs.empty() && devs.size() <= 64, DB2_EINVAL, "a device group needs 1 to 64 devices");
    std::unique_ptr<db2_group, void (*)(db2_group *)> g(new db2_group(), group_release);
    for (size_t i = 0; i < devs.size(); i++) {
        db2_context *c = nullptr;
        DB2_TRY(db2_context_create(devs[i], &c));
        g->ctxs.push_back(c);
        for (size_t j = 0; j < i; j++)
            if (devs[j] == devs[i]) {
                g->distinct = false;
                c->dup++;
            }
    }
    // peer access between all pairs (NVLink through NVSwitch): copies between devices then go directly
    if (g->distinct && devs.size() > 1) {
        for (size_t i = 0; i < devs.size(); i++) {
            DB2_CUDA(cudaSetDevice(devs[i]));
            for (size_t j = 0; j < devs.size(); j++) {
                if (i == j)
                    continue;
                int can = 0;
                DB2_CUDA(cudaDeviceCanAccessPeer(&can, devs[i], devs[j]));
                if (can) {
                    cudaError_t e = cudaDeviceEnablePeerAccess(devs[j], 0);
                    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                        DB2_CUDA(e);
                    cudaGetLastError();
                }
            }
        }
        const char *no = getenv("DAPHNE_B200_NO_NCCL");
        if (!(no && no[0] == '1') && nccl_init_group(g->ctxs) == DB2_OK)
            g->nccl = true; // otherwise: partials are combined with peer copies and the fold kernel
    }
    *out = g.release();
    return DB2_OK;
    DB2_API_END
}

int db2_group_destroy(db2_group *g) {
    if (!g)
        return DB2_OK;
    for (db2_context *c : g->ctxs) {
        bind_device(c);
        cudaStreamSynchronize(c->stream);
    }
    group_release(g);
    return DB2_OK;
}

int db2_group_size(const db2_group *g, int *n) {
    DB2_CHECK(g && n, DB2_EINVAL, "null argument");
    *n = (int)g->ctxs.size();
    return DB2_OK;
}

int db2_group_context(db2_group *g, int i, db2_context **ctx) {
    DB2_CHECK(g && ctx, DB2_EINVAL, "null argument");
    DB2_CHECK(i >= 0 && i < (int)g->ctxs.size(), DB2_EINVAL, "device index %d outside the group of %zu", i,
              g->ctxs.size());
    *ctx = g->ctxs[i];
    return DB2_OK;
}

/* 1 when partials are combined by NCCL, 0 when by peer copies and the fold kernel */
int db2_group_uses_nccl(const db2_group *g, int *yes) {
    DB2_CHECK(g && yes, DB2_EINVAL, "null argument");
    *yes = g->nccl ? 1 : 0;
    return DB2_OK;
}

int db2_group_sync(db2_group *g) {
    DB2_API_BEGIN
    DB2_CHECK(g, DB2_EINVAL, "null group");
    for (db2_context *c : g->ctxs)
        DB2_TRY(db2_context_sync(c));
    return DB2_OK;
    DB2_API_END
}

int db2_dist_from_host(db2_group *g, int dtype, int64_t rows, int64_t cols, int64_t ld, void *host, db2_dist **out) {
    DB2_API_BEGIN
    DB2_CHECK(g && out, DB2_EINVAL, "null argument");
    DB2_CHECK(rows >= 0 && cols >= 0 && ld >= cols, DB2_EINVAL, "bad shape (%lld x %lld, ld %lld)", (long long)rows,
              (long long)cols, (long long)ld);
    std::unique_ptr<db2_dist, int (*)(db2_dist *)> d(new_dist(g, 0, dtype, rows, cols), db2_dist_decref);
    const int n = (int)g->ctxs.size();
    const size_t es = dtype_size(dtype);
    for (int i = 0; i < n; i++) {
        int64_t lo, hi;
        block_of(rows, i, n, &lo, &hi);
        d->off[i] = lo;
        d->off[i + 1] = hi;
        DB2_TRY(db2_matrix_wrap_host(g->ctxs[i], dtype, hi - lo, cols, ld,
                                     static_cast<char *>(host) + (size_t)lo * ld * es, &d->shard[i]));
    }
    *out = d.release();
    return DB2_OK;
    DB2_API_END
}

int db2_dist_from_matrix(db2_group *g, db2_matrix *m, int replicate, db2_dist **out) {
    DB2_API_BEGIN
    DB2_CHECK(g && m && out, DB2_EINVAL, "null argument");
    const int n = (int)g->ctxs.size();
    std::unique_ptr<db2_dist, int (*)(db2_dist *)> d(new_dist(g, replicate ? -1 : 0, m->dtype, m->rows, m->cols),
                                                     db2_dist_decref);
    // a matrix whose latest values are on the host is cut there (no device of the group is a detour for the others)
    const bool from_host = !m->dev_valid && !m->deferred() && m->host_valid;
    for (int i = 0; i < n; i++) {
        int64_t lo = 0, hi = m->rows;
        if (!replicate)
            block_of(m->rows, i, n, &lo, &hi);
        d->off[i] = lo;
        d->off[i + 1] = hi;
        db2_context *c = g->ctxs[i];
        if (from_host) {
            DB2_TRY(db2_matrix_wrap_host(c, m->dtype, hi - lo, m->cols, m->host_ld,
                                         static_cast<char *>(m->host_ptr()) + (size_t)lo * m->host_ld * m->esize(),
                                         &d->shard[i]));
            d->shard[i]->host = m->host; // shares (and keeps alive) the parent's host buffer
            d->shard[i]->host_off = m->host_off + lo * m->host_ld;
            continue;
        }
        db2_matrix *view = nullptr;
        DB2_TRY(db2_matrix_slice_rows(m, lo, hi, &view));
        if (m->ctx == c) {
            d->shard[i] = view;
        } else {
            const int rc = copy_to_context(c, view, &d->shard[i]);
            db2_matrix_decref(view);
            DB2_TRY(rc);
        }
    }
    *out = d.release();
    return DB2_OK;
    DB2_API_END
}

/* a distributed matrix from one matrix per device (shards[i] lives on device i; references are taken): row blocks
 * (axis 0), column blocks (axis 1) or copies of one matrix (axis -1) */
int db2_dist_from_shards(db2_group *g, db2_matrix **shards, int axis, db2_dist **out) {
    DB2_API_BEGIN
    DB2_CHECK(g && shards && out, DB2_EINVAL, "null argument");
    DB2_CHECK(axis >= -1 && axis <= 1, DB2_EINVAL, "axis must be -1, 0 or 1");
    const int n = (int)g->ctxs.size();
    int64_t rows = 0, cols = 0;
    for (int i = 0; i < n; i++) {
        DB2_CHECK(shards[i] && shards[i]->ctx == g->ctxs[i], DB2_EINVAL,
                  "shard %d does not live on device index %d of the group", i, i);
        DB2_CHECK(shards[i]->dtype == shards[0]->dtype, DB2_EINVAL, "shards of different value types");
        if (axis == 0) {
            DB2_CHECK(shards[i]->cols == shards[0]->cols, DB2_EINVAL, "row blocks of different widths");
            rows += shards[i]->rows;
            cols = shards[0]->cols;
        } else if (axis == 1) {
            DB2_CHECK(shards[i]->rows == shards[0]->rows, DB2_EINVAL, "column blocks of different heights");
            cols += shards[i]->cols;
            rows = shards[0]->rows;
        } else {
            DB2_CHECK(shards[i]->rows == shards[0]->rows && shards[i]->cols == shards[0]->cols, DB2_EINVAL,
                      "copies of different shapes");
            rows = shards[0]->rows;
            cols = shards[0]->cols;
        }
    }
    db2_dist *d = new_dist(g, axis, shards[0]->dtype, rows, cols);
    int64_t at = 0;
    for (int i = 0; i < n; i++) {
        db2_matrix_incref(shards[i]);
        d->shard[i] = shards[i];
        d->off[i] = at;
        at += axis == 0 ? shards[i]->rows : (axis == 1 ? shards[i]->cols : 0);
        d->off[i + 1] = at;
    }
    *out = d;
    return DB2_OK;
    DB2_API_END
}

int db2_dist_info(const db2_dist *d, int *dtype, int64_t *rows, int64_t *cols, int *axis) {
    DB2_CHECK(d, DB2_EINVAL, "null argument");
    if (dtype)
        *dtype = d->dtype;
    if (rows)
        *rows = d->rows;
    if (cols)
        *cols = d->cols;
    if (axis)
        *axis = d->axis;
    return DB2_OK;
}

int db2_dist_shard(db2_dist *d, int i, db2_matrix **shard, int64_t *offset) {
    DB2_CHECK(d && shard, DB2_EINVAL, "null argument");
    DB2_CHECK(i >= 0 && i < (int)d->shard.size(), DB2_EINVAL, "device index %d outside the group", i);
    *shard = d->shard[i];
    if (offset)
        *offset = d->axis < 0 ? 0 : d->off[i];
    return DB2_OK;
}

int db2_dist_incref(db2_dist *d) {
    DB2_CHECK(d, DB2_EINVAL, "null argument");
    d->refs.fetch_add(1);
    return DB2_OK;
}

int db2_dist_decref(db2_dist *d) {
    if (!d)
        return DB2_OK;
    if (d->refs.fetch_sub(1) == 1) {
        for (db2_matrix *s : d->shard)
            if (s) {
                bind_device(s->ctx);
                db2_matrix_decref(s);
            }
        group_release(d->g);
        delete d;
    }
    return DB2_OK;
}

/* every device copies its block straight into its rows (columns) of dst; a replicated matrix is read from device 0 */
int db2_dist_to_host(db2_dist *d, void *dst, int64_t dst_ld) {
    DB2_API_BEGIN
    DB2_CHECK(d && (dst || d->rows * d->cols == 0), DB2_EINVAL, "null argument");
    DB2_CHECK(dst_ld >= d->cols, DB2_EINVAL, "destination leading dimension too small");
    const size_t es = dtype_size(d->dtype);
    if (d->axis < 0) {
        bind_device(d->shard[0]->ctx);
        return db2_matrix_to_host(d->shard[0], dst, dst_ld);
    }
    return for_each_device(d->g, [&](int i) -> int {
        char *p = static_cast<char *>(dst) + (d->axis == 0 ? (size_t)d->off[i] * dst_ld : (size_t)d->off[i]) * es;
        return db2_matrix_to_host(d->shard[i], p, dst_ld);
    });
    DB2_API_END
}

/* one matrix on device `index` of the group: blocks of other devices arrive by peer copies */
int db2_dist_gather(db2_dist *d, int index, db2_matrix **out) {
    DB2_API_BEGIN
    DB2_CHECK(d && out, DB2_EINVAL, "null argument");
    DB2_CHECK(index >= 0 && index < (int)d->shard.size(), DB2_EINVAL, "device index %d outside the group", index);
    db2_context *ctx = d->g->ctxs[index];
    if (d->axis < 0) {
        *out = d->shard[index];
        return db2_matrix_incref(*out);
    }
    bind_device(ctx);
    db2_matrix *full = nullptr;
    DB2_TRY(db2_matrix_create(ctx, d->dtype, d->rows, d->cols, 0, &full));
    std::unique_ptr<db2_matrix, int (*)(db2_matrix *)> guard(full, db2_matrix_decref);
    const size_t es = dtype_size(d->dtype);
    for (size_t i = 0; i < d->shard.size(); i++) {
        db2_matrix *s = d->shard[i];
        if (s->rows * s->cols == 0)
            continue;
        bind_device(s->ctx);
        DB2_TRY(ensure_device(s));
        cudaEvent_t ev;
        DB2_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        DB2_CUDA(cudaEventRecord(ev, s->ctx->stream));
        bind_device(ctx);
        DB2_CUDA(cudaStreamWaitEvent(ctx->stream, ev, 0));
        DB2_CUDA(cudaEventDestroy(ev));
        char *dst = static_cast<char *>(full->dev_ptr()) +
                    (d->axis == 0 ? (size_t)d->off[i] * full->dev_ld : (size_t)d->off[i]) * es;
        cudaMemcpy3DPeerParms p = {};
        p.srcDevice = s->ctx->device;
        p.dstDevice = ctx->device;
        p.srcPtr = make_cudaPitchedPtr(s->dev_ptr(), (size_t)s->dev_ld * es, (size_t)s->cols * es, (size_t)s->rows);
        p.dstPtr = make_cudaPitchedPtr(dst, (size_t)full->dev_ld * es, (size_t)s->cols * es, (size_t)s->rows);
        p.extent = make_cudaExtent((size_t)s->cols * es, (size_t)s->rows, 1);
        DB2_CUDA(cudaMemcpy3DPeerAsync(&p, ctx->stream));
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.d2d_bytes += (uint64_t)s->rows * s->cols * es;
    }
    // the shards may be released by their owners right after this call: the gathered copy must be complete by then
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    *out = guard.release();
    return DB2_OK;
    DB2_API_END
}

int db2_vectorizedPipelineGroup(db2_group *g, db2_dist **outputs, size_t numOutputs, const int *isScalar,
                                db2_dist **inputs, size_t numInputs, const int64_t *outRows, const int64_t *outCols,
                                const int64_t *splits, const int64_t *combines, db2_pipeline_fn fun,
                                int64_t batch_rows) {
    DB2_API_BEGIN
    DB2_CHECK(g && outputs && fun && (inputs || numInputs == 0) && splits && combines, DB2_EINVAL, "null argument");
    const int n = (int)g->ctxs.size();
    // the ROWS inputs must share one row partition (the group's); broadcast inputs must be replicated
    const db2_dist *part = nullptr;
    for (size_t i = 0; i < numInputs; i++) {
        if (isScalar && isScalar[i])
            continue;
        const db2_dist *in = inputs[i];
        DB2_CHECK(in && in->g == g, DB2_EINVAL, "pipeline input %zu does not belong to this device group", i);
        const bool bcast = splits[i] == DB2_SPLIT_NONE || in->rows == 1;
        if (bcast) {
            DB2_CHECK(in->axis < 0, DB2_EINVAL, "pipeline input %zu is broadcast to every row block and must be "
                      "replicated on the devices", i);
            continue;
        }
        DB2_CHECK(splits[i] == DB2_SPLIT_ROWS, DB2_EINVAL, "unknown VectorSplit %lld", (long long)splits[i]);
        DB2_CHECK(in->axis == 0, DB2_EINVAL, "pipeline input %zu is split by rows and must be distributed by rows", i);
        if (!part)
            part = in;
        DB2_CHECK(in->off == part->off, DB2_EINVAL, "the row-split inputs of a pipeline must share one row partition");
    }
    for (size_t o = 0; o < numOutputs; o++) {
        DB2_CHECK(combines[o] >= DB2_COMBINE_ROWS && combines[o] <= DB2_COMBINE_MAX, DB2_EINVAL,
                  "unknown VectorCombine %lld", (long long)combines[o]);
        outputs[o] = nullptr;
    }
    DB2_CHECK(!part || part->rows >= n, DB2_EUNSUPPORTED,
              "%lld rows cannot be split over %d devices: use a smaller device group", part ? (long long)part->rows : 0,
              n);
    // per device: the single-device scheduler on that device's row block
    std::vector<std::vector<db2_matrix *>> res(n, std::vector<db2_matrix *>(numOutputs, nullptr));
    auto release_all = [&]() {
        for (int d = 0; d < n; d++)
            for (db2_matrix *m : res[d])
                if (m) {
                    bind_device(g->ctxs[d]);
                    db2_matrix_decref(m);
                }
    };
    int rc = for_each_device(g, [&](int d) -> int {
        std::vector<db2_matrix *> ins(numInputs);
        for (size_t i = 0; i < numInputs; i++)
            ins[i] = (isScalar && isScalar[i]) ? reinterpret_cast<db2_matrix *>(inputs[i]) : inputs[i]->shard[d];
        return db2_vectorizedPipeline(g->ctxs[d], res[d].data(), numOutputs, isScalar, ins.data(), numInputs, outRows,
                                      outCols, splits, combines, fun, batch_rows);
    });
    if (rc != DB2_OK) {
        release_all();
        return rc;
    }
    std::vector<std::unique_ptr<db2_dist, int (*)(db2_dist *)>> outs;
    for (size_t o = 0; o < numOutputs; o++) {
        db2_matrix *r0 = res[0][o];
        const int64_t cmb = combines[o];
        if (cmb == DB2_COMBINE_ROWS || cmb == DB2_COMBINE_COLS) {
            const int axis = cmb == DB2_COMBINE_ROWS ? 0 : 1;
            int64_t total = 0;
            for (int d = 0; d < n; d++)
                total += axis == 0 ? res[d][o]->rows : res[d][o]->cols;
            outs.emplace_back(new_dist(g, axis, r0->dtype, axis == 0 ? total : r0->rows, axis == 0 ? r0->cols : total),
                              db2_dist_decref);
            db2_dist *od = outs.back().get();
            int64_t at = 0;
            for (int d = 0; d < n; d++) {
                od->off[d] = at;
                at += axis == 0 ? res[d][o]->rows : res[d][o]->cols;
                od->off[d + 1] = at;
                od->shard[d] = res[d][o];
                res[d][o] = nullptr;
            }
            continue;
        }
        // ADD / MIN / MAX: combine the devices' partials; every device ends up with the combined result
        outs.emplace_back(new_dist(g, -1, r0->dtype, r0->rows, r0->cols), db2_dist_decref);
        db2_dist *od = outs.back().get();
        rc = combine_partials(g, res, o, (int)cmb, od->shard);
        if (rc != DB2_OK) {
            release_all();
            return rc;
        }
    }
    release_all(); // the partials that were copied (fold path); moved entries are NULL
    for (size_t o = 0; o < numOutputs; o++)
        outputs[o] = outs[o].release();
    return DB2_OK;
    DB2_API_END
}

/* fn(index, context, user) on every device of the group at once, each call on that device's worker thread with the
 * device bound (the small replicated arithmetic between two pipelines -- mu = sums / n on every device -- costs one
 * hand-off instead of a walk over the devices).  Returns the first failure. */
int db2_group_run(db2_group *g, db2_group_fn fn, void *user) {
    DB2_API_BEGIN
    DB2_CHECK(g && fn, DB2_EINVAL, "null argument");
    return for_each_device(g, [&](int d) -> int { return fn(d, g->ctxs[d], user); });
    DB2_API_END
}

/* In-place-style combine of one partial per device (ms[d] on device d of the group): on return ms[d] is the combined
 * matrix of device d (the handle may have been replaced; the old one is released). */
int db2_group_allreduce(db2_group *g, db2_matrix **ms, int combine) {
    DB2_API_BEGIN
    DB2_CHECK(g && ms, DB2_EINVAL, "null argument");
    DB2_CHECK(combine == DB2_COMBINE_ADD || combine == DB2_COMBINE_MIN || combine == DB2_COMBINE_MAX, DB2_EINVAL,
              "only ADD, MIN and MAX results are combined");
    const int n = (int)g->ctxs.size();
    std::vector<std::vector<db2_matrix *>> slots(n, std::vector<db2_matrix *>(1, nullptr));
    for (int d = 0; d < n; d++) {
        DB2_CHECK(ms[d] && ms[d]->ctx == g->ctxs[d], DB2_EINVAL,
                  "partial %d does not live on device index %d of the group", d, d);
        slots[d][0] = ms[d];
    }
    std::vector<db2_matrix *> out(n, nullptr);
    DB2_TRY(combine_partials(g, slots, 0, combine, out));
    for (int d = 0; d < n; d++) {
        if (slots[d][0]) { // not consumed: a new matrix replaces it
            bind_device(g->ctxs[d]);
            db2_matrix_decref(slots[d][0]);
        }
        ms[d] = out[d];
    }
    return DB2_OK;
    DB2_API_END
}

/* a copy of src as a new matrix of ctx (any two contexts of this process; a peer copy when their devices differ) */
int db2_matrix_to_context(db2_context *ctx, db2_matrix *src, db2_matrix **out) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && src && out, DB2_EINVAL, "null argument");
    return copy_to_context(ctx, src, out);
    DB2_API_END
}

/* dst[r0 : r0 + src.rows, c0 : c0 + src.cols] = src; dst and src may live on different devices */
int db2_matrix_copy_block(db2_matrix *dst, int64_t r0, int64_t c0, db2_matrix *src) {
    DB2_API_BEGIN
    DB2_CHECK(dst && src, DB2_EINVAL, "null argument");
    DB2_CHECK(dst->dtype == src->dtype, DB2_EINVAL, "value types differ");
    DB2_CHECK(r0 >= 0 && c0 >= 0 && r0 + src->rows <= dst->rows && c0 + src->cols <= dst->cols, DB2_EINVAL,
              "block (%lld x %lld at %lld, %lld) outside the destination (%lld x %lld)", (long long)src->rows,
              (long long)src->cols, (long long)r0, (long long)c0, (long long)dst->rows, (long long)dst->cols);
    if (src->rows * src->cols == 0)
        return DB2_OK;
    bind_device(src->ctx);
    DB2_TRY(ensure_device(src));
    cudaEvent_t ev;
    DB2_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    DB2_CUDA(cudaEventRecord(ev, src->ctx->stream));
    db2_context *ctx = dst->ctx;
    bind_device(ctx);
    DB2_TRY(ensure_device(dst));
    DB2_CUDA(cudaStreamWaitEvent(ctx->stream, ev, 0));
    DB2_CUDA(cudaEventDestroy(ev));
    const size_t es = src->esize();
    cudaMemcpy3DPeerParms p = {};
    p.srcDevice = src->ctx->device;
    p.dstDevice = ctx->device;
    p.srcPtr = make_cudaPitchedPtr(src->dev_ptr(), (size_t)src->dev_ld * es, (size_t)src->cols * es, (size_t)src->rows);
    p.dstPtr = make_cudaPitchedPtr(static_cast<char *>(dst->dev_ptr()) + ((size_t)r0 * dst->dev_ld + (size_t)c0) * es,
                                   (size_t)dst->dev_ld * es, (size_t)src->cols * es, (size_t)src->rows);
    p.extent = make_cudaExtent((size_t)src->cols * es, (size_t)src->rows, 1);
    DB2_CUDA(cudaMemcpy3DPeerAsync(&p, ctx->stream));
    dst->dev->version++;
    dst->host_valid = false;
    if (src->ctx != ctx) { // the source may be released by its own context right after this call
        cudaEvent_t done;
        DB2_CUDA(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
        DB2_CUDA(cudaEventRecord(done, ctx->stream));
        bind_device(src->ctx);
        DB2_CUDA(cudaStreamWaitEvent(src->ctx->stream, done, 0));
        DB2_CUDA(cudaEventDestroy(done));
        bind_device(ctx);
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.d2d_bytes += (uint64_t)src->rows * src->cols * es;
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
