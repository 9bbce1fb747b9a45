// Runtime: per-device context with a stream-ordered memory pool, matrix handles with host/device placements,
// and the operator entry points that allocate results and launch the db2k_* kernels on the context's stream.
#include "runtime.h"

namespace db2 {

DevBuf::~DevBuf() {
    if (ready) { // the block goes back to the pool in the order of the context's stream
        bind_device(ctx);
        wait_ready(ctx, this);
    }
    if (owned) {
        if (ptr)
            ctx_free(ctx, ptr, bytes);
        ctx_release(ctx);
    }
}

static void release_cached(db2_context *ctx);

void ctx_release(db2_context *ctx) {
    if (ctx->refs.fetch_sub(1) != 1)
        return;
    bind_device(ctx);
    db2_comm_destroy(ctx);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->side_stream)
        cudaStreamSynchronize(ctx->side_stream);
    ctx->side_keep.clear();
    if (ctx->scratch)
        ctx_free(ctx, ctx->scratch, ctx->scratch_bytes);
    release_cached(ctx);
    cudaFree(ctx->dev_status);
    cudaFreeHost(ctx->host_status);
    if (ctx->side_stream) {
        cudaStreamSynchronize(ctx->side_stream);
        cudaStreamDestroy(ctx->side_stream);
    }
    for (cudaEvent_t ev : ctx->scalar_ev)
        if (ev)
            cudaEventDestroy(ev);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}
HostBuf::~HostBuf() {
    if (owned && ptr)
        cudaFreeHost(ptr);
}

static size_t round_block(size_t bytes) {
    if (bytes <= (1u << 20)) {
        size_t p = 512;
        while (p < bytes)
            p <<= 1;
        return p;
    }
    const size_t g = 2u << 20;
    return (bytes + g - 1) / g * g;
}

static void release_cached(db2_context *ctx) {
    for (auto &kv : ctx->free_blocks) {
        cudaFree(kv.second);
        ctx->block_size.erase(kv.second);
    }
    ctx->free_blocks.clear();
    ctx->cached_bytes = 0;
}

int ctx_alloc(db2_context *ctx, size_t bytes, void **out) {
    *out = nullptr;
    if (bytes == 0)
        return DB2_OK;
    bind_device(ctx);
    const size_t want = round_block(bytes);
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->free_blocks.lower_bound(want);
    if (it != ctx->free_blocks.end() && it->first <= want + want / 4) {
        *out = it->second;
        ctx->cached_bytes -= it->first;
        ctx->free_blocks.erase(it);
    } else {
        if (ctx->mem_budget && ctx->stats.live_bytes + want > ctx->mem_budget)
            return set_error(DB2_ENOMEM, "out of device memory: %zu more bytes would exceed the budget of %zu bytes of "
                                         "the context on device %d (%llu in use)",
                             want, ctx->mem_budget, ctx->device, (unsigned long long)ctx->stats.live_bytes);
        cudaError_t e = cudaMalloc(out, want);
        if (e == cudaErrorMemoryAllocation) {
            cudaGetLastError();
            cudaStreamSynchronize(ctx->stream);
            release_cached(ctx); // hand the cached blocks back to the driver once and retry
            e = cudaMalloc(out, want);
            if (e == cudaErrorMemoryAllocation) {
                cudaGetLastError();
                return set_error(DB2_ENOMEM, "out of device memory allocating %zu bytes on device %d", want,
                                 ctx->device);
            }
        }
        DB2_CUDA(e);
        ctx->block_size[*out] = want;
        ctx->stats.allocs++;
        ctx->stats.alloc_bytes += want;
    }
    ctx->stats.live_bytes += bytes;
    if (ctx->stats.live_bytes > ctx->stats.peak_bytes)
        ctx->stats.peak_bytes = ctx->stats.live_bytes;
    return DB2_OK;
}

int ctx_free(db2_context *ctx, void *ptr, size_t bytes) {
    if (!ptr)
        return DB2_OK;
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.frees++;
    ctx->stats.live_bytes -= bytes;
    auto it = ctx->block_size.find(ptr);
    if (it == ctx->block_size.end())
        return set_error(DB2_EINVAL, "freeing a block this context did not allocate");
    ctx->free_blocks.emplace(it->second, ptr);
    ctx->cached_bytes += it->second;
    return DB2_OK;
}

int ctx_scratch(db2_context *ctx, size_t bytes, void **out) {
    if (bytes > ctx->scratch_bytes) {
        size_t want = bytes < (size_t)(4u << 20) ? (size_t)(4u << 20) : bytes;
        void *p = nullptr;
        DB2_TRY(ctx_alloc(ctx, want, &p));
        if (ctx->scratch)
            ctx_free(ctx, ctx->scratch, ctx->scratch_bytes); // stream-ordered: earlier kernels still see it
        ctx->scratch = p;
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return DB2_OK;
}

std::shared_ptr<DevBuf> make_devbuf(db2_context *ctx, size_t bytes) {
    void *p = nullptr;
    int rc = ctx_alloc(ctx, bytes, &p);
    if (rc != DB2_OK)
        throw Error(rc, err_buf());
    ctx->refs.fetch_add(1);
    return std::shared_ptr<DevBuf>(new DevBuf{ctx, p, bytes, true});
}

int ensure_device(db2_matrix *m) {
    if (m->dev && m->dev->ready) {
        bind_device(m->ctx);
        wait_ready(m->ctx, m->dev.get());
    }
    if (m->dev_valid)
        return DB2_OK;
    if (m->deferred())
        return lazy_force(m);
    DB2_CHECK(m->host_valid && m->host, DB2_EINVAL, "matrix has no valid placement");
    db2_context *ctx = m->ctx;
    bind_device(ctx);
    const size_t es = m->esize();
    if (!m->dev) {
        m->dev = make_devbuf(ctx, (size_t)m->rows * m->cols * es);
        m->dev_off = 0;
        m->dev_ld = m->cols;
    } else {
        m->dev->version++;
    }
    if (m->rows * m->cols > 0) {
        if (m->host_ld == m->cols && m->dev_ld == m->cols)
            DB2_CUDA(cudaMemcpyAsync(m->dev_ptr(), m->host_ptr(), (size_t)m->rows * m->cols * es,
                                     cudaMemcpyHostToDevice, ctx->stream));
        else
            DB2_CUDA(cudaMemcpy2DAsync(m->dev_ptr(), (size_t)m->dev_ld * es, m->host_ptr(), (size_t)m->host_ld * es,
                                       (size_t)m->cols * es, (size_t)m->rows, cudaMemcpyHostToDevice, ctx->stream));
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.h2d_bytes += (uint64_t)m->rows * m->cols * es;
    }
    m->dev_valid = true;
    return DB2_OK;
}

int prepare_result(db2_context *ctx, db2_matrix **res, int dtype, int64_t rows, int64_t cols) {
    DB2_CHECK(res, DB2_EINVAL, "null result slot");
    if (*res == nullptr)
        return db2_matrix_create(ctx, dtype, rows, cols, 0, res);
    db2_matrix *r = *res;
    DB2_CHECK(r->dtype == dtype && r->rows == rows && r->cols == cols, DB2_EINVAL,
              "pre-allocated result has shape (%lld x %lld) / type %d, expected (%lld x %lld) / type %d",
              (long long)r->rows, (long long)r->cols, r->dtype, (long long)rows, (long long)cols, dtype);
    if (r->deferred()) {
        lazy_forget(r);
        r->lazy.reset();
        r->pend_src.reset();
        r->pend_op = -1;
        r->onehot.reset();
        r->syrk_of.reset();
    }
    r->is_seq = false;
    r->combined = false;
    // a buffer that deferred chains (or other handles) still read is not overwritten: the result gets a fresh one.
    // Row views are the exception: writing through a view is how results are placed into a larger matrix.
    if (r->dev)
        r->dev->version++;
    if (!r->dev || (!r->is_view && r->dev.use_count() > 1)) {
        r->dev = make_devbuf(ctx, (size_t)rows * cols * r->esize());
        r->dev_off = 0;
        r->dev_ld = cols;
    }
    r->dev_valid = true;
    r->host_valid = false;
    return DB2_OK;
}

static void count_launches(db2_context *ctx, uint64_t before) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->stats.launches += g_launches.load(std::memory_order_relaxed) - before;
}

} // namespace db2

using namespace db2;

extern "C" {

int db2_context_create(int device, db2_context **out) {
    DB2_API_BEGIN
    DB2_CHECK(out, DB2_EINVAL, "null context slot");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n < 1) {
        cudaGetLastError();
        return set_error(DB2_ECUDA, "no CUDA device available (daphne_b200 has no CPU fallback): %s",
                         cudaGetErrorString(e));
    }
    DB2_CHECK(device >= 0 && device < n, DB2_EINVAL, "requested device %d but only %d device(s) present", device, n);
    DB2_CUDA(cudaSetDevice(device));
    std::unique_ptr<db2_context> ctx(new db2_context());
    ctx->device = device;
    const char *eager = getenv("DB2_EAGER");
    ctx->eager = eager && eager[0] == '1';
    DB2_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    DB2_CUDA(cudaMalloc(&ctx->dev_status, 256));
    DB2_CUDA(cudaMemset(ctx->dev_status, 0, 256));
    DB2_CUDA(cudaMallocHost(&ctx->host_status, 256));
    *ctx->host_status = 0;
    *out = ctx.release();
    return DB2_OK;
    DB2_API_END
}

int db2_context_destroy(db2_context *ctx) {
    if (!ctx)
        return DB2_OK;
    bind_device(ctx);
    cudaStreamSynchronize(ctx->stream);
    db2_rtc_wait(); // a background compilation of a chain's kernel (fused_rtc.cu) must not outlive the process
    ctx_release(ctx);
    return DB2_OK;
}

int db2_context_device(const db2_context *ctx, int *device) {
    DB2_CHECK(ctx && device, DB2_EINVAL, "null argument");
    *device = ctx->device;
    return DB2_OK;
}
int db2_context_ordinal(const db2_context *ctx, int *dup) {
    DB2_CHECK(ctx && dup, DB2_EINVAL, "null argument");
    *dup = ctx->dup;
    return DB2_OK;
}
void *db2_context_stream(db2_context *ctx) { return ctx ? ctx->stream : nullptr; }
int db2_context_sync(db2_context *ctx) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    bind_device(ctx);
    DB2_TRY(lazy_flush_all(ctx));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    return DB2_OK;
}
int db2_context_set_mem_budget(db2_context *ctx, size_t bytes) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->mem_budget = bytes;
    return DB2_OK;
}
int db2_context_stats(db2_context *ctx, db2_stats *out) {
    DB2_CHECK(ctx && out, DB2_EINVAL, "null argument");
    std::lock_guard<std::mutex> lock(ctx->mu);
    *out = ctx->stats;
    return DB2_OK;
}

int db2_matrix_create(db2_context *ctx, int dtype, int64_t rows, int64_t cols, int zero, db2_matrix **out) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && out, DB2_EINVAL, "null argument");
    DB2_CHECK(rows >= 0 && cols >= 0, DB2_EINVAL, "negative dimension");
    DB2_CHECK(dtype >= DB2_F64 && dtype <= DB2_U8, DB2_EINVAL, "bad value type %d", dtype);
    std::unique_ptr<db2_matrix> m(new db2_matrix());
    m->ctx = ctx;
    m->dtype = dtype;
    m->rows = rows;
    m->cols = cols;
    m->dev = make_devbuf(ctx, (size_t)rows * cols * m->esize());
    m->dev_ld = cols;
    m->dev_valid = true;
    if (zero && rows * cols > 0)
        DB2_CUDA(cudaMemsetAsync(m->dev->ptr, 0, m->dev->bytes, ctx->stream));
    *out = m.release();
    return DB2_OK;
    DB2_API_END
}

int db2_matrix_wrap_host(db2_context *ctx, int dtype, int64_t rows, int64_t cols, int64_t ld, void *host,
                         db2_matrix **out) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && out, DB2_EINVAL, "null argument");
    DB2_CHECK(rows >= 0 && cols >= 0 && ld >= cols, DB2_EINVAL, "bad shape (%lld x %lld, ld %lld)", (long long)rows,
              (long long)cols, (long long)ld);
    DB2_CHECK(host || rows * cols == 0, DB2_EINVAL, "null host buffer");
    DB2_CHECK(dtype >= DB2_F64 && dtype <= DB2_U8, DB2_EINVAL, "bad value type %d", dtype);
    std::unique_ptr<db2_matrix> m(new db2_matrix());
    m->ctx = ctx;
    m->dtype = dtype;
    m->rows = rows;
    m->cols = cols;
    m->host = std::shared_ptr<HostBuf>(new HostBuf{host, (size_t)rows * ld * dtype_size(dtype), false});
    m->host_ld = ld;
    m->host_valid = true;
    *out = m.release();
    return DB2_OK;
    DB2_API_END
}

int db2_matrix_wrap_device(db2_context *ctx, int dtype, int64_t rows, int64_t cols, int64_t ld, void *dptr,
                           db2_matrix **out) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && out, DB2_EINVAL, "null argument");
    DB2_CHECK(rows >= 0 && cols >= 0 && ld >= cols, DB2_EINVAL, "bad shape");
    DB2_CHECK(dptr || rows * cols == 0, DB2_EINVAL, "null device buffer");
    DB2_CHECK(dtype >= DB2_F64 && dtype <= DB2_U8, DB2_EINVAL, "bad value type %d", dtype);
    std::unique_ptr<db2_matrix> m(new db2_matrix());
    m->ctx = ctx;
    m->dtype = dtype;
    m->rows = rows;
    m->cols = cols;
    m->dev = std::shared_ptr<DevBuf>(new DevBuf{ctx, dptr, (size_t)rows * ld * dtype_size(dtype), false});
    m->dev_ld = ld;
    m->dev_valid = true;
    *out = m.release();
    return DB2_OK;
    DB2_API_END
}

int db2_matrix_slice_rows(db2_matrix *src, int64_t r0, int64_t r1, db2_matrix **view) {
    DB2_API_BEGIN
    DB2_CHECK(src && view, DB2_EINVAL, "null argument");
    DB2_CHECK(0 <= r0 && r0 <= r1 && r1 <= src->rows, DB2_EINVAL, "row range [%lld, %lld) outside [0, %lld)",
              (long long)r0, (long long)r1, (long long)src->rows);
    std::unique_ptr<db2_matrix> m(new db2_matrix());
    m->ctx = src->ctx;
    m->dtype = src->dtype;
    m->rows = r1 - r0;
    m->cols = src->cols;
    m->is_view = true;
    // a view shares the parent's buffers; make the parent's device placement current first so that all views of a
    // host matrix share one transfer (and a deferred parent is produced once)
    if (!src->dev_valid && src->ctx)
        DB2_TRY(ensure_device(src));
    if (src->dev) {
        m->dev = src->dev;
        m->dev_off = src->dev_off + r0 * src->dev_ld;
        m->dev_ld = src->dev_ld;
        m->dev_valid = src->dev_valid;
    }
    if (src->host) {
        m->host = src->host;
        m->host_off = src->host_off + r0 * src->host_ld;
        m->host_ld = src->host_ld;
        m->host_valid = src->host_valid;
    }
    *view = m.release();
    return DB2_OK;
    DB2_API_END
}

// zero-copy view of the columns [c0, c1): same buffers, same leading dimension, the first column moved
int db2_matrix_slice_cols(db2_matrix *src, int64_t c0, int64_t c1, db2_matrix **view) {
    DB2_API_BEGIN
    DB2_CHECK(src && view, DB2_EINVAL, "null argument");
    DB2_CHECK(0 <= c0 && c0 <= c1 && c1 <= src->cols, DB2_EINVAL, "column range [%lld, %lld) outside [0, %lld)",
              (long long)c0, (long long)c1, (long long)src->cols);
    if (!src->dev_valid && src->ctx)
        DB2_TRY(ensure_device(src));
    std::unique_ptr<db2_matrix> m(new db2_matrix());
    m->ctx = src->ctx;
    m->dtype = src->dtype;
    m->rows = src->rows;
    m->cols = c1 - c0;
    m->is_view = true;
    if (src->dev) {
        m->dev = src->dev;
        m->dev_off = src->dev_off + c0;
        m->dev_ld = src->dev_ld;
        m->dev_valid = src->dev_valid;
    }
    if (src->host) {
        m->host = src->host;
        m->host_off = src->host_off + c0;
        m->host_ld = src->host_ld;
        m->host_valid = src->host_valid;
    }
    *view = m.release();
    return DB2_OK;
    DB2_API_END
}

// SliceRow / SliceCol with the reference's index rules (negative bounds count from the end) and messages
static int resolve_slice(const char *what, const char *dim, int64_t lo, int64_t hi, int64_t n, int64_t *a, int64_t *b) {
    const int64_t lo_in = lo, hi_in = hi;
    if (lo < 0) {
        lo += n;
        if (hi <= 0)
            hi += n;
    } else if (hi < 0) {
        hi += n;
    }
    if (lo < 0 || lo >= n || hi < lo || n < hi)
        return set_error(DB2_EDOMAIN, "invalid arguments '%lld, %lld' passed to %s: it must hold 0 <= lowerIncl < #%s "
                                      "and lowerIncl <= upperExcl <= #%s",
                         (long long)lo_in, (long long)hi_in, what, dim, dim);
    *a = lo;
    *b = hi;
    return DB2_OK;
}
int db2_sliceRow(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int64_t lowerIncl, int64_t upperExcl) {
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    DB2_CHECK(*res == nullptr, DB2_EUNSUPPORTED, "sliceRow returns a view: a pre-allocated result is not supported");
    int64_t a = 0, b = 0;
    DB2_TRY(resolve_slice("SliceRow", "rows", lowerIncl, upperExcl, arg->rows, &a, &b));
    return db2_matrix_slice_rows(arg, a, b, res);
}
int db2_sliceCol(db2_context *ctx, db2_matrix **res, db2_matrix *arg, int64_t lowerIncl, int64_t upperExcl) {
    DB2_CHECK(ctx && res && arg, DB2_EINVAL, "null argument");
    DB2_CHECK(*res == nullptr, DB2_EUNSUPPORTED, "sliceCol returns a view: a pre-allocated result is not supported");
    int64_t a = 0, b = 0;
    DB2_TRY(resolve_slice("SliceCol", "columns", lowerIncl, upperExcl, arg->cols, &a, &b));
    return db2_matrix_slice_cols(arg, a, b, res);
}

int db2_matrix_incref(db2_matrix *m) {
    DB2_CHECK(m, DB2_EINVAL, "null matrix");
    m->refs.fetch_add(1);
    return DB2_OK;
}
int db2_matrix_decref(db2_matrix *m) {
    if (!m)
        return DB2_OK;
    if (m->refs.fetch_sub(1) == 1) {
        if (m->deferred())
            lazy_forget(m);
        delete m;
    }
    return DB2_OK;
}
int db2_matrix_info(const db2_matrix *m, int *dtype, int64_t *rows, int64_t *cols) {
    DB2_CHECK(m, DB2_EINVAL, "null matrix");
    if (dtype)
        *dtype = m->dtype;
    if (rows)
        *rows = m->rows;
    if (cols)
        *cols = m->cols;
    return DB2_OK;
}
int db2_matrix_device_ptr(db2_matrix *m, void **dptr, int64_t *ld) {
    DB2_API_BEGIN
    DB2_CHECK(m && dptr, DB2_EINVAL, "null argument");
    DB2_TRY(ensure_device(m));
    *dptr = m->dev_ptr();
    if (ld)
        *ld = m->dev_ld;
    return DB2_OK;
    DB2_API_END
}

int db2_matrix_to_host(db2_matrix *m, void *dst, int64_t dst_ld) {
    DB2_API_BEGIN
    DB2_CHECK(m && (dst || m->rows * m->cols == 0), DB2_EINVAL, "null argument");
    DB2_CHECK(dst_ld >= m->cols, DB2_EINVAL, "destination leading dimension too small");
    const size_t es = m->esize();
    if (m->rows * m->cols == 0)
        return DB2_OK;
    if (m->deferred())
        DB2_TRY(lazy_force(m));
    if (m->dev_valid) {
        db2_context *ctx = m->ctx;
        bind_device(ctx);
        wait_ready(ctx, m->dev.get());
        if ((dst_ld == m->cols && m->dev_ld == m->cols) || m->rows == 1) // contiguous: one linear copy
            DB2_CUDA(cudaMemcpyAsync(dst, m->dev_ptr(), (size_t)m->rows * m->cols * es, cudaMemcpyDeviceToHost,
                                     ctx->stream));
        else
            DB2_CUDA(cudaMemcpy2DAsync(dst, (size_t)dst_ld * es, m->dev_ptr(), (size_t)m->dev_ld * es,
                                       (size_t)m->cols * es, (size_t)m->rows, cudaMemcpyDeviceToHost, ctx->stream));
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.d2h_bytes += (uint64_t)m->rows * m->cols * es;
    } else {
        DB2_CHECK(m->host_valid, DB2_EINVAL, "matrix has no valid placement");
        for (int64_t r = 0; r < m->rows; r++)
            memcpy(static_cast<char *>(dst) + r * dst_ld * es, static_cast<char *>(m->host_ptr()) + r * m->host_ld * es,
                   (size_t)m->cols * es);
    }
    return DB2_OK;
    DB2_API_END
}

// The same copy on the context's side stream, ordered after everything queued on the compute stream so far; returns
// without waiting.  A step's results can so travel to the host while the next step's input travels to the device
// (PCIe carries both directions at once).  dst must stay valid, and should be pinned, until db2_context_side_sync.
int db2_matrix_to_host_async(db2_matrix *m, void *dst, int64_t dst_ld) {
    DB2_API_BEGIN
    DB2_CHECK(m && (dst || m->rows * m->cols == 0), DB2_EINVAL, "null argument");
    DB2_CHECK(dst_ld >= m->cols, DB2_EINVAL, "destination leading dimension too small");
    if (m->rows * m->cols == 0)
        return DB2_OK;
    if (m->deferred())
        DB2_TRY(lazy_force(m));
    if (!m->dev_valid)
        return db2_matrix_to_host(m, dst, dst_ld);
    db2_context *ctx = m->ctx;
    bind_device(ctx);
    const size_t es = m->esize();
    wait_ready(ctx, m->dev.get());
    if (!ctx->side_stream)
        DB2_CUDA(cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
    cudaEvent_t queued;
    DB2_CUDA(cudaEventCreateWithFlags(&queued, cudaEventDisableTiming));
    DB2_CUDA(cudaEventRecord(queued, ctx->stream));
    DB2_CUDA(cudaStreamWaitEvent(ctx->side_stream, queued, 0));
    DB2_CUDA(cudaEventDestroy(queued));
    if ((dst_ld == m->cols && m->dev_ld == m->cols) || m->rows == 1)
        DB2_CUDA(cudaMemcpyAsync(dst, m->dev_ptr(), (size_t)m->rows * m->cols * es, cudaMemcpyDeviceToHost,
                                 ctx->side_stream));
    else
        DB2_CUDA(cudaMemcpy2DAsync(dst, (size_t)dst_ld * es, m->dev_ptr(), (size_t)m->dev_ld * es, (size_t)m->cols * es,
                                   (size_t)m->rows, cudaMemcpyDeviceToHost, ctx->side_stream));
    bool drain = false;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->side_keep.push_back(m->dev);
        ctx->stats.d2h_bytes += (uint64_t)m->rows * m->cols * es;
        drain = ctx->side_keep.size() >= 256; // a caller that never waits must not pin device memory without bound
    }
    if (drain)
        return db2_context_side_sync(ctx);
    return DB2_OK;
    DB2_API_END
}
// waits for the copies (and collectives) queued on the side stream
int db2_context_side_sync(db2_context *ctx) {
    DB2_CHECK(ctx, DB2_EINVAL, "null context");
    bind_device(ctx);
    if (ctx->side_stream)
        DB2_CUDA(cudaStreamSynchronize(ctx->side_stream));
    std::vector<std::shared_ptr<DevBuf>> done;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        done.swap(ctx->side_keep);
    }
    return DB2_OK;
}

// ---------------------------------------------------------------------------
// operator calls
// ---------------------------------------------------------------------------

int db2_ewBinaryMat(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && lhs && rhs, DB2_EINVAL, "null argument");
    DB2_CHECK(lhs->dtype == rhs->dtype, DB2_EUNSUPPORTED, "ewBinaryMat: value types of lhs and rhs differ");
    // shape check before anything is allocated (message of EwBinaryMat.h:98-106)
    const bool same = lhs->rows == rhs->rows && lhs->cols == rhs->cols;
    const bool rvec = lhs->cols == rhs->cols && (rhs->rows == 1 || lhs->rows == 1);
    const bool cvec = lhs->rows == rhs->rows && (rhs->cols == 1 || lhs->cols == 1);
    DB2_CHECK(same || rvec || cvec, DB2_EINVAL,
              "EwBinaryMat(Dense) - lhs and rhs must either have the same dimensions, or one of them must be a "
              "row/column vector with the width/height of the other, but lhs has shape (%lld x %lld) and rhs has "
              "shape (%lld x %lld)",
              (long long)lhs->rows, (long long)lhs->cols, (long long)rhs->rows, (long long)rhs->cols);
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_CHECK(res, DB2_EINVAL, "null result slot");
    bool handled = false;
    DB2_TRY(lazy_try_binary(ctx, op, res, lhs, rhs, &handled));
    if (handled) {
        count_launches(ctx, before);
        return DB2_OK;
    }
    DB2_TRY(ensure_device(lhs));
    DB2_TRY(ensure_device(rhs));
    DB2_TRY(prepare_result(ctx, res, lhs->dtype, lhs->rows, lhs->cols));
    db2_matrix *r = *res;
    DB2_TRY(db2k_ew_binary(lhs->dtype, op, lhs->dev_ptr(), lhs->rows, lhs->cols, lhs->dev_ld, rhs->dev_ptr(),
                           rhs->rows, rhs->cols, rhs->dev_ld, r->dev_ptr(), r->dev_ld, ctx->stream));
    count_launches(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_outerBinary(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, db2_matrix *rhs) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && lhs && rhs, DB2_EINVAL, "null argument");
    DB2_CHECK(lhs->dtype == rhs->dtype, DB2_EUNSUPPORTED, "outerBinary: value types of lhs and rhs differ");
    DB2_CHECK(lhs->cols == 1, DB2_EINVAL, "outerBinary: lhs must be a column (mx1) matrix");
    DB2_CHECK(rhs->rows == 1, DB2_EINVAL, "outerBinary: rhs must be a row (1xn) matrix");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(lhs));
    DB2_TRY(ensure_device(rhs));
    DB2_TRY(prepare_result(ctx, res, lhs->dtype, lhs->rows, rhs->cols));
    db2_matrix *r = *res;
    DB2_TRY(db2k_outer_binary(lhs->dtype, op, lhs->dev_ptr(), lhs->dev_ld, lhs->rows, rhs->dev_ptr(), rhs->cols,
                              r->dev_ptr(), r->dev_ld, ctx->stream));
    count_launches(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_ewBinaryObjSca(db2_context *ctx, int op, db2_matrix **res, db2_matrix *lhs, const void *scalar) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && lhs && scalar, DB2_EINVAL, "null argument");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_CHECK(res, DB2_EINVAL, "null result slot");
    bool handled = false;
    DB2_TRY(lazy_try_scalar(ctx, op, res, lhs, scalar, &handled));
    if (handled) {
        count_launches(ctx, before);
        return DB2_OK;
    }
    DB2_TRY(ensure_device(lhs));
    DB2_TRY(prepare_result(ctx, res, lhs->dtype, lhs->rows, lhs->cols));
    db2_matrix *r = *res;
    DB2_TRY(db2k_ew_binary_sca(lhs->dtype, op, lhs->dev_ptr(), lhs->rows, lhs->cols, lhs->dev_ld, scalar,
                               r->dev_ptr(), r->dev_ld, ctx->stream));
    count_launches(ctx, before);
    return DB2_OK;
    DB2_API_END
}

static bool has_domain(int op) {
    return op == DB2_U_SQRT || op == DB2_U_LN || op == DB2_U_ASIN || op == DB2_U_ACOS;
}

int db2_ewUnaryMat(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && arg, DB2_EINVAL, "null argument");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_CHECK(res, DB2_EINVAL, "null result slot");
    bool handled = false;
    DB2_TRY(lazy_try_unary(ctx, op, res, arg, &handled));
    if (handled) {
        count_launches(ctx, before);
        return DB2_OK;
    }
    DB2_TRY(ensure_device(arg));
    DB2_TRY(prepare_result(ctx, res, arg->dtype, arg->rows, arg->cols));
    db2_matrix *r = *res;
    const bool dom = has_domain(op);
    DB2_TRY(db2k_ew_unary(arg->dtype, op, arg->dev_ptr(), arg->rows, arg->cols, arg->dev_ld, r->dev_ptr(), r->dev_ld,
                          dom ? ctx->dev_status : nullptr, ctx->stream));
    count_launches(ctx, before);
    if (dom) {
        // the reference throws std::domain_error from inside the kernel call, so the check has to be synchronous
        DB2_CUDA(cudaMemcpyAsync(ctx->host_status, ctx->dev_status, sizeof(int32_t), cudaMemcpyDeviceToHost,
                                 ctx->stream));
        DB2_CUDA(cudaStreamSynchronize(ctx->stream));
        if (*ctx->host_status != 0) {
            *ctx->host_status = 0;
            DB2_CUDA(cudaMemsetAsync(ctx->dev_status, 0, sizeof(int32_t), ctx->stream));
            static const char *names[] = {"MINUS", "ABS", "SIGN", "SQRT", "EXP", "LN", "SIN", "COS", "TAN", "ASIN",
                                          "ACOS"};
            return set_error(DB2_EDOMAIN, "invalid argument passed to unary func %s (outside its domain)", names[op]);
        }
    }
    return DB2_OK;
    DB2_API_END
}

static int agg_result_dtype(int op, int dtype) {
    return (op == DB2_AGG_IDXMIN || op == DB2_AGG_IDXMAX) ? DB2_U64 : dtype;
}

int db2_aggRow(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && arg, DB2_EINVAL, "null argument");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_CHECK(res, DB2_EINVAL, "null result slot");
    bool handled = false;
    DB2_TRY(lazy_try_agg_row(ctx, op, res, arg, &handled));
    if (handled) {
        count_launches(ctx, before);
        return DB2_OK;
    }
    DB2_TRY(ensure_device(arg));
    DB2_TRY(prepare_result(ctx, res, agg_result_dtype(op, arg->dtype), arg->rows, 1));
    db2_matrix *r = *res;
    DB2_TRY(db2k_agg_row(arg->dtype, op, arg->dev_ptr(), arg->rows, arg->cols, arg->dev_ld, r->dev_ptr(), r->dev_ld,
                         ctx->stream));
    count_launches(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_aggCol(db2_context *ctx, int op, db2_matrix **res, db2_matrix *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && arg, DB2_EINVAL, "null argument");
    bind_device(ctx);
    const uint64_t before = g_launches.load();
    DB2_CHECK(res, DB2_EINVAL, "null result slot");
    bool handled = false;
    DB2_TRY(onehot_try_agg_col(ctx, op, res, arg, &handled));
    if (handled)
        return DB2_OK;
    DB2_TRY(colstats_try_agg_col(ctx, op, res, arg, &handled));
    if (handled)
        return DB2_OK;
    DB2_TRY(lazy_try_agg_col(ctx, op, res, arg, &handled));
    if (handled) {
        count_launches(ctx, before);
        return DB2_OK;
    }
    DB2_TRY(ensure_device(arg));
    DB2_TRY(prepare_result(ctx, res, agg_result_dtype(op, arg->dtype), 1, arg->cols));
    db2_matrix *r = *res;
    const size_t sb = db2k_agg_col_scratch_bytes(arg->dtype, op, arg->rows, arg->cols);
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, sb, &scratch));
    DB2_TRY(db2k_agg_col(arg->dtype, op, arg->dev_ptr(), arg->rows, arg->cols, arg->dev_ld, r->dev_ptr(), scratch,
                         ctx->scratch_bytes, ctx->stream));
    count_launches(ctx, before);
    return DB2_OK;
    DB2_API_END
}

int db2_aggAll(db2_context *ctx, int op, void *res_host, db2_matrix *arg) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && arg && res_host, DB2_EINVAL, "null argument");
    bind_device(ctx);
    {
        bool handled = false;
        DB2_TRY(lazy_try_agg_all(ctx, op, static_cast<double *>(res_host), arg, &handled));
        if (handled)
            return DB2_OK;
    }
    const uint64_t before = g_launches.load();
    DB2_TRY(ensure_device(arg));
    const size_t sb = db2k_agg_all_scratch_bytes(arg->dtype, op, arg->rows, arg->cols) + 64;
    void *scratch = nullptr;
    DB2_TRY(ctx_scratch(ctx, sb, &scratch));
    // the scalar result sits in the first 16 bytes of the scratch area, partials behind it
    DB2_TRY(db2k_agg_all(arg->dtype, op, arg->dev_ptr(), arg->rows, arg->cols, arg->dev_ld, scratch,
                         static_cast<char *>(scratch) + 64, ctx->scratch_bytes - 64, ctx->stream));
    count_launches(ctx, before);
    DB2_CUDA(cudaMemcpyAsync(res_host, scratch, arg->esize(), cudaMemcpyDeviceToHost, ctx->stream));
    DB2_CUDA(cudaStreamSynchronize(ctx->stream));
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.d2h_bytes += arg->esize();
    }
    return DB2_OK;
    DB2_API_END
}

// ---- a scalar that the host needs later: start now, wait when it is needed ----
// The two halves of aggAll (and of reading a 1 x 1 matrix).  Between them the caller may queue more work on the
// context, so the device does not idle while the host looks at the value: a loop whose condition is a reduction
// (`while (sum(u != c) > 0)`) queues its next trip before it waits for the previous trip's count.  Two slots.
static double *scalar_slot(db2_context *ctx, int slot) { return reinterpret_cast<double *>(ctx->host_status + 48) + slot; }

static int scalar_mark(db2_context *ctx, int slot) {
    if (!ctx->scalar_ev[slot])
        DB2_CUDA(cudaEventCreateWithFlags(&ctx->scalar_ev[slot], cudaEventDisableTiming));
    DB2_CUDA(cudaEventRecord(ctx->scalar_ev[slot], ctx->stream));
    return DB2_OK;
}

int db2_aggAllStart(db2_context *ctx, int op, db2_matrix *arg, int slot) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && arg, DB2_EINVAL, "null argument");
    DB2_CHECK(slot == 0 || slot == 1, DB2_EINVAL, "scalar slot %d (0 or 1)", slot);
    DB2_CHECK(arg->dtype == DB2_F64, DB2_EUNSUPPORTED, "aggAllStart: f64 only");
    bind_device(ctx);
    bool handled = false;
    DB2_TRY(lazy_try_agg_all_start(ctx, op, scalar_slot(ctx, slot), arg, &handled));
    if (!handled) { // any other argument: the complete call now, the value parked in the slot
        double v = 0.0;
        DB2_TRY(db2_aggAll(ctx, op, &v, arg));
        *scalar_slot(ctx, slot) = v;
    }
    return scalar_mark(ctx, slot);
    DB2_API_END
}

int db2_scalarStart(db2_context *ctx, db2_matrix *m, int slot) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && m, DB2_EINVAL, "null argument");
    DB2_CHECK(slot == 0 || slot == 1, DB2_EINVAL, "scalar slot %d (0 or 1)", slot);
    DB2_CHECK(m->dtype == DB2_F64 && m->rows == 1 && m->cols == 1, DB2_EINVAL, "scalarStart: a 1 x 1 f64 matrix");
    bind_device(ctx);
    DB2_TRY(ensure_device(m));
    DB2_CUDA(cudaMemcpyAsync(scalar_slot(ctx, slot), m->dev_ptr(), sizeof(double), cudaMemcpyDeviceToHost,
                             ctx->stream));
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.d2h_bytes += sizeof(double);
    }
    return scalar_mark(ctx, slot);
    DB2_API_END
}

int db2_scalarWait(db2_context *ctx, int slot, double *res) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res, DB2_EINVAL, "null argument");
    DB2_CHECK((slot == 0 || slot == 1) && ctx->scalar_ev[slot], DB2_EINVAL, "scalar slot %d was not started", slot);
    bind_device(ctx);
    DB2_CUDA(cudaEventSynchronize(ctx->scalar_ev[slot]));
    *res = *scalar_slot(ctx, slot);
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
