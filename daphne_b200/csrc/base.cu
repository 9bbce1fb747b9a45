// Error state, device queries and thin device-memory/stream/event helpers of the C-ABI.
#include "common.cuh"

#include <mutex>

namespace db2 {

std::atomic<uint64_t> g_launches{0};

char *err_buf() {
    static thread_local char buf[ERR_BUF_LEN] = {0};
    return buf;
}

int set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf(), ERR_BUF_LEN, fmt, ap);
    va_end(ap);
    return code;
}

int sm_count() {
    static std::mutex mu;
    static int cached[64];
    static bool have[64] = {false};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return 148; // B200; only reached by size queries made without a device
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = 148;
        }
        cached[dev] = n;
        have[dev] = true;
    }
    return cached[dev];
}

} // namespace db2

using namespace db2;

extern "C" {

const char *db2_last_error(void) { return err_buf(); }
const char *db2_version(void) { return "daphne_b200 0.1 (sm_100a)"; }

int db2_device_count(int *count) {
    DB2_CHECK(count, DB2_EINVAL, "null count");
    cudaError_t e = cudaGetDeviceCount(count);
    if (e != cudaSuccess) {
        *count = 0;
        cudaGetLastError();
        return set_error(DB2_ECUDA, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    return DB2_OK;
}
int db2_set_device(int device) {
    DB2_CUDA(cudaSetDevice(device));
    return DB2_OK;
}
int db2_sm_count(int *count) {
    DB2_CHECK(count, DB2_EINVAL, "null count");
    *count = sm_count();
    return DB2_OK;
}

int db2_malloc(void **dptr, size_t bytes) {
    DB2_CHECK(dptr, DB2_EINVAL, "null dptr");
    *dptr = nullptr;
    if (bytes == 0)
        return DB2_OK;
    cudaError_t e = cudaMalloc(dptr, bytes);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return set_error(DB2_ENOMEM, "out of device memory allocating %zu bytes", bytes);
    }
    DB2_CUDA(e);
    return DB2_OK;
}
int db2_free(void *dptr) {
    if (dptr)
        DB2_CUDA(cudaFree(dptr));
    return DB2_OK;
}
int db2_malloc_host(void **hptr, size_t bytes) {
    DB2_CHECK(hptr, DB2_EINVAL, "null hptr");
    *hptr = nullptr;
    if (bytes == 0)
        return DB2_OK;
    DB2_CUDA(cudaMallocHost(hptr, bytes));
    return DB2_OK;
}
int db2_free_host(void *hptr) {
    if (hptr)
        DB2_CUDA(cudaFreeHost(hptr));
    return DB2_OK;
}
int db2_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes)
        DB2_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return DB2_OK;
}
int db2_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes)
        DB2_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return DB2_OK;
}
int db2_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream) {
    if (bytes)
        DB2_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return DB2_OK;
}
int db2_memset(void *dst, int byte, size_t bytes, void *stream) {
    if (bytes)
        DB2_CUDA(cudaMemsetAsync(dst, byte, bytes, as_stream(stream)));
    return DB2_OK;
}
int db2_stream_create(void **stream) {
    DB2_CHECK(stream, DB2_EINVAL, "null stream");
    cudaStream_t s;
    DB2_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = s;
    return DB2_OK;
}
int db2_stream_destroy(void *stream) {
    if (stream)
        DB2_CUDA(cudaStreamDestroy(as_stream(stream)));
    return DB2_OK;
}
int db2_stream_sync(void *stream) {
    DB2_CUDA(cudaStreamSynchronize(as_stream(stream)));
    return DB2_OK;
}
int db2_device_sync(void) {
    DB2_CUDA(cudaDeviceSynchronize());
    return DB2_OK;
}
int db2_event_create(void **event) {
    DB2_CHECK(event, DB2_EINVAL, "null event");
    cudaEvent_t e;
    DB2_CUDA(cudaEventCreate(&e));
    *event = e;
    return DB2_OK;
}
int db2_event_destroy(void *event) {
    if (event)
        DB2_CUDA(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
    return DB2_OK;
}
int db2_event_record(void *event, void *stream) {
    DB2_CUDA(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
    return DB2_OK;
}
int db2_event_elapsed_ms(void *start, void *stop, float *ms) {
    DB2_CHECK(ms, DB2_EINVAL, "null ms");
    DB2_CUDA(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(stop)));
    DB2_CUDA(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start), reinterpret_cast<cudaEvent_t>(stop)));
    return DB2_OK;
}
uint64_t db2_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

} // extern "C"
