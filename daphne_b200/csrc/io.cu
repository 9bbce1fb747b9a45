// Device-direct matrix ingest: DAPHNE's binary matrix format (.dbdf) read straight into a device placement.
//
// The reference reads a .dbdf file into a host DenseMatrix through 1 MiB std::vector chunks (ReadDaphne.h:58-100,
// DaphneSerializer.h:79-260) and the CUDA backend later copies that pageable memory to the device synchronously
// (AllocationDescriptorCUDA.h:60-68).  Here the file goes through two pinned staging buffers: while one is on its way
// to the device (cudaMemcpyAsync on the context's stream) the next piece of the file is read into the other, so a
// multi-GiB input is limited by the slower of the file system and PCIe, never by a pageable copy, and no host copy of
// the matrix exists afterwards.  Writing is the mirror image.
//
// Layout of a dense file (doc/BinaryFormat.md; DaphneFile.h:22-41; DaphneSerializer.h:117-172), little endian, packed:
//   u8 version = 1 | u8 data type = 1 (DenseMatrix) | u64 rows | u64 cols | u8 value type code
//   u64 block row = 0 | u64 block column = 0 | u32 block rows | u32 block cols | u8 block type = 1 (dense)
//   u8 value type code | rows * cols values, row-major                                     (header: 45 bytes)
// Value type codes are ValueTypeCode's (ValueTypeCode.h:29-43): SI64 = 2, UI64 = 5, F32 = 6, F64 = 7.
#include "runtime.h"

#include <cerrno>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

namespace db2 {

constexpr size_t DBDF_HEADER = 45;
constexpr size_t STAGE_BYTES = (size_t)64 << 20;

static int vt_code_to_dtype(int code) {
    switch (code) {
    case 2: return DB2_I64;
    case 5: return DB2_U64;
    case 6: return DB2_F32;
    case 7: return DB2_F64;
    default: return -1;
    }
}
static int dtype_to_vt_code(int dtype) {
    switch (dtype) {
    case DB2_I64: return 2;
    case DB2_U64: return 5;
    case DB2_F32: return 6;
    default: return 7;
    }
}

struct Fd {
    int fd = -1;
    ~Fd() {
        if (fd >= 0)
            close(fd);
    }
};
struct Staging { // two pinned buffers with an event each
    void *buf[2] = {nullptr, nullptr};
    cudaEvent_t ev[2] = {nullptr, nullptr};
    ~Staging() {
        for (int i = 0; i < 2; i++) {
            if (buf[i])
                cudaFreeHost(buf[i]);
            if (ev[i])
                cudaEventDestroy(ev[i]);
        }
    }
    int init(size_t bytes) {
        for (int i = 0; i < 2; i++) {
            DB2_CUDA(cudaMallocHost(&buf[i], bytes));
            DB2_CUDA(cudaEventCreateWithFlags(&ev[i], cudaEventDisableTiming));
        }
        return DB2_OK;
    }
};

static int read_fully(int fd, void *dst, size_t bytes, off_t off, const char *path) {
    size_t done = 0;
    while (done < bytes) {
        const ssize_t n = pread(fd, static_cast<char *>(dst) + done, bytes - done, off + (off_t)done);
        if (n < 0 && errno == EINTR)
            continue;
        DB2_CHECK(n > 0, DB2_EINVAL, "%s: file ends after %zu of %zu value bytes", path, (size_t)off + done - DBDF_HEADER,
                  (size_t)off + bytes - DBDF_HEADER);
        done += (size_t)n;
    }
    return DB2_OK;
}
static int write_fully(int fd, const void *src, size_t bytes, const char *path) {
    size_t done = 0;
    while (done < bytes) {
        const ssize_t n = write(fd, static_cast<const char *>(src) + done, bytes - done);
        if (n < 0 && errno == EINTR)
            continue;
        DB2_CHECK(n > 0, DB2_EINVAL, "%s: write failed: %s", path, strerror(errno));
        done += (size_t)n;
    }
    return DB2_OK;
}

} // namespace db2

using namespace db2;

extern "C" {

int db2_readDaphne(db2_context *ctx, db2_matrix **res, const char *path) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && res && path, DB2_EINVAL, "null argument");
    DB2_CHECK(*res == nullptr, DB2_EINVAL, "readDaphne allocates its result");
    Fd f;
    f.fd = open(path, O_RDONLY);
    DB2_CHECK(f.fd >= 0, DB2_EINVAL, "cannot open %s: %s", path, strerror(errno));
    unsigned char h[DBDF_HEADER];
    {
        const ssize_t n = pread(f.fd, h, DBDF_HEADER, 0);
        DB2_CHECK(n == (ssize_t)DBDF_HEADER, DB2_EINVAL, "%s: shorter than a .dbdf header", path);
    }
    uint64_t rows, cols;
    uint32_t brows, bcols;
    memcpy(&rows, h + 2, 8);
    memcpy(&cols, h + 10, 8);
    memcpy(&brows, h + 35, 4);
    memcpy(&bcols, h + 39, 4);
    DB2_CHECK(h[0] == 1, DB2_EUNSUPPORTED, "%s: .dbdf version %d (only 1 is defined)", path, (int)h[0]);
    DB2_CHECK(h[1] == 1, DB2_EUNSUPPORTED, "%s: data type %d is not a DenseMatrix", path, (int)h[1]);
    const int dtype = vt_code_to_dtype(h[18]);
    DB2_CHECK(dtype >= 0, DB2_EUNSUPPORTED, "%s: value type code %d is not implemented on the device", path, (int)h[18]);
    DB2_CHECK(h[43] == 1 && h[44] == h[18], DB2_EUNSUPPORTED, "%s: only one dense block of the matrix' value type",
              path);
    DB2_CHECK(rows <= UINT32_MAX && cols <= UINT32_MAX && brows == (uint32_t)rows && bcols == (uint32_t)cols,
              DB2_EUNSUPPORTED, "%s: the block does not span the matrix", path);
    const size_t es = dtype_size(dtype);
    size_t total = 0;
    DB2_CHECK(!__builtin_mul_overflow((size_t)rows, (size_t)cols, &total) && !__builtin_mul_overflow(total, es, &total),
              DB2_EINVAL, "%s: %llu x %llu values do not fit the address space", path, (unsigned long long)rows,
              (unsigned long long)cols);
    struct stat sb;
    DB2_CHECK(fstat(f.fd, &sb) == 0 && (size_t)sb.st_size >= DBDF_HEADER + total, DB2_EINVAL,
              "%s: %lld x %lld values need %zu bytes after the header, the file has %lld", path, (long long)rows,
              (long long)cols, total, (long long)sb.st_size - (long long)DBDF_HEADER);
    bind_device(ctx);
    db2_matrix *m = nullptr;
    DB2_TRY(db2_matrix_create(ctx, dtype, (int64_t)rows, (int64_t)cols, 0, &m));
    std::unique_ptr<db2_matrix, int (*)(db2_matrix *)> guard(m, db2_matrix_decref);
    if (total > 0) {
        Staging st;
        const size_t chunk = total < STAGE_BYTES ? total : STAGE_BYTES;
        DB2_TRY(st.init(chunk));
        char *dst = static_cast<char *>(m->dev_ptr());
        int b = 0;
        for (size_t off = 0; off < total; off += chunk, b ^= 1) {
            const size_t n = total - off < chunk ? total - off : chunk;
            DB2_CUDA(cudaEventSynchronize(st.ev[b])); // the copy that last used this buffer has left it
            DB2_TRY(read_fully(f.fd, st.buf[b], n, (off_t)(DBDF_HEADER + off), path));
            DB2_CUDA(cudaMemcpyAsync(dst + off, st.buf[b], n, cudaMemcpyHostToDevice, ctx->stream));
            DB2_CUDA(cudaEventRecord(st.ev[b], ctx->stream));
        }
        DB2_CUDA(cudaStreamSynchronize(ctx->stream)); // the staging buffers are released on return
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.h2d_bytes += total;
    }
    *res = guard.release();
    return DB2_OK;
    DB2_API_END
}

int db2_writeDaphne(db2_context *ctx, db2_matrix *m, const char *path) {
    DB2_API_BEGIN
    DB2_CHECK(ctx && m && path, DB2_EINVAL, "null argument");
    DB2_CHECK(m->rows <= (int64_t)UINT32_MAX && m->cols <= (int64_t)UINT32_MAX, DB2_EUNSUPPORTED,
              "a single .dbdf block holds at most 2^32 - 1 rows and columns");
    bind_device(ctx);
    DB2_TRY(ensure_device(m));
    Fd f;
    f.fd = open(path, O_WRONLY | O_CREAT | O_TRUNC, 0644);
    DB2_CHECK(f.fd >= 0, DB2_EINVAL, "cannot create %s: %s", path, strerror(errno));
    unsigned char h[DBDF_HEADER];
    memset(h, 0, sizeof(h));
    const uint64_t rows = (uint64_t)m->rows, cols = (uint64_t)m->cols;
    const uint32_t brows = (uint32_t)rows, bcols = (uint32_t)cols;
    h[0] = 1;
    h[1] = 1;
    memcpy(h + 2, &rows, 8);
    memcpy(h + 10, &cols, 8);
    h[18] = (unsigned char)dtype_to_vt_code(m->dtype);
    memcpy(h + 35, &brows, 4);
    memcpy(h + 39, &bcols, 4);
    h[43] = 1;
    h[44] = h[18];
    DB2_TRY(write_fully(f.fd, h, DBDF_HEADER, path));
    const size_t es = m->esize(), row_bytes = (size_t)m->cols * es, total = (size_t)m->rows * row_bytes;
    if (total > 0) {
        Staging st;
        size_t rows_per = STAGE_BYTES / row_bytes;
        if (rows_per < 1)
            rows_per = 1;
        if (rows_per > (size_t)m->rows)
            rows_per = (size_t)m->rows;
        DB2_TRY(st.init(rows_per * row_bytes));
        const char *src = static_cast<const char *>(m->dev_ptr());
        // copy piece i + 1 to the host while piece i is written to the file
        size_t pending_n = 0;
        int pending_b = -1, b = 0;
        for (size_t r = 0; r < (size_t)m->rows; r += rows_per, b ^= 1) {
            const size_t nr = (size_t)m->rows - r < rows_per ? (size_t)m->rows - r : rows_per;
            DB2_CUDA(cudaMemcpy2DAsync(st.buf[b], row_bytes, src + r * (size_t)m->dev_ld * es, (size_t)m->dev_ld * es,
                                       row_bytes, nr, cudaMemcpyDeviceToHost, ctx->stream));
            DB2_CUDA(cudaEventRecord(st.ev[b], ctx->stream));
            if (pending_b >= 0) {
                DB2_CUDA(cudaEventSynchronize(st.ev[pending_b]));
                DB2_TRY(write_fully(f.fd, st.buf[pending_b], pending_n, path));
            }
            pending_b = b;
            pending_n = nr * row_bytes;
        }
        DB2_CUDA(cudaEventSynchronize(st.ev[pending_b]));
        DB2_TRY(write_fully(f.fd, st.buf[pending_b], pending_n, path));
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->stats.d2h_bytes += total;
    }
    return DB2_OK;
    DB2_API_END
}

} // extern "C"
