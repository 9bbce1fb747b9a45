// Shared host/device helpers for the daphne_b200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <limits>
#include <type_traits>

#include "../../include/daphne_b200.h"

namespace db2 {

// ---------------------------------------------------------------------------
// error reporting: thread-local message + status code
// ---------------------------------------------------------------------------
char *err_buf();  // thread-local buffer of ERR_BUF_LEN bytes
constexpr size_t ERR_BUF_LEN = 1024;

int set_error(int code, const char *fmt, ...);

#define DB2_CUDA(call)                                                                                                \
    do {                                                                                                               \
        cudaError_t e__ = (call);                                                                                      \
        if (e__ != cudaSuccess)                                                                                        \
            return ::db2::set_error(DB2_ECUDA, "%s failed at %s:%d: %s", #call, __FILE__, __LINE__,                     \
                                    cudaGetErrorString(e__));                                                          \
    } while (0)

#define DB2_CHECK(cond, code, ...)                                                                                     \
    do {                                                                                                               \
        if (!(cond))                                                                                                   \
            return ::db2::set_error(code, __VA_ARGS__);                                                                \
    } while (0)

#define DB2_TRY(call)                                                                                                  \
    do {                                                                                                               \
        int rc__ = (call);                                                                                             \
        if (rc__ != DB2_OK)                                                                                            \
            return rc__;                                                                                               \
    } while (0)

// counts every kernel launch of this library (reported by the measurement harness)
extern std::atomic<uint64_t> g_launches;
inline int after_launch(const char *what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return set_error(DB2_ECUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return DB2_OK;
}

// number of SMs of the current device (cached per device)
int sm_count();

// Once-per-DEVICE flag.  cudaFuncSetAttribute applies to the device that is current when it is called, and one process
// may hold contexts on several devices, so the opt-in to large dynamic shared memory is tracked per device (a repeated
// call by two racing threads is harmless).
struct PerDeviceOnce {
    std::atomic<uint64_t> done{0};
    static int dev() {
        int d = 0;
        if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) {
            cudaGetLastError();
            d = 63;
        }
        return d;
    }
    bool need() const { return !((done.load(std::memory_order_acquire) >> dev()) & 1u); }
    void mark() { done.fetch_or(uint64_t(1) << dev(), std::memory_order_release); }
};

inline size_t dtype_size(int dtype) {
    return dtype == DB2_U8 ? 1 : ((dtype == DB2_F32 || dtype == DB2_I32 || dtype == DB2_U32) ? 4 : 8);
}

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

__host__ __device__ inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---------------------------------------------------------------------------
// dtype dispatch
// ---------------------------------------------------------------------------
#define DB2_DISPATCH_DTYPE(dtype, VT, ...)                                                                             \
    switch (dtype) {                                                                                                   \
    case DB2_F64: {                                                                                                    \
        using VT = double;                                                                                             \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    case DB2_F32: {                                                                                                    \
        using VT = float;                                                                                              \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    case DB2_I64: {                                                                                                    \
        using VT = int64_t;                                                                                            \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    default:                                                                                                           \
        return ::db2::set_error(DB2_EUNSUPPORTED, "unsupported value type code %d", (int)(dtype));                     \
    }

// all six value types of the elementwise binary kernels (EwBinaryMat / EwBinaryObjSca)
#define DB2_DISPATCH_DTYPE_EW(dtype, VT, ...)                                                                          \
    switch (dtype) {                                                                                                   \
    case DB2_F64: {                                                                                                    \
        using VT = double;                                                                                             \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    case DB2_F32: {                                                                                                    \
        using VT = float;                                                                                              \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    case DB2_I64: {                                                                                                    \
        using VT = int64_t;                                                                                            \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    case DB2_U64: {                                                                                                    \
        using VT = uint64_t;                                                                                           \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    case DB2_I32: {                                                                                                    \
        using VT = int32_t;                                                                                            \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    case DB2_U32: {                                                                                                    \
        using VT = uint32_t;                                                                                           \
        __VA_ARGS__;                                                                                                   \
    } break;                                                                                                           \
    default:                                                                                                           \
        return ::db2::set_error(DB2_EUNSUPPORTED, "unsupported value type code %d", (int)(dtype));                     \
    }

// ---------------------------------------------------------------------------
// device helpers
// ---------------------------------------------------------------------------

// A 16-byte packet of value type VT (2 x f64/i64 or 4 x f32); global loads and stores of it are 128-bit.
template <typename VT> struct alignas(16) Pack {
    static constexpr int N = 16 / sizeof(VT);
    VT v[N];
};

template <typename VT> __device__ __forceinline__ Pack<VT> ld_pack(const VT *p) {
    return *reinterpret_cast<const Pack<VT> *>(p);
}
// streaming load: data read once, do not keep in L1
template <typename VT> __device__ __forceinline__ Pack<VT> ld_pack_stream(const VT *p) {
    Pack<VT> r;
    const int4 t = __ldcs(reinterpret_cast<const int4 *>(p));
    *reinterpret_cast<int4 *>(&r) = t;
    return r;
}
template <typename VT> __device__ __forceinline__ void st_pack(VT *p, const Pack<VT> &x) {
    *reinterpret_cast<Pack<VT> *>(p) = x;
}
template <typename VT> __device__ __forceinline__ void st_pack_stream(VT *p, const Pack<VT> &x) {
    __stcs(reinterpret_cast<int4 *>(p), *reinterpret_cast<const int4 *>(&x));
}

template <typename VT> __host__ __device__ __forceinline__ VT pos_inf_or_max() {
    if constexpr (std::is_same_v<VT, double>)
        return (VT)INFINITY;
    else if constexpr (std::is_same_v<VT, float>)
        return (VT)INFINITY;
    else if constexpr (std::is_same_v<VT, int64_t>)
        return INT64_MAX;
    else
        return (VT)UINT64_MAX;
}
template <typename VT> __host__ __device__ __forceinline__ VT neg_inf_or_min() {
    if constexpr (std::is_same_v<VT, double>)
        return (VT)-INFINITY;
    else if constexpr (std::is_same_v<VT, float>)
        return (VT)-INFINITY;
    else if constexpr (std::is_same_v<VT, int64_t>)
        return INT64_MIN;
    else
        return (VT)0;
}

template <typename T> __device__ __forceinline__ T shfl_down(T v, int delta, int width = 32) {
    if constexpr (sizeof(T) == 8) {
        long long x;
        memcpy(&x, &v, 8);
        x = __shfl_down_sync(0xffffffffu, x, delta, width);
        T r;
        memcpy(&r, &x, 8);
        return r;
    } else {
        int x;
        memcpy(&x, &v, 4);
        x = __shfl_down_sync(0xffffffffu, x, delta, width);
        T r;
        memcpy(&r, &x, 4);
        return r;
    }
}
template <typename T> __device__ __forceinline__ T shfl_xor(T v, int mask, int width = 32) {
    if constexpr (sizeof(T) == 8) {
        long long x;
        memcpy(&x, &v, 8);
        x = __shfl_xor_sync(0xffffffffu, x, mask, width);
        T r;
        memcpy(&r, &x, 8);
        return r;
    } else {
        int x;
        memcpy(&x, &v, 4);
        x = __shfl_xor_sync(0xffffffffu, x, mask, width);
        T r;
        memcpy(&r, &x, 4);
        return r;
    }
}

inline int next_pow2(int64_t x) {
    int p = 1;
    while (p < x && p < (1 << 30))
        p <<= 1;
    return p;
}

} // namespace db2
