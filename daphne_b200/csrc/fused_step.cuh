// The scalar arithmetic of one step of a deferred elementwise chain (fused.cuh), shared by the kernels that evaluate
// chains: the dense passes (fused.cu) and the epilogue of the CSR row aggregation (csr.cu).
#pragma once

#include "fused.cuh"

namespace db2 {

__device__ __forceinline__ bool safe_divisor(double d) {
    const unsigned hi = (unsigned)__double2hiint(d), lo = (unsigned)__double2loint(d);
    const int e = (hi >> 20) & 0x7ff;
    const bool all_ones = ((hi & 0xfffffu) == 0xfffffu) && (lo == 0xffffffffu);
    return e > 923 && e < 1123 && !all_ones; // |d| in (2^-100, 2^100)
}
// reciprocal used by fast_div, or 0.0 = "take the generic division"
__device__ __forceinline__ double div_helper(double d) { return safe_divisor(d) ? __drcp_rn(d) : 0.0; }

__device__ __forceinline__ double fast_div(double a, double d, double y) {
    const int ea = (__double2hiint(a) >> 20) & 0x7ff;
    if (y != 0.0) {
        if (ea > 123 && ea < 1923) { // |a| in (2^-900, 2^900): no intermediate can over- or underflow
            const double q = __dmul_rn(a, y);
            const double r = __fma_rn(-q, d, a);
            return __fma_rn(r, y, q);
        }
        if (a == 0.0)
            return __dmul_rn(a, y); // signed zero
    }
    return __ddiv_rn(a, d);
}

// value (op) operand on GV values; `o` holds the operand, `y` the division helper (only read for FO_DIV)
template <int N>
__device__ __forceinline__ void apply_step(int op, bool reversed, double (&v)[N], const double (&o)[N],
                                           const double (&y)[N]) {
#define DB2_FSTEP(EXPR_FWD, EXPR_REV)                                                                                  \
    if (!reversed) {                                                                                                   \
        _Pragma("unroll") for (int i = 0; i < N; i++) { const double a = v[i], b = o[i]; (void)b; v[i] = (EXPR_FWD); } \
    } else {                                                                                                           \
        _Pragma("unroll") for (int i = 0; i < N; i++) { const double a = v[i], b = o[i]; (void)b; v[i] = (EXPR_REV); } \
    }                                                                                                                  \
    break;
    switch (op) {
    case FO_ADD: DB2_FSTEP(__dadd_rn(a, b), __dadd_rn(b, a))
    case FO_SUB: DB2_FSTEP(__dsub_rn(a, b), __dsub_rn(b, a))
    case FO_MUL: DB2_FSTEP(__dmul_rn(a, b), __dmul_rn(b, a))
    case FO_DIV:
        if (!reversed) {
#pragma unroll
            for (int i = 0; i < N; i++)
                v[i] = fast_div(v[i], o[i], y[i]);
        } else {
#pragma unroll
            for (int i = 0; i < N; i++)
                v[i] = __ddiv_rn(o[i], v[i]);
        }
        break;
    case FO_SQUARE: DB2_FSTEP(__dmul_rn(a, a), __dmul_rn(a, a))
    case FO_EQ: DB2_FSTEP((double)(a == b), (double)(b == a))
    case FO_NEQ: DB2_FSTEP((double)(a != b), (double)(b != a))
    case FO_LT: DB2_FSTEP((double)(a < b), (double)(b < a))
    case FO_LE: DB2_FSTEP((double)(a <= b), (double)(b <= a))
    case FO_GT: DB2_FSTEP((double)(a > b), (double)(b > a))
    case FO_GE: DB2_FSTEP((double)(a >= b), (double)(b >= a))
    case FO_MIN: DB2_FSTEP(((b < a) ? b : a), ((a < b) ? a : b))
    case FO_MAX: DB2_FSTEP(((a < b) ? b : a), ((b < a) ? a : b))
    case FO_AND: DB2_FSTEP((double)((a != 0.0) && (b != 0.0)), (double)((b != 0.0) && (a != 0.0)))
    case FO_OR: DB2_FSTEP((double)((a != 0.0) || (b != 0.0)), (double)((b != 0.0) || (a != 0.0)))
    case FO_NEG: DB2_FSTEP(-a, -a)
    case FO_ABS: DB2_FSTEP(fabs(a), fabs(a))
    case FO_SIGN:
        DB2_FSTEP(((a == 0) ? 0.0 : ((a < 0) ? -1.0 : ((a > 0) ? 1.0 : (double)NAN))),
                  ((a == 0) ? 0.0 : ((a < 0) ? -1.0 : ((a > 0) ? 1.0 : (double)NAN))))
    case FO_FLOOR: DB2_FSTEP(floor(a), floor(a))
    case FO_CEIL: DB2_FSTEP(ceil(a), ceil(a))
    case FO_ROUND: DB2_FSTEP(round(a), round(a))
    case FO_ISNAN: DB2_FSTEP((double)(a != a), (double)(a != a))
    default: break;
    }
#undef DB2_FSTEP
}

} // namespace db2
